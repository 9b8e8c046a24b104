/*
 * C ABI of the B200 (sm_100a) flash grouped-query attention library  --  libcllo_flash_gqa.so
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless the name says host.
 * All functions are asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 * default stream), act on the CURRENT device, return 0 on success or a negative CLLO_E_* code,
 * and never abort the process or trap on the device.  The library allocates no device memory
 * except where a function's comment says so.
 *
 * Tensors are bf16 (uint16 bit patterns), accumulation is fp32.  head_dim must be 128.
 *
 * Each entry point names the upstream (LiuYiyang-Canton/cuda_llm_ops) interface it stands in for.
 */
#ifndef CLLO_FLASH_GQA_H_
#define CLLO_FLASH_GQA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CLLO_OK 0
#define CLLO_E_BAD_ARG (-1)       /* null / misaligned pointer, non-positive size, Hq % Hkv != 0 */
#define CLLO_E_UNSUPPORTED (-2)   /* head_dim != 128, wrong GPU architecture */
#define CLLO_E_WORKSPACE (-3)     /* workspace missing or too small */
#define CLLO_E_CUDA (-4)          /* a CUDA call failed; see cllo_last_cuda_error() */
#define CLLO_E_DEVICE_TIMEOUT (-6) /* a bounded wait inside a kernel gave up; results are invalid */

/* K/V cache layouts */
#define CLLO_KV_BSHD 0 /* [B, S, Hkv, D]  upstream C++ layout (decode_flash_gqa_kernel.cu:144-148) */
#define CLLO_KV_BHSD 1 /* [B, Hkv, S, D]  upstream Triton layout (decode_flash_gqa_kernel.py:50-53) */

/* May be OR-ed into a decode call's kv_layout: the caller vouches that the arrival counters (the first 4 KB of
 * the workspace) are zero -- it zeroed the workspace once (cudaMemset of all of it is fine) and since then nothing but
 * calls of this library, none of which ended in CLLO_E_DEVICE_TIMEOUT, has written to it.  The call then skips the
 * memset node it would otherwise put in front of the kernel (the kernel leaves the counters zero).  Ignored when
 * num_workers exceeds 1024. */
#define CLLO_WS_COUNTERS_ZERO 0x100

/* Width of one packed partial row: D un-normalised fp32 outputs, then m, then l. */
#define CLLO_PARTIAL_WIDTH(D) ((D) + 2)

int cllo_version(void);
const char* cllo_status_string(int status);
/* cudaError_t value of the most recent failing CUDA call made by this library on this thread. */
int cllo_last_cuda_error(void);
/* Synchronises the current device, returns CLLO_OK or CLLO_E_DEVICE_TIMEOUT if any kernel of this
 * library recorded a timed-out wait since the last call, and clears the record.  detail (host,
 * nullable) receives {code, block, site, aux}. */
int cllo_device_status(int detail[4]);
/* Frees the per-device scratch that LaunchFlashGqaBf16Kernel's compatibility path may have cached.  Call it
 * when no launch of that path is in flight on any thread. */
int cllo_shutdown(void);

/*
 * Single-token GQA decode:  O[b, h, :] = softmax(scale * q[b,h,:] . K[b,:,h/G,:]^T) V[b,:,h/G,:]
 *
 * Stands in for decode_flash_gqa_bf16_kernel + LaunchFlashGqaBf16Kernel
 * (src/cplusplus/FlashGQA/decode_flash_gqa_kernel.cu:119-389, :405-470; declared in
 * include/cplusplus/FlashGQA/decode_flash_gqa_kernel.cuh:28-38) and for the Triton twin
 * launch_decode_flash_gqa_bf16_kernel (src/python/Triton/decode_flash_gqa_kernel.py:137-196).
 * Unlike upstream it accepts any group size G = Hq/Hkv >= 1 and any S >= 1.
 *
 *   q [B,Hq,D]   k,v per kv_layout   o [B,Hq,D] bf16
 *   workspace / workspace_bytes: scratch of at least cllo_gqa_decode_workspace_bytes(...) bytes,
 *       256-byte aligned, contents arbitrary.  The KV range of every (batch, kv head) is cut into equal
 *       shares for `num_workers` persistent thread blocks; shares that cover only part of a head leave
 *       fp32 partials (O, m, l) in the workspace, and the last block to finish a head's share merges them
 *       by log-sum-exp (second pass, same kernel; the call zeroes its arrival counters with a memset node
 *       on `stream` first, unless kv_layout carries CLLO_WS_COUNTERS_ZERO).  Calls that may overlap on the
 *       GPU need a workspace each.
 *   num_workers: 0 = chosen by the library: between 0.7 and 0.87 blocks per SM of the current device,
 *       preferring a count that gives every block whole (batch, kv head) units or equal cuts of them.
 *   Group sizes above 16: the query heads of a group are served in blocks of 16 and each block streams the
 *       group's K/V again, so G = 32 reads K/V twice (no upstream configuration has G > 16).
 *   partial_out (nullable): when given, `o` is ignored and the call writes, for every (b, h), one
 *       packed fp32 row [D+2] = {un-normalised O, m = max scaled score, l = sum exp(score - m)} of
 *       THIS call's KV range.  This is what a KV-position-sharded caller all-gathers and feeds to
 *       cllo_gqa_combine_bf16.
 */
size_t cllo_gqa_decode_workspace_bytes(int B, int S, int Hq, int Hkv, int D, int num_workers);
int cllo_gqa_decode_bf16(const void* q, const void* k, const void* v, float scale, void* o,
                         void* workspace, size_t workspace_bytes,
                         int B, int S, int Hq, int Hkv, int D,
                         int kv_layout, int num_workers, float* partial_out, void* stream);

/*
 * One decode step with the rotary embedding and the KV-cache append folded into the attention kernel.
 * Stands in for the sequence RopeBf16Kernel on the new token's Q and K (src/cplusplus/RoPE/rope_kernel.cu:33-107,
 * hidden = head_dim: interleaved pairs (2i, 2i+1) of each head rotated by position * base^(-2i/D)), a cache append,
 * and decode_flash_gqa_bf16_kernel -- three passes upstream, one kernel here:
 *   q [B,Hq,D] and k_new, v_new [B,Hkv,D]: the new token, un-rotated;
 *   k_cache, v_cache: the caches in kv_layout with a token capacity of S_capacity >= S ([B,S_capacity,Hkv,D] or
 *       [B,Hkv,S_capacity,D]); positions [0, S-1) hold earlier tokens (keys already rotated).  The call writes the
 *       rotated k_new and v_new into position S-1 and attends over positions [0, S);
 *   positions (device, nullable): [B] rotary position of the new token per sequence; NULL = S-1 for all;
 *   everything else as cllo_gqa_decode_bf16.  The query is rotated as it is loaded; it is not written back.
 */
int cllo_gqa_decode_rope_append_bf16(const void* q, const void* k_new, const void* v_new,
                                     void* k_cache, void* v_cache, const int* positions, float rope_base,
                                     float scale, void* o, void* workspace, size_t workspace_bytes,
                                     int B, int S, int S_capacity, int Hq, int Hkv, int D,
                                     int kv_layout, int num_workers, void* stream);

/* How a decode call would be cut up: plan[0] = workers actually launched, plan[1] = KV tiles per
 * (batch, kv head, 16-query-head block), plan[2..3] = total tiles (low, high 32 bits), plan[4] = 1 if some
 * head's share is cut between workers (partials are merged), plan[5] = tokens per tile.  Host-only arithmetic; sm_count <= 0 means "ask the device". */
int cllo_gqa_decode_plan(int B, int S, int Hq, int Hkv, int D, int num_workers, int sm_count, int plan[6]);

/* Upstream's launcher signature without a workspace argument (LaunchFlashGqaBf16Kernel,
 * decode_flash_gqa_kernel.cuh:28-38): K/V in CLLO_KV_BSHD, default stream.  Uses o_intermediate
 * ([B,Hq,D] fp32, upstream's scratch argument) as workspace when it is large enough; otherwise it
 * cudaMallocs one scratch buffer per device on first use and keeps it until cllo_shutdown(). */
int cllo_gqa_decode_bf16_compat(const void* q, const void* k, const void* v, float scale, void* o,
                                float* o_intermediate, int B, int S, int Hq, int Hkv, int D);

/*
 * Decode without any allocation, by the caller or by the library.  (No counterpart upstream: upstream's
 * launcher takes its scratch from the caller.)
 *
 * Some hosts of this library cannot provide a workspace: an inference server that has handed every byte
 * of device memory to its KV-cache pool and forbids plugins to allocate; a latency-critical decode loop
 * that cannot afford the device-wide synchronisation a cudaMalloc/cudaFree implies; a caller that only
 * receives the tensors' pointers.  For them this variant keeps the split-KV partials in a fixed
 * __device__ array inside the library (4 KB + CLLO_NOALLOC_MAX_WORKERS * 16,640 bytes, about 2.5 MiB, resident
 * on every GPU that loads the library until the process exits).  It calls neither cudaMalloc nor
 * cudaFree nor any allocating routine.
 *
 * Same arguments and results as cllo_gqa_decode_bf16 without workspace and partial_out.  Limits:
 *   - num_workers > CLLO_NOALLOC_MAX_WORKERS is refused with CLLO_E_WORKSPACE (the partials would not
 *     fit); num_workers == 0 uses min(the library's own choice, CLLO_NOALLOC_MAX_WORKERS).  B, S and the head counts are
 *     not limited by the scratch: its size depends on the number of workers only.  On a GPU with so many
 *     SMs that the library would choose more than CLLO_NOALLOC_MAX_WORKERS blocks (about 185 SMs and up) the
 *     default is capped and the call is slower than cllo_gqa_decode_bf16 with a workspace.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current) and remembers it; make that first call outside any stream capture.
 *   - All calls on one device share the one array and it keeps the previous call's contents.  The only
 *     part that has to start at zero, the arrival counters, is cleared by a memset on `stream` at the
 *     start of every call (every partial that is merged was written earlier in the same call); but two
 *     calls that overlap on the GPU (different streams) race on the array: serialise them.
 */
#define CLLO_NOALLOC_MAX_WORKERS 160
int cllo_gqa_decode_bf16_noalloc(const void* q, const void* k, const void* v, float scale, void* o,
                                 int B, int S, int Hq, int Hkv, int D,
                                 int kv_layout, int num_workers, void* stream);

/*
 * Log-sum-exp merge of nsplit packed partials:  partials [nsplit][rows][D+2] fp32 -> o [rows][D] bf16.
 * rows = B*Hq.  Splits with l == 0 are ignored.  Same (m, l) monoid as the running update in
 * decode_flash_gqa_kernel.cu:353-371 and TileMaxSumReduce (src/cplusplus/Softmax/softmax_kernel.cu:21-34).
 * Upstream has no multi-GPU path; this is the second pass of the split-KV decode exposed for callers
 * that shard one sequence's KV cache by position across GPUs.
 */
int cllo_gqa_combine_bf16(const float* partials, int nsplit, void* o, long long rows, int D, void* stream);

/*
 * One sequence (or batch) whose KV cache is sharded by POSITION over the GPUs of one node.  Upstream has no
 * multi-GPU code; these entry points are the exchange step such a caller needs, over peer memory (plain peer
 * loads/stores and flag words; no library collective, no multicast).
 *
 * Buffers, per rank, in memory that every rank has mapped (CUDA IPC, symmetric memory, ...), zeroed once before
 * the first step:
 *   gather  cllo_gqa_shard_gather_bytes(world, B, Hq, D) bytes: [2][world][B*Hq][D+2] fp32
 *   flags   cllo_gqa_shard_flag_bytes(world) bytes: [world][CLLO_SHARD_MAX_UNITS] uint32 + one counter word
 * peer_gather / peer_flags are HOST arrays of `world` device pointers, entry p = rank p's buffer as mapped into
 * THIS process; entry `rank` is the local one.  B * Hkv * ceil((Hq/Hkv)/16) must not exceed CLLO_SHARD_MAX_UNITS.
 *
 *   epoch: 1, 2, 3, ... the same on every rank for the same step; or 0 on every rank and every step, in which case
 *       the kernels derive the step from a completion counter in the flag buffer (a call sequence that never changes its arguments,
 *       e.g. one replayed from a CUDA graph).  Every rank must make one call per step.  A rank that is late by more
 *       than the wait limit (about a second unless changed by cllo_set_exchange_wait_limit) makes the others' wait
 *       expire: their output rows are filled with NaN and cllo_device_status() reports CLLO_E_DEVICE_TIMEOUT.
 *
 * cllo_gqa_decode_sharded_bf16: the whole step in one kernel.  Split-KV decode of this rank's S_local positions
 *   (arguments as cllo_gqa_decode_bf16); as the last piece of each (batch, kv head) arrives, that head's merged
 *   (O, m, l) rows are stored into every peer's gather buffer, the peers' rows are awaited and the final bf16
 *   o [B,Hq,D] is written -- on every rank.  The exchange of early heads overlaps the decode of late ones.
 * cllo_gqa_exchange_combine_bf16: the same exchange for a packed partial that already exists
 *   (local_partial [B*Hq][D+2], e.g. partial_out of cllo_gqa_decode_bf16, or l = 0 rows from a rank whose share of
 *   the sequence is empty).  Ranks may mix the two entry points within a step.
 * cllo_set_exchange_wait_limit: upper bound of one flag wait in SM clock cycles (<= 0 restores the default);
 *   applies to later launches of either entry point.
 */
#define CLLO_MAX_PEERS 16
#define CLLO_SHARD_MAX_UNITS 256
size_t cllo_gqa_shard_gather_bytes(int world, int B, int Hq, int D);
size_t cllo_gqa_shard_flag_bytes(int world);
int cllo_set_exchange_wait_limit(long long sm_cycles);
int cllo_gqa_decode_sharded_bf16(const void* q, const void* k, const void* v, float scale, void* o,
                                 void* workspace, size_t workspace_bytes,
                                 int B, int S_local, int Hq, int Hkv, int D,
                                 int kv_layout, int num_workers,
                                 void* const* peer_gather, void* const* peer_flags, int rank, int world,
                                 unsigned epoch, void* stream);
int cllo_gqa_exchange_combine_bf16(const float* local_partial, void* const* peer_gather, void* const* peer_flags,
                                   int rank, int world, unsigned epoch, void* o,
                                   int B, int Hq, int Hkv, int D, void* stream);

/*
 * Multi-token (prefill) GQA forward:  O = softmax(mask(scale * Q K^T)) V,  lse = m + log(l).
 * Stands in for flash_gqa_forward_bf16_kernel + launch_flash_gqa_forward_bf16_kernel
 * (src/python/Triton/flash_gqa_kernel.py:16-138, :185-338).  Layout as upstream:
 *   q,o [B,Hq,Sq,D]   k,v [B,Hkv,Skv,D]   lse [B,Hq,Sq] fp32 (nullable)
 * causal != 0 keeps kv <= q (top-left aligned, flash_gqa_kernel.py:104,114).
 * scale must be finite and non-zero (CLLO_E_BAD_ARG otherwise; negative is fine) -- here and in the sliding-window
 * and MLA-shaped forwards below.
 */
int cllo_gqa_prefill_fwd_bf16(const void* q, const void* k, const void* v, float scale, int causal,
                              void* o, float* lse,
                              int B, int Sq, int Skv, int Hq, int Hkv, int D, void* stream);

/*
 * The same forward with a caller-owned workspace (no upstream counterpart: upstream's launcher has no scratch).
 * A chunk of query tokens against a long cache -- non-causal, few query rows, few (batch, kv head) pairs -- gives
 * too few thread blocks to fill the GPU; with a workspace of cllo_gqa_prefill_workspace_bytes(...) bytes (16-byte
 * aligned, contents arbitrary) the call cuts the kv range into shares for different blocks and merges the shares'
 * partials (flash-decoding; the merge is the combine kernel of cllo_gqa_combine_bf16).  The size query returns 0 when
 * the shape would not be cut; workspace may then be NULL.  Results are those of cllo_gqa_prefill_fwd_bf16 up to
 * fp32 summation order.
 */
size_t cllo_gqa_prefill_workspace_bytes(int B, int Sq, int Skv, int Hq, int Hkv, int causal);
int cllo_gqa_prefill_fwd_ws_bf16(const void* q, const void* k, const void* v, float scale, int causal,
                                 void* o, float* lse, void* workspace, size_t workspace_bytes,
                                 int B, int Sq, int Skv, int Hq, int Hkv, int D, void* stream);

/*
 * Sliding-window attention forward with a sink term (the mask variant of the prefill forward):
 * a query at position i sees kv positions [i - (window_size - 1), i]; the softmax denominator of head h
 * is sum(exp(s - m)) + sink_value[h] * exp(-m); rows without any visible key give zeros and
 * lse = log(max(sink, 1e-9)).  Stands in for flash_swa_forward_bf16_kernel +
 * launch_flash_swa_forward_bf16_kernel (src/python/Triton/SWA/flash_swa_kernel.py:15-160, :186-330).
 * Same tensors and layouts as cllo_gqa_prefill_fwd_bf16; sink_value is fp32 [Hq] on the device.
 */
int cllo_swa_prefill_fwd_bf16(const void* q, const void* k, const void* v, float scale, int window_size,
                              const float* sink_value, void* o, float* lse,
                              int B, int Sq, int Skv, int Hq, int Hkv, int D, void* stream);

/*
 * MLA-shaped attention forward (Q and K heads wider than V heads): O = softmax(mask(scale * Q K^T)) V, lse = m + log(l).
 * Stands in for flash_mla_forward_bf16_kernel + launch_flash_mla_forward_bf16_kernel
 * (src/python/Triton/flash_mla_kernel.py:16-268, :315-508).  Layout as upstream:
 *   q [B,Hq,Sq,Dqk]   k [B,Hkv,Skv,Dqk]   v [B,Hkv,Skv,Dv]   o [B,Hq,Sq,Dv]   lse [B,Hq,Sq] fp32 (nullable)
 * causal != 0 keeps kv <= q (top-left aligned).  Dqk = 192 and Dv = 128 (upstream's benchmark shape) only.
 */
int cllo_mla_prefill_fwd_bf16(const void* q, const void* k, const void* v, float scale, int causal,
                              void* o, float* lse,
                              int B, int Sq, int Skv, int Hq, int Hkv, int Dqk, int Dv, void* stream);

/*
 * Sparse-index GQA forward: every query token attends to its own list of kv tokens, shared by the query heads
 * of a group.  Stands in for flash_sgqa_forward_bf16_kernel + launch_flash_sgqa_forward_bf16_kernel
 * (src/python/Triton/SparseGQA/flash_sgqa_kernel.py:15-138, :202-396).
 *   q,o [B,Hq,Sq,D]   k,v [B,Hkv,Skv,D]   lse [B,Hq,Sq] fp32 (nullable)
 *   sparse_kv_indices int32 [B,Hkv,Sq,num_sparse_kv] on the device
 * An entry counts when 0 <= index < Skv and, with causal != 0, index <= the query position; every other entry
 * (upstream pads with -1) is ignored, repeated entries count as often as they appear, a row whose list holds no
 * valid entry gives zeros and lse = -inf.  D = 128 and Hq / Hkv <= 16.
 */
int cllo_sgqa_prefill_fwd_bf16(const void* q, const void* k, const void* v, const int* sparse_kv_indices,
                               int num_sparse_kv, float scale, int causal, void* o, float* lse,
                               int B, int Sq, int Skv, int Hq, int Hkv, int D, void* stream);

/*
 * GQA attention backward: grad_q, grad_k, grad_v from grad_o, given the forward's inputs, output and lse.
 * Stands in for flash_gqa_backward_bf16_kernel + rowwise_dot_o_grad_o_kernel +
 * launch_flash_gqa_backward_bf16_kernel (src/python/Triton/flash_gqa_backward_kernel.py:159-310, :16-48,
 * :312-478).  Layouts as the forward: q, o, grad_o, grad_q [B,Hq,Sq,D]; k, v, grad_k, grad_v [B,Hkv,Skv,D]
 * bf16; lse [B,Hq,Sq] fp32 as written by cllo_gqa_prefill_fwd_bf16.  grad_k / grad_v are summed over the
 * query heads of each group in fp32 and rounded once; no atomics, results are deterministic.
 * workspace: cllo_gqa_bwd_workspace_bytes(...) bytes, 256-byte aligned: one fp32 per query row, plus -- when
 * there are too few (kv head, kv tile) pairs to fill the GPU and the query heads of a group are therefore
 * divided among several blocks -- fp32 partial grad_k / grad_v per head split (summed in a fixed order).
 */
size_t cllo_gqa_bwd_workspace_bytes(int B, int Sq, int Skv, int Hq, int Hkv);
int cllo_gqa_bwd_bf16(const void* q, const void* k, const void* v, const void* o, const float* lse,
                      const void* grad_o, float scale, int causal,
                      void* grad_q, void* grad_k, void* grad_v,
                      void* workspace, size_t workspace_bytes,
                      int B, int Sq, int Skv, int Hq, int Hkv, int D, void* stream);

/*
 * Backward of the sliding-window + sink forward: same kernels and workspace as cllo_gqa_bwd_bf16 with the
 * window mask; the sink reaches the gradients only through lse (it has no value vector), so it is not an
 * argument.  Stands in for flash_swa_backward_bf16_kernel + launch_flash_swa_backward_bf16_kernel
 * (src/python/Triton/SWA/flash_swa_backward_kernel.py).
 */
int cllo_swa_bwd_bf16(const void* q, const void* k, const void* v, const void* o, const float* lse,
                      const void* grad_o, float scale, int window_size,
                      void* grad_q, void* grad_k, void* grad_v,
                      void* workspace, size_t workspace_bytes,
                      int B, int Sq, int Skv, int Hq, int Hkv, int D, void* stream);

/*
 * Rotary position embedding (the step before attention): input/output [B, S, hidden] bf16, interleaved pairs
 * (2i, 2i+1) rotated by token * base^(-2i/hidden); in place allowed.  Stands in for RopeBf16Kernel +
 * LaunchRopeBf16Kernel (src/cplusplus/RoPE/rope_kernel.cu:33-107, :117-147; declared in
 * include/cplusplus/RoPE/rope_kernel.cuh:22).  hidden must be a multiple of 8 and at most 1024.
 */
int cllo_rope_bf16(const void* input, void* output, int B, int S, int hidden, float base, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CLLO_FLASH_GQA_H_ */
