// C ABI of libcllo_flash_gqa.so (see include/cllo_flash_gqa.h).  Single translation unit: the kernels
// share one device status word.
#include "gqa_decode.cuh"
#include "gqa_prefill.cuh"
#include "gqa_exchange.cuh"
#include "gqa_backward.cuh"
#include "rope.cuh"
#include "sgqa_prefill.cuh"
#include "mla_prefill.cuh"

#include <cstdio>
#include <cstring>

using namespace cllo;

// Scratch for cllo_gqa_decode_bf16_noalloc: room for the split-KV partials (and arrival counters) of up to
// CLLO_NOALLOC_MAX_WORKERS persistent blocks.  It lives in the library image, so every GPU that loads
// the library carries these ~2.5 MiB until the process exits.  Host code must never hand this NAME to
// a kernel: on the host it is only a stand-in, the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[
    decode::kSlotOffsetBytes + static_cast<size_t>(CLLO_NOALLOC_MAX_WORKERS) * 2 * decode::kSlotFloats * sizeof(float)];
static void* g_noalloc_ptr[kMaxDevices];  // device address of the array, looked up once per device
static std::mutex g_noalloc_mutex;

extern "C" {

int cllo_version(void) { return 100; }

const char* cllo_status_string(int status) {
    switch (status) {
        case CLLO_OK: return "ok";
        case CLLO_E_BAD_ARG: return "bad argument";
        case CLLO_E_UNSUPPORTED: return "unsupported shape or device";
        case CLLO_E_WORKSPACE: return "workspace missing or too small";
        case CLLO_E_CUDA: return "CUDA call failed";
        case CLLO_E_DEVICE_TIMEOUT: return "a bounded wait inside a kernel timed out";
        default: return "unknown status";
    }
}

int cllo_last_cuda_error(void) { return t_last_cuda_error; }

int cllo_device_status(int detail[4]) {
    int host[4] = {0, 0, 0, 0};
    CLLO_CUDA_TRY(cudaDeviceSynchronize());
    CLLO_CUDA_TRY(cudaMemcpyFromSymbol(host, g_status, sizeof(host)));
    if (host[0] != 0) {
        const int zero[4] = {0, 0, 0, 0};
        CLLO_CUDA_TRY(cudaMemcpyToSymbol(g_status, zero, sizeof(zero)));
    }
    if (detail) std::memcpy(detail, host, sizeof(host));
    return host[0] == 0 ? CLLO_OK : CLLO_E_DEVICE_TIMEOUT;
}

int cllo_shutdown(void) {
    int restore = 0;
    if (cudaGetDevice(&restore) != cudaSuccess) {
        (void)cudaGetLastError();
        return CLLO_OK;  // no device, nothing cached
    }
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    for (int d = 0; d < kMaxDevices; ++d) {
        if (g_dev[d].legacy_ws || !g_dev[d].retired_ws.empty()) {
            if (cudaSetDevice(d) == cudaSuccess) {
                (void)cudaFree(g_dev[d].legacy_ws);
                for (void* old : g_dev[d].retired_ws) (void)cudaFree(old);
            }
            g_dev[d].retired_ws.clear();
            g_dev[d].legacy_ws = nullptr;
            g_dev[d].legacy_ws_bytes = 0;
        }
    }
    (void)cudaSetDevice(restore);
    (void)cudaGetLastError();
    return CLLO_OK;
}

size_t cllo_gqa_decode_workspace_bytes(int B, int S, int Hq, int Hkv, int D, int num_workers) {
    int sm = 0;
    if (num_workers <= 0) {
        DeviceInfo* di = nullptr;
        if (current_device_info(&di) == CLLO_OK) sm = di->sm_count;
        if (sm <= 0) sm = 256;  // no device visible: an upper bound for any current part
    }
    decode::Plan plan;
    if (decode::make_plan(B, S, Hq, Hkv, D, num_workers, sm, &plan) != CLLO_OK) return 0;
    return plan.ws_bytes;
}

int cllo_gqa_decode_plan(int B, int S, int Hq, int Hkv, int D, int num_workers, int sm_count, int out[6]) {
    if (!out) return CLLO_E_BAD_ARG;
    if (sm_count <= 0 && num_workers <= 0) {
        DeviceInfo* di = nullptr;
        int rc = current_device_info(&di);
        if (rc != CLLO_OK) return rc;
        sm_count = di->sm_count;
    }
    decode::Plan plan;
    int rc = decode::make_plan(B, S, Hq, Hkv, D, num_workers, sm_count, &plan);
    if (rc != CLLO_OK) return rc;
    out[0] = plan.prm.W;
    out[1] = plan.prm.n_t;
    out[2] = static_cast<int>(plan.prm.T & 0xffffffffLL);
    out[3] = static_cast<int>(plan.prm.T >> 32);
    out[4] = plan.needs_merge ? 1 : 0;
    out[5] = decode::kTok;
    return CLLO_OK;
}

// Tensor maps of the most recent K/V cache seen by this host thread: a decode loop calls with the same cache
// step after step, and encoding two maps costs about as much host time as the launch itself.
struct KvMapCache {
    const void* k = nullptr;
    const void* v = nullptr;
    int B = 0, S = 0, S_cap = 0, Hkv = 0, layout = -1;
    CUtensorMap tm_k, tm_v;
};
static thread_local KvMapCache t_kv_maps;

static int decode_launch(const void* q, const void* k, const void* v, float scale, void* o, void* workspace,
                         size_t workspace_bytes, int B, int S, int Hq, int Hkv, int D, int kv_layout, int num_workers,
                         float* partial_out, const shard::Params* sp, cudaStream_t st,
                         decode::RopeParams* rp = nullptr, int S_cap = 0) {
    if (!q || !k || !v || (!o && !partial_out)) return CLLO_E_BAD_ARG;
    if (S_cap == 0) S_cap = S;
    if (S_cap < S) return CLLO_E_BAD_ARG;
    const bool counters_zero = (kv_layout & CLLO_WS_COUNTERS_ZERO) != 0;
    kv_layout &= ~CLLO_WS_COUNTERS_ZERO;
    if (kv_layout != CLLO_KV_BSHD && kv_layout != CLLO_KV_BHSD) return CLLO_E_BAD_ARG;
    if (!aligned_to(q, 16) || !aligned_to(k, 16) || !aligned_to(v, 16) || (o && !aligned_to(o, 16)) ||
        (partial_out && !aligned_to(partial_out, 8)))
        return CLLO_E_BAD_ARG;
    DeviceInfo* di = nullptr;
    int rc = current_device_info(&di);
    if (rc != CLLO_OK) return rc;
    if (di->cc_major != 10) return CLLO_E_UNSUPPORTED;
    decode::Plan plan;
    rc = decode::make_plan(B, S, Hq, Hkv, D, num_workers, di->sm_count, &plan);
    if (rc != CLLO_OK) return rc;
    if (!workspace || workspace_bytes < plan.ws_bytes || !aligned_to(workspace, 256)) return CLLO_E_WORKSPACE;

    decode::Params& p = plan.prm;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.o = static_cast<__nv_bfloat16*>(o);
    p.partial_out = partial_out;
    p.ws = reinterpret_cast<float*>(static_cast<char*>(workspace) + plan.slot_offset);
    p.counters = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + plan.counter_offset);
    p.scale_log2 = scale * decode::kLog2e;
    p.kv_layout = kv_layout;

    KvMapCache& mc = t_kv_maps;
    if (mc.k != k || mc.v != v || mc.B != B || mc.S != S || mc.S_cap != S_cap || mc.Hkv != Hkv ||
        mc.layout != kv_layout) {
        mc.layout = -1;
        rc = decode::encode_kv_map(&mc.tm_k, k, B, S, Hkv, kv_layout, S_cap);
        if (rc != CLLO_OK) return rc;
        rc = decode::encode_kv_map(&mc.tm_v, v, B, S, Hkv, kv_layout, S_cap);
        if (rc != CLLO_OK) return rc;
        mc.k = k;
        mc.v = v;
        mc.B = B;
        mc.S = S;
        mc.S_cap = S_cap;
        mc.Hkv = Hkv;
        mc.layout = kv_layout;
    }

    if (!di->decode_attr_set) {
        CLLO_CUDA_TRY(cudaFuncSetAttribute(decode::decode_splitkv_kernel<false, false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, decode::kSmemBytes));
        CLLO_CUDA_TRY(cudaFuncSetAttribute(decode::decode_splitkv_kernel<true, false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, decode::kSmemBytes));
        CLLO_CUDA_TRY(cudaFuncSetAttribute(decode::decode_splitkv_kernel<false, true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, decode::kSmemBytes));
        di->decode_attr_set = true;
    }
    // arrival counters of the units that a worker boundary cuts: zero at kernel start.  The kernel leaves them
    // zero, so a caller that keeps a workspace for this library alone can vouch for them and save the memset node.
    if (plan.needs_merge && !(counters_zero && plan.counters_fixed))
        CLLO_CUDA_TRY(cudaMemsetAsync(static_cast<char*>(workspace) + plan.counter_offset, 0, plan.counter_bytes, st));
    static const shard::Params no_shard = {};
    static const decode::RopeParams no_rope = {};
    if (rp) {
        const long long row = decode::kD;
        rp->tok_stride = kv_layout == CLLO_KV_BSHD ? row * Hkv : row;
        rp->head_stride = kv_layout == CLLO_KV_BSHD ? row : row * S_cap;
        rp->batch_stride = row * S_cap * Hkv;
        decode::decode_splitkv_kernel<false, true><<<p.W, decode::kThreads, decode::kSmemBytes, st>>>(mc.tm_k, mc.tm_v, p,
                                                                                                      no_shard, *rp);
    } else if (sp) {
        decode::decode_splitkv_kernel<true, false><<<p.W, decode::kThreads, decode::kSmemBytes, st>>>(mc.tm_k, mc.tm_v, p,
                                                                                                      *sp, no_rope);
    } else {
        decode::decode_splitkv_kernel<false, false><<<p.W, decode::kThreads, decode::kSmemBytes, st>>>(mc.tm_k, mc.tm_v,
                                                                                                       p, no_shard, no_rope);
    }
    CLLO_CUDA_TRY(cudaGetLastError());
    return CLLO_OK;
}

int cllo_gqa_decode_bf16(const void* q, const void* k, const void* v, float scale, void* o, void* workspace,
                         size_t workspace_bytes, int B, int S, int Hq, int Hkv, int D, int kv_layout,
                         int num_workers, float* partial_out, void* stream) {
    return decode_launch(q, k, v, scale, o, workspace, workspace_bytes, B, S, Hq, Hkv, D, kv_layout, num_workers,
                         partial_out, nullptr, static_cast<cudaStream_t>(stream));
}

int cllo_gqa_decode_sharded_bf16(const void* q, const void* k, const void* v, float scale, void* o, void* workspace,
                                 size_t workspace_bytes, int B, int S_local, int Hq, int Hkv, int D, int kv_layout,
                                 int num_workers, void* const* peer_gather, void* const* peer_flags, int rank,
                                 int world, unsigned epoch, void* stream) {
    if (!o) return CLLO_E_BAD_ARG;
    shard::Params sp;
    int rc = exchange::fill_shard_params(&sp, peer_gather, peer_flags, rank, world, epoch, B, Hq, Hkv);
    if (rc != CLLO_OK) return rc;
    return decode_launch(q, k, v, scale, o, workspace, workspace_bytes, B, S_local, Hq, Hkv, D, kv_layout,
                         num_workers, nullptr, &sp, static_cast<cudaStream_t>(stream));
}

int cllo_gqa_decode_rope_append_bf16(const void* q, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                                     const int* positions, float rope_base, float scale, void* o, void* workspace,
                                     size_t workspace_bytes, int B, int S, int S_capacity, int Hq, int Hkv, int D,
                                     int kv_layout, int num_workers, void* stream) {
    if (!k_new || !v_new || !o) return CLLO_E_BAD_ARG;
    if (!aligned_to(k_new, 8) || !aligned_to(v_new, 8)) return CLLO_E_BAD_ARG;
    if (!(rope_base > 0.f) || D != decode::kD) return D != decode::kD ? CLLO_E_UNSUPPORTED : CLLO_E_BAD_ARG;
    decode::RopeParams rp = {};
    rp.k_new = static_cast<const __nv_bfloat16*>(k_new);
    rp.v_new = static_cast<const __nv_bfloat16*>(v_new);
    rp.k_cache = static_cast<__nv_bfloat16*>(k_cache);
    rp.v_cache = static_cast<__nv_bfloat16*>(v_cache);
    rp.positions = positions;
    // the inverse frequencies come from the host's powf, as in cllo_rope_bf16 with hidden = head_dim
    const float inv_d = 1.0f / static_cast<float>(decode::kD);
    for (int i = 0; i < decode::kD / 2; ++i) rp.inv_freq[i] = std::pow(rope_base, -2.0f * static_cast<float>(i) * inv_d);
    return decode_launch(q, k_cache, v_cache, scale, o, workspace, workspace_bytes, B, S, Hq, Hkv, D, kv_layout,
                         num_workers, nullptr, nullptr, static_cast<cudaStream_t>(stream), &rp, S_capacity);
}

size_t cllo_gqa_shard_gather_bytes(int world, int B, int Hq, int D) {
    if (world < 1 || world > CLLO_MAX_PEERS || B <= 0 || Hq <= 0 || D != shard::kD) return 0;
    return static_cast<size_t>(2) * world * B * Hq * shard::kPW * sizeof(float);
}

size_t cllo_gqa_shard_flag_bytes(int world) {
    if (world < 1 || world > CLLO_MAX_PEERS) return 0;
    return (static_cast<size_t>(world) * shard::kMaxUnits + 1) * sizeof(unsigned);
}

int cllo_set_exchange_wait_limit(long long sm_cycles) {
    exchange::g_wait_limit.store(sm_cycles > 0 ? sm_cycles : kWaitLimitCycles);
    return CLLO_OK;
}

int cllo_gqa_combine_bf16(const float* partials, int nsplit, void* o, long long rows, int D, void* stream) {
    if (!partials || !o || nsplit <= 0 || rows <= 0) return CLLO_E_BAD_ARG;
    if (D != decode::kD) return CLLO_E_UNSUPPORTED;
    if (rows > 0x7fffffffLL) return CLLO_E_UNSUPPORTED;
    decode::combine_rows_kernel<<<static_cast<unsigned>((rows + decode::kCombineRows - 1) / decode::kCombineRows),
                                  decode::kCombineRows * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        partials, nsplit, rows, static_cast<__nv_bfloat16*>(o), nullptr);
    CLLO_CUDA_TRY(cudaGetLastError());
    return CLLO_OK;
}

int cllo_gqa_exchange_combine_bf16(const float* local_partial, void* const* peer_gather, void* const* peer_flags,
                                   int rank, int world, unsigned epoch, void* o, int B, int Hq, int Hkv, int D,
                                   void* stream) {
    return exchange::launch(local_partial, peer_gather, peer_flags, rank, world, epoch, o, B, Hq, Hkv, D,
                            static_cast<cudaStream_t>(stream));
}

// The forward with an optional workspace.  A chunk of query tokens against a long cache (non-causal, fewer than 256
// rows per head) runs on the two-tile kernel with the heads of a group as extra rows, and -- given a workspace -- with
// the kv range cut into shares for different blocks when the blocks would otherwise not fill the GPU.
static int prefill_dispatch(const void* q, const void* k, const void* v, float scale, int causal, void* o, float* lse,
                            void* workspace, size_t workspace_bytes, int B, int Sq, int Skv, int Hq, int Hkv, int D,
                            cudaStream_t stream) {
    if (D == 128 && B > 0 && Sq > 0 && Skv > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && !causal) {
        DeviceInfo* di = nullptr;
        if (current_device_info(&di) == CLLO_OK) {
            prefill::Layout L = prefill::choose_layout(B, Sq, Skv, Hq, Hkv, causal, 0, nullptr, di->sm_count,
                                                       workspace != nullptr);
            if (L.n_split > 1 && workspace_bytes < L.ws_bytes)
                L = prefill::choose_layout(B, Sq, Skv, Hq, Hkv, causal, 0, nullptr, di->sm_count, false);
            const long long blocks = static_cast<long long>(B) * L.Hq_eff * ((L.Sq_eff + 255) / 256) * L.n_split;
            // worth it when the kv range is shared out, or when the merged rows alone give the GPU enough blocks
            if (L.n_split > 1 || (L.merged && blocks >= di->sm_count))
                return prefill::launch(q, k, v, scale, causal, 0, nullptr, o, lse, B, Sq, Skv, Hq, Hkv, D, stream, &L,
                                       workspace);
        }
    }
    // all query rows in one 128-row tile (chunked prefill, a few decode tokens): the one-tile kernel, which does not
    // spend half its work on an empty second tile
    if (D == 128 && Sq > 0 && Sq <= 128)
        return mla::launch(q, k, v, scale, causal, o, lse, B, Sq, Skv, Hq, Hkv, D, D, stream);
    return prefill::launch(q, k, v, scale, causal, 0, nullptr, o, lse, B, Sq, Skv, Hq, Hkv, D, stream);
}

int cllo_gqa_prefill_fwd_bf16(const void* q, const void* k, const void* v, float scale, int causal, void* o,
                              float* lse, int B, int Sq, int Skv, int Hq, int Hkv, int D, void* stream) {
    return prefill_dispatch(q, k, v, scale, causal, o, lse, nullptr, 0, B, Sq, Skv, Hq, Hkv, D,
                            static_cast<cudaStream_t>(stream));
}

size_t cllo_gqa_prefill_workspace_bytes(int B, int Sq, int Skv, int Hq, int Hkv, int causal) {
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return 0;
    int sm = 0;
    DeviceInfo* di = nullptr;
    if (current_device_info(&di) == CLLO_OK) sm = di->sm_count;
    if (sm <= 0) sm = 256;  // no device visible: the largest cut any current part would ask for
    return prefill::choose_layout(B, Sq, Skv, Hq, Hkv, causal, 0, nullptr, sm, true).ws_bytes;
}

int cllo_gqa_prefill_fwd_ws_bf16(const void* q, const void* k, const void* v, float scale, int causal, void* o,
                                 float* lse, void* workspace, size_t workspace_bytes, int B, int Sq, int Skv, int Hq,
                                 int Hkv, int D, void* stream) {
    return prefill_dispatch(q, k, v, scale, causal, o, lse, workspace, workspace_bytes, B, Sq, Skv, Hq, Hkv, D,
                            static_cast<cudaStream_t>(stream));
}

int cllo_rope_bf16(const void* input, void* output, int B, int S, int hidden, float base, void* stream) {
    return rope::launch(input, output, B, S, hidden, base, static_cast<cudaStream_t>(stream));
}

size_t cllo_gqa_bwd_workspace_bytes(int B, int Sq, int Skv, int Hq, int Hkv) {
    int sm = 1 << 20;  // no device visible: size for the finest head split
    DeviceInfo* di = nullptr;
    if (current_device_info(&di) == CLLO_OK && di->sm_count > 0) sm = di->sm_count;
    return backward::workspace_bytes(B, Sq, Skv, Hq, Hkv, sm);
}

int cllo_gqa_bwd_bf16(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* grad_o,
                      float scale, int causal, void* grad_q, void* grad_k, void* grad_v, void* workspace,
                      size_t workspace_bytes, int B, int Sq, int Skv, int Hq, int Hkv, int D, void* stream) {
    return backward::launch(q, k, v, o, lse, grad_o, scale, causal, 0, grad_q, grad_k, grad_v, workspace, workspace_bytes,
                            B, Sq, Skv, Hq, Hkv, D, static_cast<cudaStream_t>(stream));
}

int cllo_swa_bwd_bf16(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* grad_o,
                      float scale, int window_size, void* grad_q, void* grad_k, void* grad_v, void* workspace,
                      size_t workspace_bytes, int B, int Sq, int Skv, int Hq, int Hkv, int D, void* stream) {
    if (window_size <= 0) return CLLO_E_BAD_ARG;
    return backward::launch(q, k, v, o, lse, grad_o, scale, 1, window_size, grad_q, grad_k, grad_v, workspace,
                            workspace_bytes, B, Sq, Skv, Hq, Hkv, D, static_cast<cudaStream_t>(stream));
}

int cllo_swa_prefill_fwd_bf16(const void* q, const void* k, const void* v, float scale, int window_size,
                              const float* sink_value, void* o, float* lse, int B, int Sq, int Skv, int Hq, int Hkv,
                              int D, void* stream) {
    if (window_size <= 0 || !sink_value) return CLLO_E_BAD_ARG;
    return prefill::launch(q, k, v, scale, 1, window_size, sink_value, o, lse, B, Sq, Skv, Hq, Hkv, D,
                           static_cast<cudaStream_t>(stream));
}

int cllo_mla_prefill_fwd_bf16(const void* q, const void* k, const void* v, float scale, int causal, void* o, float* lse,
                              int B, int Sq, int Skv, int Hq, int Hkv, int Dqk, int Dv, void* stream) {
    return mla::launch(q, k, v, scale, causal, o, lse, B, Sq, Skv, Hq, Hkv, Dqk, Dv, static_cast<cudaStream_t>(stream));
}

int cllo_sgqa_prefill_fwd_bf16(const void* q, const void* k, const void* v, const int* sparse_kv_indices,
                               int num_sparse_kv, float scale, int causal, void* o, float* lse, int B, int Sq, int Skv,
                               int Hq, int Hkv, int D, void* stream) {
    return sgqa::launch(q, k, v, sparse_kv_indices, num_sparse_kv, scale, causal, o, lse, B, Sq, Skv, Hq, Hkv, D,
                        static_cast<cudaStream_t>(stream));
}

// Decode for callers that may not allocate device memory: the partials go to the fixed array above.
int cllo_gqa_decode_bf16_noalloc(const void* q, const void* k, const void* v, float scale, void* o, int B, int S,
                                 int Hq, int Hkv, int D, int kv_layout, int num_workers, void* stream) {
    if (num_workers > CLLO_NOALLOC_MAX_WORKERS) return CLLO_E_WORKSPACE;  // would not fit the fixed scratch
    int dev = 0;
    DeviceInfo* di = nullptr;
    int rc = current_device_info(&di, &dev);
    if (rc != CLLO_OK) return rc;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_ptr[dev]) {
            // set-up, once per device, with that device current (current_device_info asked which it is)
            void* ptr = nullptr;
            CLLO_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
            if (!ptr) return CLLO_E_CUDA;
            g_noalloc_ptr[dev] = ptr;
        }
        scratch = g_noalloc_ptr[dev];
    }
    if (num_workers <= 0) {
        decode::Plan plan;
        rc = decode::make_plan(B, S, Hq, Hkv, D, 0, di->sm_count, &plan);
        if (rc != CLLO_OK) return rc;
        num_workers = plan.prm.W < CLLO_NOALLOC_MAX_WORKERS ? plan.prm.W : CLLO_NOALLOC_MAX_WORKERS;
    }
    return cllo_gqa_decode_bf16(q, k, v, scale, o, scratch, sizeof(g_noalloc_scratch), B, S, Hq, Hkv, D, kv_layout,
                                num_workers, nullptr, stream);
}

// Source-compatibility path for upstream's C++ launcher signature (no workspace argument): use the
// caller's fp32 oIntermediate buffer [B,Hq,D] when it is large enough, else a per-device scratch that
// this library allocates once and keeps (released by cllo_shutdown()).
int cllo_gqa_decode_bf16_compat(const void* q, const void* k, const void* v, float scale, void* o,
                                float* o_intermediate, int B, int S, int Hq, int Hkv, int D) {
    DeviceInfo* di = nullptr;
    int rc = current_device_info(&di);
    if (rc != CLLO_OK) return rc;
    decode::Plan plan;
    rc = decode::make_plan(B, S, Hq, Hkv, D, 0, di->sm_count, &plan);
    if (rc != CLLO_OK) return rc;
    void* ws = nullptr;
    size_t ws_bytes = 0;
    const size_t inter_bytes = static_cast<size_t>(B) * Hq * D * sizeof(float);
    if (o_intermediate && inter_bytes >= plan.ws_bytes && aligned_to(o_intermediate, 256)) {
        ws = o_intermediate;
        ws_bytes = inter_bytes;
    } else {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (di->legacy_ws_bytes < plan.ws_bytes) {
            // an outgrown buffer is kept until cllo_shutdown(): another host thread may be between its look-up
            // and its launch on it
            void* fresh = nullptr;
            CLLO_CUDA_TRY(cudaMalloc(&fresh, plan.ws_bytes));
            if (di->legacy_ws) di->retired_ws.push_back(di->legacy_ws);
            di->legacy_ws = fresh;
            di->legacy_ws_bytes = plan.ws_bytes;
        }
        ws = di->legacy_ws;
        ws_bytes = di->legacy_ws_bytes;
    }
    return cllo_gqa_decode_bf16(q, k, v, scale, o, ws, ws_bytes, B, S, Hq, Hkv, D, CLLO_KV_BSHD, 0, nullptr,
                                nullptr);
}

}  // extern "C"
