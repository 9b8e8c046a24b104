// GQA attention backward for sm_100a (tcgen05 / tensor memory) without atomics: one grid (bwd_grads_kernel) of two
// kinds of block,
//
//   bwd_dq_block      one block per (batch, query head, 128 query rows); loops over KV tiles.
//                     S = Q K^T and dP = dO V^T into tensor memory; 256 threads turn them into
//                     dS = P o (dP - D) * scale with P = exp(scale*S - lse) (no row reduction: the forward
//                     pass left lse, a small pre-pass leaves D = rowsum(dO o O)); dS goes back to tensor
//                     memory as bf16 (a region of its own, two buffers) and feeds dQ += dS K as the A operand.
//   bwd_dkdv_block    one block per (batch, kv head, 128 kv rows); loops over all query rows of all heads of
//                     the group in steps of 64 rows.  It forms the TRANSPOSED tiles directly, S^T = K Q^T and
//                     dP^T = V dO^T, so that P^T and dS^T are again A operands in tensor memory for
//                     dV += P^T dO and dK += dS^T Q: no transposes through shared memory, and dK/dV are
//                     summed over the heads of the group in the accumulators: one rounding, deterministic.
//                     Steps alternate between two element-wise groups with their own halves of S^T and dP^T,
//                     so the products of one step run while the other step's P^T, dS^T are being formed.
//                     When (kv head, kv tile) pairs are too few to fill the GPU (one kv head, short
//                     sequence) the heads of a group are divided among several blocks; their fp32 partials
//                     go to the workspace and bwd_reduce_kernel sums them in a fixed order.
//
// Both recompute S and dP (7 tile products per (q tile, kv tile) instead of the minimal 5); in exchange no
// gradient is accumulated through global memory.  Tensor memory: dQ kernel S | dP | dS[0] | dS[1] | dQ (pipelined
// over the kv tiles, see there), dK/dV kernel S^T (2 x 64) | dP^T (2 x 64) | dV | dK (all 512 columns; P^T and dS^T
// are written over S^T and dP^T).  Shared-memory operand layouts, descriptors, TMA boxes and barrier conventions
// are those of the forward kernel (gqa_prefill.cuh).  In both kernels the warp that issues the MMAs runs its loop
// as a whole warp with the MMAs predicated on one lane (tc_mma_ss_lo_if): it is the pace-maker of the block.
//
// Upstream: flash_gqa_backward_bf16_kernel, src/python/Triton/flash_gqa_backward_kernel.py:159-310 (one
// Triton program per (kv block, query head), dQ/dK/dV accumulated with fp32 atomics) and
// rowwise_dot_o_grad_o_kernel (:16-48).
#pragma once

#include "gqa_prefill.cuh"

namespace cllo {
namespace backward {

using prefill::kBM;
using prefill::kBN;
using prefill::kD;
using prefill::kHalfBytes;
using prefill::kIdescPV;
using prefill::kIdescQK;
using prefill::kLog2e;
using prefill::kTileBytes;
using prefill::smem_desc;
using prefill::tc_commit;
using prefill::tc_fence_after;
using prefill::tc_fence_before;
using prefill::tc_mma_ss;
using prefill::tc_mma_ts;
using prefill::tc_commit_if;
using prefill::tc_mma_ss_lo_if;
using prefill::tc_mma_ts_lo_if;
using prefill::tmem_alloc;
using prefill::tmem_dealloc;
using prefill::tmem_ld32_wait;
using prefill::tmem_relinquish;
using prefill::tmem_st32;
using prefill::tmem_wait_st;
using prefill::add2;
using prefill::fma2;
using prefill::pk2;
using prefill::upk2;

__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

constexpr int kThreads = 320;  // warps 0-7 element-wise, 8 TMA, 9 MMA

enum : int {
    SITE_BWD_FIXED = 40,
    SITE_BWD_STREAM_FULL = 41,
    SITE_BWD_STREAM_EMPTY = 42,
    SITE_BWD_S_FULL = 43,
    SITE_BWD_DS_FULL = 44,
    SITE_BWD_DRAIN = 45,
};

// Epilogue staging.  The 256 element-wise threads hold a 128 x 128 fp32 tile, one row per thread (tensor-memory lane)
// and 64 of its columns each; stored row by thread, every store instruction would touch 32 rows (measured: 11,000
// cycles for the 128 KB of one dK/dV block).  So a tile goes through shared memory (free once the last MMA has retired),
// rows padded by 16 bytes so that both the row-per-thread writes and the row-per-warp reads are conflict-free, and
// leaves with 512 contiguous bytes per store instruction.
constexpr int kStageRowF32 = kD * 4 + 16;
constexpr int kStageRowBf16 = kD * 2 + 16;
// 32 values of one row, columns [col0, col0 + 32)
__device__ __forceinline__ void stage_f32(uint8_t* tile, int row, int col0, const float (&v)[32]) {
    float4* dst = reinterpret_cast<float4*>(tile + row * kStageRowF32 + col0 * 4);
#pragma unroll
    for (int e = 0; e < 32; e += 4) dst[e >> 2] = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
}
__device__ __forceinline__ void stage_bf16(uint8_t* tile, int row, int col0, const float (&v)[32]) {
    uint4* dst = reinterpret_cast<uint4*>(tile + row * kStageRowBf16 + col0 * 2);
#pragma unroll
    for (int e = 0; e < 32; e += 8) {
        uint4 pkt;
        pkt.x = pack_bf16x2(v[e + 0], v[e + 1]);
        pkt.y = pack_bf16x2(v[e + 2], v[e + 3]);
        pkt.z = pack_bf16x2(v[e + 4], v[e + 5]);
        pkt.w = pack_bf16x2(v[e + 6], v[e + 7]);
        dst[e >> 3] = pkt;
    }
}
// The first `rows` rows of a staged tile to `out` (row r at out + r * kD); warp w8 of 8 takes every eighth row (fp32)
// or every eighth pair of rows (bf16: half a warp per row).
__device__ __forceinline__ void unstage_f32(const uint8_t* tile, float* out, int rows, int w8, int lane) {
    for (int r = w8; r < rows; r += 8)
        *reinterpret_cast<float4*>(out + static_cast<long long>(r) * kD + lane * 4) =
            *reinterpret_cast<const float4*>(tile + r * kStageRowF32 + lane * 16);
}
__device__ __forceinline__ void unstage_bf16(const uint8_t* tile, __nv_bfloat16* out, int rows, int w8, int lane) {
    for (int r = 2 * w8 + (lane >> 4); r < rows; r += 16)
        *reinterpret_cast<uint4*>(out + static_cast<long long>(r) * kD + (lane & 15) * 8) =
            *reinterpret_cast<const uint4*>(tile + r * kStageRowBf16 + (lane & 15) * 16);
}

struct Params {
    const float* lse;    // [B,Hq,Sq], natural log units (forward output)
    const float* delta;  // [B,Hq,Sq], rowsum(dO o O)
    __nv_bfloat16* dq;   // [B,Hq,Sq,D]
    __nv_bfloat16* dk;   // [B,Hkv,Skv,D]
    __nv_bfloat16* dv;   // [B,Hkv,Skv,D]
    float* dkv_partial;  // head_splits > 1: fp32 [split][2: dV, dK][B,Hkv,Skv,D]
    float scale;
    int B, Sq, Skv, Hq, Hkv, G, causal, n_qt, n_kt;
    int head_splits;     // the query heads of a group are divided among this many blocks per kv tile
    int window;          // > 0: sliding window, a query sees kv in [q - (window - 1), q] (implies causal)
};

// tensor-memory column of the A operand for k-step ks when the 128 K-values were written by two
// warpgroups, each into the first 32 columns of its own 64-column half
__device__ __forceinline__ uint32_t a_col(int ks) { return static_cast<uint32_t>(ks < 4 ? ks * 8 : 64 + (ks - 4) * 8); }

// D[row] = sum_d dO[row][d] * O[row][d]; one warp per row of 128 dims
__global__ void __launch_bounds__(256) bwd_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                                        const __nv_bfloat16* __restrict__ grad_o,
                                                        float* __restrict__ delta, long long rows) {
    const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint2 a = *reinterpret_cast<const uint2*>(o + row * kD + lane * 4);
    const uint2 g = *reinterpret_cast<const uint2*>(grad_o + row * kD + lane * 4);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(g2[i]);
        acc += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) delta[row] = acc;
}

// Four S-type MMAs (both operands in shared memory, k steps 32 bytes apart, all accumulating) issued by the leader
// lane, behind a look at an mbarrier that every lane takes at its own barrier and reads only after the fourth MMA,
// so that the round trip of the look is covered by the MMAs.
__device__ __forceinline__ uint32_t tc_ss4_run_after_look(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                                          uint32_t idesc, uint32_t leader, uint32_t look_bar,
                                                          uint32_t look_parity) {
    uint32_t seen;
    asm volatile(
        "{\n\t"
        ".reg .pred pt, q, w;\n\t"
        ".reg .b64 da, db;\n\t"
        ".reg .b32 a, b;\n\t"
        "setp.ne.b32 q, %6, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 w, [%7], %8;\n\t"
        "mov.b64 da, {%2, %4};\n\t mov.b64 db, {%3, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %5, pt;\n\t"
        "add.u32 a, %2, 2;\n\t add.u32 b, %3, 2;\n\t mov.b64 da, {a, %4};\n\t mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %5, pt;\n\t"
        "add.u32 a, %2, 4;\n\t add.u32 b, %3, 4;\n\t mov.b64 da, {a, %4};\n\t mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %5, pt;\n\t"
        "add.u32 a, %2, 6;\n\t add.u32 b, %3, 6;\n\t mov.b64 da, {a, %4};\n\t mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %5, pt;\n\t"
        "selp.u32 %0, 1, 0, w;\n\t"
        "}"
        : "=r"(seen)
        : "r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(leader), "r"(look_bar), "r"(look_parity)
        : "memory");
    return seen;
}

// ------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------
// Pipelined over the kv tiles through tensor memory: S(j) and dP(j) land in two fixed regions, the element-wise threads
// copy them to registers at once and hand the regions back, so S(j+1), dP(j+1) are computed while dS(j) is being
// formed; dS has two homes, so dQ += dS(j) K(j) runs while dS(j+1) is written.
//   tensor memory: S (128) | dP (128) | dS[0] (64) | dS[1] (64) | dQ (128)
//   shared memory: Q, dO (fixed) | K x 3 stages (a K tile is still needed by the late dQ product) | V x 2 stages
namespace dq {
constexpr int kKStages = 3;
constexpr int kVStages = 2;
constexpr int kSmemK = 2 * kTileBytes;
constexpr int kSmemV = kSmemK + kKStages * kTileBytes;
constexpr int kSmemBar = kSmemV + kVStages * kTileBytes;  // 224 KB
constexpr int kNumBars = 20;
constexpr int kSmemBytes = kSmemBar + kNumBars * 8 + 32 + 1024;
constexpr uint32_t kColS = 0, kColDP = 128, kColDS = 256, kColDQ = 384;
struct Bars {
    uint32_t base;
    __device__ uint32_t fixed_full() const { return base; }
    __device__ uint32_t k_full(int s) const { return base + 8 * (1 + s); }
    __device__ uint32_t v_full(int s) const { return base + 8 * (4 + s); }
    __device__ uint32_t k_empty(int s) const { return base + 8 * (6 + s); }   // dQ(j) retired: K stage j % 3 free
    __device__ uint32_t sdp_full(int s) const { return base + 8 * (9 + s); }  // S(j), dP(j) landed (j % 2); V stage free
    __device__ uint32_t ds_full(int s) const { return base + 8 * (11 + s); }  // dS[j % 2] stored
    __device__ uint32_t dq_done(int s) const { return base + 8 * (13 + s); }  // dQ(j) retired: dS[j % 2] free
    __device__ uint32_t c_free() const { return base + 8 * 15; }              // S, dP of step j copied to registers
    __device__ uint32_t drain() const { return base + 8 * 16; }
};
}  // namespace dq

__device__ __forceinline__ void bwd_dq_block(const CUtensorMap* tm_q, const CUtensorMap* tm_k, const CUtensorMap* tm_v,
                                             const CUtensorMap* tm_do, const Params& p, long long block_id) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const dq::Bars bars{base + dq::kSmemBar};
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + dq::kSmemBar + dq::kNumBars * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + dq::kSmemBar + dq::kNumBars * 8 + 8);
    // warp index through a shuffle: the compiler then knows it to be the same in every lane
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

    long long id = block_id;
    const int g = static_cast<int>(id % p.G);
    id /= p.G;
    const int qt = p.n_qt - 1 - static_cast<int>(id % p.n_qt);  // heavy causal tiles first
    id /= p.n_qt;
    const int kvh = static_cast<int>(id % p.Hkv);
    const int b = static_cast<int>(id / p.Hkv);
    const int h = kvh * p.G + g;
    const int q0 = qt * kBM;
    // kv tiles [j_lo, j_lo + n_kv) can hold something visible to this block's rows
    int j_hi = p.n_kt;
    if (p.causal) {
        const int lim = (q0 + kBM - 1) / kBN + 1;
        j_hi = lim < j_hi ? lim : j_hi;
    }
    int j_lo = 0;
    if (p.window > 0 && q0 - (p.window - 1) > 0) j_lo = (q0 - (p.window - 1)) / kBN;
    if (j_lo > j_hi - 1) j_lo = j_hi - 1;
    const int n_kv = j_hi - j_lo;

    const uint32_t sm_q = base, sm_do = base + kTileBytes;
    auto sm_k = [&](int s) { return base + dq::kSmemK + s * kTileBytes; };
    auto sm_v = [&](int s) { return base + dq::kSmemV + s * kTileBytes; };
    auto load_k = [&](int j) {
        const int s = j % dq::kKStages;
        mbar_arrive_expect_tx(bars.k_full(s), kTileBytes);
        tma_load_4d(sm_k(s), tm_k, bars.k_full(s), 0, (j_lo + j) * kBN, kvh, b);
        tma_load_4d(sm_k(s) + kHalfBytes, tm_k, bars.k_full(s), 64, (j_lo + j) * kBN, kvh, b);
    };
    auto load_v = [&](int j) {
        const int s = j % dq::kVStages;
        mbar_arrive_expect_tx(bars.v_full(s), kTileBytes);
        tma_load_4d(sm_v(s), tm_v, bars.v_full(s), 0, (j_lo + j) * kBN, kvh, b);
        tma_load_4d(sm_v(s) + kHalfBytes, tm_v, bars.v_full(s), 64, (j_lo + j) * kBN, kvh, b);
    };

    if (warp == 8 && lane == 0) {
        mbar_init(bars.fixed_full(), 1);
        for (int s = 0; s < 3; ++s) {
            mbar_init(bars.k_full(s), 1);
            mbar_init(bars.k_empty(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(bars.v_full(s), 1);
            mbar_init(bars.sdp_full(s), 1);
            mbar_init(bars.ds_full(s), 2 * kBM);
            mbar_init(bars.dq_done(s), 1);
        }
        mbar_init(bars.c_free(), 2 * kBM);
        mbar_init(bars.drain(), 1);
        *abort_flag = 0;
        fence_mbar_init();
        // the first copies start before the block has met at its first barrier
        mbar_arrive_expect_tx(bars.fixed_full(), 2 * kTileBytes);
        tma_load_4d(sm_q, tm_q, bars.fixed_full(), 0, q0, h, b);
        tma_load_4d(sm_q + kHalfBytes, tm_q, bars.fixed_full(), 64, q0, h, b);
        tma_load_4d(sm_do, tm_do, bars.fixed_full(), 0, q0, h, b);
        tma_load_4d(sm_do + kHalfBytes, tm_do, bars.fixed_full(), 64, q0, h, b);
        load_k(0);
        load_v(0);
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tm_s = tmem_base + dq::kColS, tm_dp = tmem_base + dq::kColDP, tm_dq = tmem_base + dq::kColDQ;

    if (warp == 8) {
        if (lane == 0) {
            for (int j = 1; j < n_kv; ++j) {
                if (j >= dq::kKStages)  // stage j % 3 held K(j-3): free once dQ(j-3) has retired
                    mbar_wait(bars.k_empty(j % dq::kKStages), static_cast<uint32_t>((j - 3) / 3) & 1u, abort_flag,
                              SITE_BWD_STREAM_EMPTY, j);
                load_k(j);
                if (j >= dq::kVStages)  // stage j % 2 held V(j-2): free once dP(j-2) has retired
                    mbar_wait(bars.sdp_full(j & 1), static_cast<uint32_t>((j - 2) >> 1) & 1u, abort_flag,
                              SITE_BWD_STREAM_EMPTY, j);
                load_v(j);
            }
            if (*abort_flag) {
                for (int j = (n_kv > 2 ? n_kv - 2 : 0); j < n_kv; ++j) {
                    const long long t0 = clock64();
                    while (!(mbar_try_wait(bars.k_full(j % 3), static_cast<uint32_t>(j / 3) & 1u) &&
                             mbar_try_wait(bars.v_full(j & 1), static_cast<uint32_t>(j >> 1) & 1u)) &&
                           clock64() - t0 < kWaitLimitCycles / 64) {
                    }
                }
            }
        }
    } else if (warp == 9) {
        // One thread issues every MMA; per kv tile one run of 16 (S and dP of the NEXT tile) and one of 8 (dQ of this
        // tile), each behind one look at its barriers (the whole warp looks at once, one barrier per lane).
        // The whole warp runs the issue code with the MMAs predicated on the leader lane (see tc_mma_ss_lo_if), on the
        // low words of the descriptors (per k step and per stage only a constant is added).
        const uint32_t leader = lane == 0 ? 1u : 0u;
        const uint32_t hi = prefill::smem_desc_hi(1024);
        const uint32_t q_lo = prefill::smem_desc_lo(sm_q, 16), do_lo = prefill::smem_desc_lo(sm_do, 16);
        const uint32_t k_kmaj = prefill::smem_desc_lo(sm_k(0), 16), v_kmaj = prefill::smem_desc_lo(sm_v(0), 16);
        const uint32_t k_mnmaj = prefill::smem_desc_lo(sm_k(0), kHalfBytes);
        // S = Q K^T and dP = dO V^T of tile j; the last four k steps of dP go out behind a look at (bar, par) that
        // every lane takes and reads after them
        auto issue_sdp = [&](int j, uint32_t bar, uint32_t par) {
            const uint32_t ka = k_kmaj + static_cast<uint32_t>(j % dq::kKStages) * (kTileBytes >> 4);
            const uint32_t va = v_kmaj + static_cast<uint32_t>(j & 1) * (kTileBytes >> 4);
            tc_mma_ss_lo_if<false>(leader, tm_s, q_lo, ka, hi, kIdescQK);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks) {
                const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
                tc_mma_ss_lo_if<true>(leader, tm_s, q_lo + off, ka + off, hi, kIdescQK);
            }
            tc_mma_ss_lo_if<false>(leader, tm_dp, do_lo, va, hi, kIdescQK);
#pragma unroll
            for (int ks = 1; ks < 4; ++ks)
                tc_mma_ss_lo_if<true>(leader, tm_dp, do_lo + ((ks * 32) >> 4), va + ((ks * 32) >> 4), hi, kIdescQK);
            return tc_ss4_run_after_look(tm_dp, do_lo + (kHalfBytes >> 4), va + (kHalfBytes >> 4), hi, kIdescQK, leader,
                                         bar, par);
        };
        // what a lane looks at before S, dP of tile j + 1 are issued: lane 0 S, dP of tile j copied out; 1 K(j + 1)
        // arrived; 2 V(j + 1) arrived (the other lanes repeat lane 0)
        auto landing_barrier = [&](int j, uint32_t& bar, uint32_t& par) {
            bar = bars.c_free();
            par = static_cast<uint32_t>(j) & 1u;
            if (lane == 1) {
                bar = bars.k_full((j + 1) % dq::kKStages);
                par = static_cast<uint32_t>((j + 1) / 3) & 1u;
            } else if (lane == 2) {
                bar = bars.v_full((j + 1) & 1);
                par = static_cast<uint32_t>((j + 1) >> 1) & 1u;
            }
        };
        mbar_wait(bars.fixed_full(), 0, abort_flag, SITE_BWD_FIXED, 0);
        mbar_wait(bars.k_full(0), 0, abort_flag, SITE_BWD_STREAM_FULL, 0);
        mbar_wait(bars.v_full(0), 0, abort_flag, SITE_BWD_STREAM_FULL, 0);
        tc_fence_after();
        issue_sdp(0, bars.fixed_full(), 0);
        tc_commit_if(leader, bars.sdp_full(0));
        // Per kv tile two runs, S, dP of the next tile (16 MMAs) and dQ of this tile (8); each run carries, before its
        // last MMAs, the look at the barriers of the run after it, read when the run has been issued.
        bool landing_seen = false;
#pragma unroll 1
        for (int j = 0; j < n_kv; ++j) {
            uint32_t my_bar, my_par;
            bool ds_seen = false;
            if (j + 1 < n_kv) {
                if (!landing_seen) {
                    landing_barrier(j, my_bar, my_par);
                    if (!__all_sync(0xffffffffu, mbar_try_wait(my_bar, my_par))) {
                        if (lane < 3) mbar_wait(my_bar, my_par, abort_flag, SITE_BWD_STREAM_FULL, j);
                        __syncwarp();
                    }
                }
                tc_fence_after();
                const uint32_t mine = issue_sdp(j + 1, bars.ds_full(j & 1), static_cast<uint32_t>(j >> 1) & 1u);
                tc_commit_if(leader, bars.sdp_full((j + 1) & 1));
                ds_seen = __all_sync(0xffffffffu, mine != 0);
            }
            if (!ds_seen)
                mbar_wait(bars.ds_full(j & 1), static_cast<uint32_t>(j >> 1) & 1u, abort_flag, SITE_BWD_DS_FULL, j);
            tc_fence_after();
            const uint32_t kb = k_mnmaj + static_cast<uint32_t>(j % dq::kKStages) * (kTileBytes >> 4);
            const uint32_t dsa = tmem_base + dq::kColDS + (j & 1) * 64;
            // dQ (+)= dS K (K tile as the MN-major B operand), with the look for S, dP of tile j + 2
            if (j + 2 < n_kv) {
                landing_barrier(j + 1, my_bar, my_par);
            } else {
                my_bar = bars.fixed_full();
                my_par = 0;
            }
            const uint32_t mine = prefill::tc_pv_run_with_look(tm_dq, dsa, kb, hi, kIdescPV, j == 0 ? 0u : 1u, leader,
                                                               my_bar, my_par);
            landing_seen = __all_sync(0xffffffffu, mine != 0);
            tc_commit_if(leader, bars.dq_done(j & 1));
            tc_commit_if(leader, bars.k_empty(j % dq::kKStages));
        }
        __syncwarp();
        if (lane == 0) {
            tc_commit(bars.drain());
            mbar_wait(bars.drain(), 0, abort_flag, SITE_BWD_DRAIN, 0);
            if (*abort_flag) {
                const long long t0 = clock64();
                while (!mbar_try_wait(bars.drain(), 0) && clock64() - t0 < kWaitLimitCycles / 64) {
                }
            }
        }
    } else {
        // element-wise: thread = (query row, 64 of the 128 kv columns)
        const int half = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        const int qi = q0 + row;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const bool row_ok = qi < p.Sq;
        const long long vec_idx = (static_cast<long long>(b) * p.Hq + h) * p.Sq + qi;
        const float lse2 = row_ok ? p.lse[vec_idx] * kLog2e : 0.f;
        const float drow = row_ok ? p.delta[vec_idx] : 0.f;
        const float c = p.scale * kLog2e;
#pragma unroll 1
        for (int j = 0; j < n_kv; ++j) {
            mbar_wait(bars.sdp_full(j & 1), static_cast<uint32_t>(j >> 1) & 1u, abort_flag, SITE_BWD_S_FULL, j);
            __syncwarp();
            tc_fence_after();
            float sv[64], dpv[64];
            {
                float t0[32], t1[32];
                tmem_ld32_wait(tm_s + lane_base + half * 64, t0);
                tmem_ld32_wait(tm_s + lane_base + half * 64 + 32, t1);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    sv[e] = t0[e];
                    sv[32 + e] = t1[e];
                }
                tmem_ld32_wait(tm_dp + lane_base + half * 64, t0);
                tmem_ld32_wait(tm_dp + lane_base + half * 64 + 32, t1);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    dpv[e] = t0[e];
                    dpv[32 + e] = t1[e];
                }
            }
            tc_fence_before();
            mbar_arrive(bars.c_free());  // both regions are in registers: the next tile's S and dP may land

            // columns this row may see in this tile (only diagonal and tail tiles need the test)
            const int kvt0 = (j_lo + j) * kBN;  // first kv position of this tile
            int limit = p.Skv - 1 - kvt0;
            if (p.causal) {
                const int cl = qi - kvt0;
                limit = cl < limit ? cl : limit;
            }
            const int first = p.window > 0 ? qi - (p.window - 1) - kvt0 : 0;
            const bool need_mask = (kvt0 + kBN > p.Skv) || (p.causal && (kvt0 + kBN - 1 > q0)) ||
                                   (p.window > 0 && (kvt0 < q0 + kBM - 1 - (p.window - 1)));
            const uint64_t c2 = pk2(c, c), nl2 = pk2(-lse2, -lse2);
            const uint64_t sc2 = pk2(p.scale, p.scale), nds2 = pk2(-drow * p.scale, -drow * p.scale);
            uint32_t pk[32];
            const int col0 = half * 64;
#pragma unroll
            for (int e = 0; e < 64; e += 2) {
                float y0, y1;
                upk2(fma2(pk2(sv[e], sv[e + 1]), c2, nl2), y0, y1);
                float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
                if (need_mask) {
                    p0 = (col0 + e <= limit && col0 + e >= first) ? p0 : 0.f;
                    p1 = (col0 + e + 1 <= limit && col0 + e + 1 >= first) ? p1 : 0.f;
                }
                // dS = P * (dP - D) * scale
                float d0, d1;
                upk2(mul2(pk2(p0, p1), fma2(pk2(dpv[e], dpv[e + 1]), sc2, nds2)), d0, d1);
                pk[e >> 1] = pack_bf16x2(d0, d1);
            }
            // dS[j % 2] still feeds dQ += dS(j-2) K(j-2) until that product has retired
            if (j >= 2) {
                mbar_wait(bars.dq_done(j & 1), static_cast<uint32_t>((j - 2) >> 1) & 1u, abort_flag, SITE_BWD_DS_FULL, j);
                __syncwarp();
                tc_fence_after();
            }
            // dS (bf16): this half's 64 values are columns [32 * half, 32 * half + 32) of dS[j % 2]
            tmem_st32(tmem_base + dq::kColDS + (j & 1) * 64 + lane_base + half * 32, pk);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bars.ds_full(j & 1));
        }
        // epilogue: dQ -> bf16
        mbar_wait(bars.drain(), 0, abort_flag, SITE_BWD_DRAIN, 1);
        __syncwarp();
        tc_fence_after();
        // through shared memory (see stage_f32); every MMA has retired, so the Q tile's place is free
        uint8_t* tile = gen_base;
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
            float ov[32];
            tmem_ld32_wait(tm_dq + lane_base + half * 64 + cc * 32, ov);
            stage_bf16(tile, row, half * 64 + cc * 32, ov);
        }
        named_bar_sync(1, 2 * kBM);
        const int rows_here = p.Sq - q0 < kBM ? p.Sq - q0 : kBM;
        unstage_bf16(tile, p.dq + ((static_cast<long long>(b) * p.Hq + h) * p.Sq + q0) * kD, rows_here, warp, lane);
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------------------
// dK, dV
// ------------------------------------------------------------------------------------------------
// A step is 64 query rows of one head against the block's 128 kv rows.  Steps alternate between two element-wise
// groups of 128 threads (group = step parity), each with its own 64-column halves of S^T and dP^T in tensor memory
// and its own pair of barriers, so the products of one group's steps run while the other group forms P^T and dS^T:
//   MMA thread   S^T,dP^T(0) | S^T,dP^T(1) | wait dS(0): dV,dK(0), S^T,dP^T(2) | wait dS(1): dV,dK(1), S^T,dP^T(3) | ...
//   group 0      ............. P^T,dS^T(0) ............................ P^T,dS^T(2) ...
//   group 1      ........................... P^T,dS^T(1) ............................ P^T,dS^T(3) ...
// (the tensor pipe executes one thread's MMAs in issue order, so S^T(st+2) may be issued over P^T(st) right behind
// the products that read it).  Q and dO arrive as 64-row tiles in four 32 KB stages.
//   tensor memory: S^T (2 x 64) | dP^T (2 x 64) | dV (128) | dK (128)
//   shared memory: K, V (fixed) | [4 stages][Q 64 rows, dO 64 rows] | lse, delta of the step [group][parity][2][64]
namespace dkdv {
constexpr int kBQ = 64;                       // query rows per step
constexpr int kStages = 4;
constexpr int kQHalfBytes = kBQ * 128;        // one 64-column half of a 64-row tile
constexpr int kQTileBytes = 2 * kQHalfBytes;  // 16 KB
constexpr int kStageBytes = 2 * kQTileBytes;  // Q + dO
constexpr int kSmemStream = 2 * kTileBytes;
constexpr int kSmemVec = kSmemStream + kStages * kStageBytes;
constexpr int kSmemBar = kSmemVec + 2 * 2 * 2 * kBQ * 4;
constexpr int kNumBars = 14;
constexpr int kSmemBytes = kSmemBar + kNumBars * 8 + 32 + 1024;
// S^T and dP^T of one step: M = 128 kv rows, N = 64 query rows
constexpr uint32_t kIdescScores = (kIdescQK & ~(0x3fu << 17)) | ((kBQ >> 3) << 17);
struct Bars {
    uint32_t base;
    __device__ uint32_t fixed_full() const { return base; }
    __device__ uint32_t stream_full(int s) const { return base + 8 * (1 + s); }
    __device__ uint32_t stream_empty(int s) const { return base + 8 * (5 + s); }
    __device__ uint32_t s_full(int g) const { return base + 8 * (9 + g); }    // S^T, dP^T of group g's step landed
    __device__ uint32_t ds_full(int g) const { return base + 8 * (11 + g); }  // P^T, dS^T of group g's step stored
    __device__ uint32_t drain() const { return base + 8 * 13; }
};
}  // namespace dkdv

__device__ __forceinline__ void bwd_dkdv_block(const CUtensorMap* tm_q, const CUtensorMap* tm_k, const CUtensorMap* tm_v,
                                               const CUtensorMap* tm_do, const Params& p, long long block_id) {
    using namespace dkdv;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const dkdv::Bars bars{base + dkdv::kSmemBar};
    float* vec = reinterpret_cast<float*>(gen_base + dkdv::kSmemVec);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + dkdv::kSmemBar + dkdv::kNumBars * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + dkdv::kSmemBar + dkdv::kNumBars * 8 + 8);
    // warp index through a shuffle: the compiler then knows it to be the same in every lane
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

    long long id = block_id;
    const int split = static_cast<int>(id % p.head_splits);
    id /= p.head_splits;
    const int jt = static_cast<int>(id % p.n_kt);  // early kv tiles carry the most query tiles when causal
    id /= p.n_kt;
    const int kvh = static_cast<int>(id % p.Hkv);
    const int b = static_cast<int>(id / p.Hkv);
    const int kv0 = jt * kBN;
    const int i_lo = p.causal ? kv0 / kBQ : 0;  // first 64-row query tile that can see this kv tile
    int i_hi = (p.Sq + kBQ - 1) / kBQ;          // one past the last one (a window ends it early)
    if (p.window > 0) {
        const int lim = (kv0 + kBN - 1 + p.window - 1) / kBQ + 1;
        i_hi = lim < i_hi ? lim : i_hi;
    }
    const int n_i = i_hi - i_lo;                 // may be <= 0 when Skv > Sq: nothing to accumulate
    const int heads_here = p.G / p.head_splits;  // head_splits divides G
    const int head0 = kvh * p.G + split * heads_here;
    const int n_steps = n_i > 0 ? n_i * heads_here : 0;

    const uint32_t sm_k = base, sm_v = base + kTileBytes;
    auto sm_q = [&](int s) { return base + dkdv::kSmemStream + s * kStageBytes; };
    auto sm_do = [&](int s) { return base + dkdv::kSmemStream + s * kStageBytes + kQTileBytes; };
    // copy thread: position in (head, 64-row query tile) order and the copies of one step
    int ld_h = head0, ld_i = 0;
    auto load_step = [&](int st) {
        const int s = st % dkdv::kStages;
        const int qrow0 = (i_lo + ld_i) * kBQ;
        mbar_arrive_expect_tx(bars.stream_full(s), kStageBytes);
        tma_load_4d(sm_q(s), tm_q, bars.stream_full(s), 0, qrow0, ld_h, b);
        tma_load_4d(sm_q(s) + kQHalfBytes, tm_q, bars.stream_full(s), 64, qrow0, ld_h, b);
        tma_load_4d(sm_do(s), tm_do, bars.stream_full(s), 0, qrow0, ld_h, b);
        tma_load_4d(sm_do(s) + kQHalfBytes, tm_do, bars.stream_full(s), 64, qrow0, ld_h, b);
        if (++ld_i == n_i) {
            ld_i = 0;
            ++ld_h;
        }
    };
    if (warp == 8 && lane == 0) {
        mbar_init(bars.fixed_full(), 1);
        for (int s = 0; s < dkdv::kStages; ++s) {
            mbar_init(bars.stream_full(s), 1);
            mbar_init(bars.stream_empty(s), 1);
        }
        for (int g = 0; g < 2; ++g) {
            mbar_init(bars.s_full(g), 1);
            mbar_init(bars.ds_full(g), kBM);
        }
        mbar_init(bars.drain(), 1);
        *abort_flag = 0;
        fence_mbar_init();
        // the first copies start before the block has met at its first barrier (every stage is free)
        if (n_steps > 0) {
            mbar_arrive_expect_tx(bars.fixed_full(), 2 * kTileBytes);
            tma_load_4d(sm_k, tm_k, bars.fixed_full(), 0, kv0, kvh, b);
            tma_load_4d(sm_k + kHalfBytes, tm_k, bars.fixed_full(), 64, kv0, kvh, b);
            load_step(0);
            tma_load_4d(sm_v, tm_v, bars.fixed_full(), 0, kv0, kvh, b);
            tma_load_4d(sm_v + kHalfBytes, tm_v, bars.fixed_full(), 64, kv0, kvh, b);
            for (int st = 1; st < dkdv::kStages && st < n_steps; ++st) load_step(st);
        }
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tm_st = tmem_base, tm_dpt = tmem_base + 128, tm_dv = tmem_base + 256, tm_dk = tmem_base + 384;

    if (warp == 8) {
        if (lane == 0 && n_steps > 0) {
            for (int st = dkdv::kStages; st < n_steps; ++st) {
                const int s = st % dkdv::kStages;
                const uint32_t use = static_cast<uint32_t>(st / dkdv::kStages);
                // (a barrier of the stage's own: the commit behind S^T of step st - 2 also covers the products that
                // read this stage, but this thread runs up to two phases of that barrier ahead, which a parity wait
                // cannot tell apart)
                mbar_wait(bars.stream_empty(s), (use & 1u) ^ 1u, abort_flag, SITE_BWD_STREAM_EMPTY, st);
                load_step(st);
            }
            if (*abort_flag) {
                for (int st = (n_steps > dkdv::kStages ? n_steps - dkdv::kStages : 0); st < n_steps; ++st) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bars.stream_full(st % dkdv::kStages),
                                          static_cast<uint32_t>(st / dkdv::kStages) & 1u) &&
                           clock64() - t0 < kWaitLimitCycles / 64) {
                    }
                }
            }
        }
    } else if (warp == 9) {
        // Lane 0 issues every MMA; the whole warp stays in the loop because the looks at the next step's barriers are
        // taken by all lanes (one barrier per lane).  The issuing thread is the pace-maker of the block: a look at
        // an mbarrier whose result is needed at once, or a commit, each leave the tensor pipe idle for the round trip
        // (memory-pipe instructions are carried out in order behind the queued MMAs).  So a step is ONE run of 24
        // MMAs -- dV, dK of step st, then S^T, dP^T of step st + 2 -- with the looks for the next run issued before
        // the run's last four MMAs and read only after them, and both commits at the end of the run.
        if (n_steps > 0) {
            const uint32_t leader = lane == 0 ? 1u : 0u;
            mbar_wait(bars.fixed_full(), 0, abort_flag, SITE_BWD_FIXED, 0);
            // Low descriptor words (per k step and per stage only a constant is added: the tiles are 1024-byte aligned
            // and no sum leaves the 14-bit address field).
            const uint32_t hi = prefill::smem_desc_hi(1024);
            const uint32_t k_lo = prefill::smem_desc_lo(sm_k, 16), v_lo = prefill::smem_desc_lo(sm_v, 16);
            const uint32_t q_kmaj = prefill::smem_desc_lo(sm_q(0), 16), do_kmaj = prefill::smem_desc_lo(sm_do(0), 16);
            const uint32_t q_mnmaj = prefill::smem_desc_lo(sm_q(0), kQHalfBytes);
            const uint32_t do_mnmaj = prefill::smem_desc_lo(sm_do(0), kQHalfBytes);
            constexpr uint32_t kOffKv4 = (kHalfBytes) >> 4, kOffQ4 = (kQHalfBytes) >> 4;  // k step 4: second 64-dim half
            auto stream_parity = [&](int st) { return static_cast<uint32_t>(st / dkdv::kStages) & 1u; };
            // S^T = K Q^T (all eight k steps) and the first four k steps of dP^T = V dO^T of step st
            auto issue_scores_head = [&](int st) {
                const uint32_t soff = static_cast<uint32_t>(st % dkdv::kStages) * (kStageBytes >> 4);
                const uint32_t col = static_cast<uint32_t>(st & 1) * kBQ;
                const uint32_t qa = q_kmaj + soff, da = do_kmaj + soff;
                tc_mma_ss_lo_if<false>(leader, tm_st + col, k_lo, qa, hi, kIdescScores);
#pragma unroll
                for (int ks = 1; ks < 8; ++ks)
                    tc_mma_ss_lo_if<true>(leader, tm_st + col, k_lo + (((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4),
                                          qa + (((ks >> 2) * kQHalfBytes + (ks & 3) * 32) >> 4), hi, kIdescScores);
                tc_mma_ss_lo_if<false>(leader, tm_dpt + col, v_lo, da, hi, kIdescScores);
#pragma unroll
                for (int ks = 1; ks < 4; ++ks)
                    tc_mma_ss_lo_if<true>(leader, tm_dpt + col, v_lo + ((ks * 32) >> 4), da + ((ks * 32) >> 4), hi,
                                          kIdescScores);
            };
            // the last four k steps of dP^T of step st, with a look at (bar, par) issued first and read afterwards
            auto issue_scores_tail = [&](int st, uint32_t bar, uint32_t par) {
                const uint32_t soff = static_cast<uint32_t>(st % dkdv::kStages) * (kStageBytes >> 4);
                const uint32_t col = static_cast<uint32_t>(st & 1) * kBQ;
                return tc_ss4_run_after_look(tm_dpt + col, v_lo + kOffKv4, do_kmaj + soff + kOffQ4, hi, kIdescScores,
                                             leader, bar, par);
            };
            // what a lane looks at before the run of step st: lane 0 ds_full(st), lane 1 stream_full(st + 2) (the
            // other lanes, and lane 1 when there is no step st + 2, repeat lane 0)
            auto my_barrier = [&](int st, uint32_t& bar, uint32_t& par, int& site) {
                bar = bars.ds_full(st & 1);
                par = static_cast<uint32_t>(st >> 1) & 1u;
                site = SITE_BWD_DS_FULL;
                if (lane == 1 && st + 2 < n_steps) {
                    bar = bars.stream_full((st + 2) % dkdv::kStages);
                    par = stream_parity(st + 2);
                    site = SITE_BWD_STREAM_FULL;
                }
            };
            for (int st = 0; st < 2 && st < n_steps; ++st) {
                mbar_wait(bars.stream_full(st), 0, abort_flag, SITE_BWD_STREAM_FULL, st);
                tc_fence_after();
                issue_scores_head(st);
                issue_scores_tail(st, bars.stream_full(st), 0);
                tc_commit_if(leader, bars.s_full(st & 1));
            }
            bool seen = false;
#pragma unroll 1
            for (int st = 0; st < n_steps; ++st) {
                uint32_t my_bar, my_par;
                int my_site;
                if (!seen) {
                    my_barrier(st, my_bar, my_par, my_site);
                    if (!__all_sync(0xffffffffu, mbar_try_wait(my_bar, my_par))) {
                        if (lane < 2) mbar_wait(my_bar, my_par, abort_flag, my_site, st);
                        __syncwarp();
                    }
                }
                const bool more = st + 2 < n_steps;
                const uint32_t soff = static_cast<uint32_t>(st % dkdv::kStages) * (kStageBytes >> 4);
                const uint32_t col = static_cast<uint32_t>(st & 1) * kBQ;
                const uint32_t db = do_mnmaj + soff, qb = q_mnmaj + soff;
                const uint32_t acc0 = st == 0 ? 0u : 1u;
                tc_fence_after();
                tc_mma_ts_lo_if(leader, tm_dv, tm_st + col, db, hi, kIdescPV, acc0);  // dV (+)= P^T dO
#pragma unroll
                for (int ks = 1; ks < 4; ++ks)
                    tc_mma_ts_lo_if(leader, tm_dv, tm_st + col + ks * 8, db + ks * (2048 >> 4), hi, kIdescPV, 1u);
                tc_mma_ts_lo_if(leader, tm_dk, tm_dpt + col, qb, hi, kIdescPV, acc0);  // dK (+)= dS^T Q
#pragma unroll
                for (int ks = 1; ks < 4; ++ks)
                    tc_mma_ts_lo_if(leader, tm_dk, tm_dpt + col + ks * 8, qb + ks * (2048 >> 4), hi, kIdescPV, 1u);
                if (more) issue_scores_head(st + 2);
                seen = false;
                if (st + 1 < n_steps) {
                    my_barrier(st + 1, my_bar, my_par, my_site);
                    const uint32_t mine =
                        more ? issue_scores_tail(st + 2, my_bar, my_par) : (mbar_try_wait(my_bar, my_par) ? 1u : 0u);
                    seen = __all_sync(0xffffffffu, mine != 0);
                }
                if (more) tc_commit_if(leader, bars.s_full(st & 1));
                tc_commit_if(leader, bars.stream_empty(st % dkdv::kStages));
            }
        }
        __syncwarp();
        if (lane == 0 && n_steps > 0) {
            tc_commit(bars.drain());
            mbar_wait(bars.drain(), 0, abort_flag, SITE_BWD_DRAIN, 0);
            if (*abort_flag) {
                const long long t0 = clock64();
                while (!mbar_try_wait(bars.drain(), 0) && clock64() - t0 < kWaitLimitCycles / 64) {
                }
            }
        }
    } else {
        // element-wise: thread = (kv row, group); a group takes every other step (64 query columns)
        const int grp = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        const int kvi = kv0 + row;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t my_st = tm_st + lane_base + grp * kBQ, my_dpt = tm_dpt + lane_base + grp * kBQ;
        const float c = p.scale * kLog2e;
        const int gtid = threadIdx.x & 127;
        float* vgrp = vec + grp * (2 * 2 * kBQ);
        int h = head0, i = grp;
        while (n_i > 0 && i >= n_i) {
            i -= n_i;
            ++h;
        }
#pragma unroll 1
        for (int st = grp, it = 0; st < n_steps; st += 2, ++it) {
            const int qrow0 = (i_lo + i) * kBQ;
            // stage lse*log2e and delta*scale of the 64 query rows of this step (zeros beyond Sq)
            float* vbuf = vgrp + (it & 1) * (2 * kBQ);
            {
                const int qr = qrow0 + (gtid & (kBQ - 1));
                const long long vi = (static_cast<long long>(b) * p.Hq + h) * p.Sq + qr;
                float val = 0.f;
                if (qr < p.Sq) val = gtid < kBQ ? p.lse[vi] * kLog2e : p.delta[vi] * p.scale;
                vbuf[gtid] = val;
            }
            named_bar_sync(1 + grp, kBM);
            mbar_wait(bars.s_full(grp), static_cast<uint32_t>(it) & 1u, abort_flag, SITE_BWD_S_FULL, st);
            __syncwarp();
            tc_fence_after();
            // query columns that see this kv row: q >= kv (causal) and q < Sq (only edge tiles need the test)
            const int first = p.causal ? kvi - qrow0 : 0;
            int limit = p.Sq - 1 - qrow0;
            if (p.window > 0) {
                const int wl = kvi + (p.window - 1) - qrow0;  // last query that still has this kv in its window
                limit = wl < limit ? wl : limit;
            }
            const bool need_mask = (qrow0 + kBQ > p.Sq) || (p.causal && (kv0 + kBN - 1 > qrow0)) ||
                                   (p.window > 0 && (qrow0 + kBQ - 1 > kv0 + (p.window - 1)));
            const uint64_t c2 = pk2(c, c), sc2 = pk2(p.scale, p.scale);
            uint32_t pkp[32], pkd[32];
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int col0 = cc * 32;
                float sv[32], dpv[32];
                tmem_ld32_wait(my_st + col0, sv);
                tmem_ld32_wait(my_dpt + col0, dpv);
#pragma unroll
                for (int e = 0; e < 32; e += 4) {
                    // lse*log2e and delta*scale of four query columns at a time (same address for the whole warp)
                    const float4 l4 = *reinterpret_cast<const float4*>(vbuf + col0 + e);
                    const float4 d4 = *reinterpret_cast<const float4*>(vbuf + kBQ + col0 + e);
#pragma unroll
                    for (int u = 0; u < 4; u += 2) {
                        const int q_a = col0 + e + u, q_b = q_a + 1;
                        const uint64_t nl2 = u == 0 ? pk2(-l4.x, -l4.y) : pk2(-l4.z, -l4.w);
                        const uint64_t nd2 = u == 0 ? pk2(-d4.x, -d4.y) : pk2(-d4.z, -d4.w);
                        float y0, y1;
                        upk2(fma2(pk2(sv[e + u], sv[e + u + 1]), c2, nl2), y0, y1);
                        float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
                        if (need_mask) {
                            p0 = (q_a >= first && q_a <= limit) ? p0 : 0.f;
                            p1 = (q_b >= first && q_b <= limit) ? p1 : 0.f;
                        }
                        float d0, d1;
                        upk2(mul2(pk2(p0, p1), fma2(pk2(dpv[e + u], dpv[e + u + 1]), sc2, nd2)), d0, d1);
                        pkp[cc * 16 + ((e + u) >> 1)] = pack_bf16x2(p0, p1);
                        pkd[cc * 16 + ((e + u) >> 1)] = pack_bf16x2(d0, d1);
                    }
                }
            }
            tmem_st32(my_st, pkp);
            tmem_st32(my_dpt, pkd);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bars.ds_full(grp));
            i += 2;
            while (i >= n_i) {
                i -= n_i;
                ++h;
            }
        }
        // epilogue: dV, dK -> bf16 (zeros when no query tile reaches this kv tile); thread = (kv row, 64 of 128 dims)
        const int half = grp;
        if (n_steps > 0) {
            mbar_wait(bars.drain(), 0, abort_flag, SITE_BWD_DRAIN, 1);
            __syncwarp();
            tc_fence_after();
        }
        // both tiles through shared memory (see stage_f32); every MMA has retired, so all of it is free
        static_assert(2 * kBN * kStageRowF32 <= dkdv::kSmemVec, "the staged tiles must fit below the vectors");
        const int rows_here = p.Skv - kv0 < kBN ? p.Skv - kv0 : kBN;
        const long long tile_off = ((static_cast<long long>(b) * p.Hkv + kvh) * p.Skv + kv0) * kD;
        const long long tensor_elems = static_cast<long long>(p.B) * p.Hkv * p.Skv * kD;
        const bool partial = p.head_splits > 1;  // fp32 partial of this head split; summed by bwd_reduce_kernel
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
            uint8_t* tile = gen_base + which * (kBN * kStageRowF32);
            const uint32_t src = (which == 0 ? tm_dv : tm_dk) + lane_base + half * 64;
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                float ov[32];
                if (n_steps > 0) {
                    tmem_ld32_wait(src + cc * 32, ov);
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) ov[e] = 0.f;
                }
                if (partial)
                    stage_f32(tile, row, half * 64 + cc * 32, ov);
                else
                    stage_bf16(tile, row, half * 64 + cc * 32, ov);
            }
        }
        named_bar_sync(3, 2 * kBM);
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
            const uint8_t* tile = gen_base + which * (kBN * kStageRowF32);
            if (partial)
                unstage_f32(tile, p.dkv_partial + (split * 2LL + which) * tensor_elems + tile_off, rows_here, warp, lane);
            else
                unstage_bf16(tile, (which == 0 ? p.dv : p.dk) + tile_off, rows_here, warp, lane);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Both kinds of block in ONE grid: the dK/dV blocks first (they are the longer ones), then the dQ blocks, which move
// onto the SMs as the last wave of dK/dV blocks drains -- two launches would leave each kernel's last wave to itself
// (512 equal blocks on 148 SMs: 4 waves where 3.46 would do).  Neither kind reads what the other writes.  Measured
// against the alternatives (upstream's shape causal / non-causal / B=2, Hq=32, Hkv=4, S=8192 causal, us per call): two
// launches 273 / 512 / 3858; the second launched with programmatic stream serialisation 272 / 474 / 3900; this grid
// 278 / 475 / 3470; the two kinds interleaved block by block 380 / 676 / 5060 (an SM that alternates between the two
// bodies runs both much slower).
__global__ void __launch_bounds__(kThreads, 1)
bwd_grads_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ CUtensorMap tm_q64, const __grid_constant__ CUtensorMap tm_do64, const Params p,
                 const unsigned blocks_kv) {
    if (blockIdx.x < blocks_kv)
        bwd_dkdv_block(&tm_q64, &tm_k, &tm_v, &tm_do64, p, blockIdx.x);
    else
        bwd_dq_block(&tm_q, &tm_k, &tm_v, &tm_do, p, blockIdx.x - blocks_kv);
}
constexpr int kGradsSmemBytes = dq::kSmemBytes > dkdv::kSmemBytes ? dq::kSmemBytes : dkdv::kSmemBytes;

// Sum of the head splits' fp32 partials -> bf16 dV and dK (fixed order: deterministic).  4 elements per thread.
__global__ void __launch_bounds__(256) bwd_reduce_kernel(const float* __restrict__ partial, int splits,
                                                         long long tensor_elems, __nv_bfloat16* __restrict__ dv,
                                                         __nv_bfloat16* __restrict__ dk) {
    const long long i4 = (blockIdx.x * 256LL + threadIdx.x) * 4;
    if (i4 >= 2 * tensor_elems) return;
    const int which = i4 >= tensor_elems ? 1 : 0;
    const long long off = i4 - which * tensor_elems;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
        const float4 x = *reinterpret_cast<const float4*>(partial + (s * 2LL + which) * tensor_elems + off);
        acc.x += x.x;
        acc.y += x.y;
        acc.z += x.z;
        acc.w += x.w;
    }
    uint2 pk;
    pk.x = pack_bf16x2(acc.x, acc.y);
    pk.y = pack_bf16x2(acc.z, acc.w);
    *reinterpret_cast<uint2*>((which ? dk : dv) + off) = pk;
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
// With few kv heads and a short sequence there are too few (kv head, kv tile) blocks to fill the GPU; the query
// heads of a group are then divided among `splits` blocks (a divisor of G) whose fp32 partials are summed.  One dK/dV
// block per SM is enough: the dQ blocks of the same grid fill whatever the dK/dV blocks leave uneven, and every
// further split costs a block start-up and 128 KB of partials (upstream's shape: 8 splits 252 us per call, 16 splits
// 274 us).
static int choose_head_splits(int G, long long kv_blocks, int sm_count) {
    int splits = 1;
    for (int d = 1; d <= G; ++d) {
        if (G % d != 0) continue;
        splits = d;
        if (kv_blocks * d >= sm_count) break;
    }
    return splits;
}

static size_t delta_bytes(int B, int Sq, int Hq) {
    return (static_cast<size_t>(B) * Hq * Sq * sizeof(float) + 255) / 256 * 256;
}

static size_t workspace_bytes(int B, int Sq, int Skv, int Hq, int Hkv, int sm_count) {
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return 0;
    const long long kv_blocks = static_cast<long long>(B) * Hkv * ((Skv + kBN - 1) / kBN);
    const int splits = choose_head_splits(Hq / Hkv, kv_blocks, sm_count);
    size_t bytes = delta_bytes(B, Sq, Hq);
    if (splits > 1) bytes += static_cast<size_t>(splits) * 2 * B * Hkv * Skv * kD * sizeof(float);
    return bytes;
}

static int launch(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* grad_o,
                  float scale, int causal, int window, void* grad_q, void* grad_k, void* grad_v, void* workspace,
                  size_t workspace_size, int B, int Sq, int Skv, int Hq, int Hkv, int D, cudaStream_t stream) {
    if (window < 0) return CLLO_E_BAD_ARG;
    if (!q || !k || !v || !o || !lse || !grad_o || !grad_q || !grad_k || !grad_v) return CLLO_E_BAD_ARG;
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) return CLLO_E_BAD_ARG;
    if (Hq % Hkv != 0) return CLLO_E_BAD_ARG;
    const void* ptrs[] = {q, k, v, o, grad_o, grad_q, grad_k, grad_v};
    for (const void* ptr : ptrs)
        if (!aligned_to(ptr, 16)) return CLLO_E_BAD_ARG;
    if (D != kD) return CLLO_E_UNSUPPORTED;
    DeviceInfo* di = nullptr;
    int rc = current_device_info(&di);
    if (rc != CLLO_OK) return rc;
    if (di->cc_major != 10) return CLLO_E_UNSUPPORTED;
    if (!workspace || workspace_size < workspace_bytes(B, Sq, Skv, Hq, Hkv, di->sm_count) || !aligned_to(workspace, 256))
        return CLLO_E_WORKSPACE;

    Params p;
    p.lse = lse;
    p.delta = static_cast<const float*>(workspace);
    p.dq = static_cast<__nv_bfloat16*>(grad_q);
    p.dk = static_cast<__nv_bfloat16*>(grad_k);
    p.dv = static_cast<__nv_bfloat16*>(grad_v);
    p.scale = scale;
    p.B = B;
    p.Sq = Sq;
    p.Skv = Skv;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = Hq / Hkv;
    p.causal = (causal || window > 0) ? 1 : 0;
    p.window = window;
    p.n_qt = (Sq + kBM - 1) / kBM;
    p.n_kt = (Skv + kBN - 1) / kBN;
    const long long rows = static_cast<long long>(B) * Hq * Sq;
    const long long blocks_dq = static_cast<long long>(B) * Hq * p.n_qt;
    const long long kv_tiles = static_cast<long long>(B) * Hkv * p.n_kt;
    p.head_splits = choose_head_splits(p.G, kv_tiles, di->sm_count);
    p.dkv_partial = p.head_splits > 1
                        ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + delta_bytes(B, Sq, Hq))
                        : nullptr;
    const long long blocks_kv = kv_tiles * p.head_splits;
    // every grid size is checked before the first launch, so a refused call has written nothing
    const long long tensor_elems = static_cast<long long>(B) * Hkv * Skv * kD;
    const long long blocks_reduce = (2 * tensor_elems / 4 + 255) / 256;
    if (blocks_dq + blocks_kv > 0x7fffffffLL || (rows + 7) / 8 > 0x7fffffffLL ||
        (p.head_splits > 1 && blocks_reduce > 0x7fffffffLL))
        return CLLO_E_UNSUPPORTED;

    CUtensorMap tm_q, tm_k, tm_v, tm_do, tm_q64, tm_do64;  // the dK/dV kernel takes Q and dO in 64-row tiles
    if ((rc = prefill::encode_bhsd_map(&tm_q, q, B, Hq, Sq)) != CLLO_OK) return rc;
    if ((rc = prefill::encode_bhsd_map(&tm_k, k, B, Hkv, Skv)) != CLLO_OK) return rc;
    if ((rc = prefill::encode_bhsd_map(&tm_v, v, B, Hkv, Skv)) != CLLO_OK) return rc;
    if ((rc = prefill::encode_bhsd_map(&tm_do, grad_o, B, Hq, Sq)) != CLLO_OK) return rc;
    if ((rc = prefill::encode_bhsd_map(&tm_q64, q, B, Hq, Sq, dkdv::kBQ)) != CLLO_OK) return rc;
    if ((rc = prefill::encode_bhsd_map(&tm_do64, grad_o, B, Hq, Sq, dkdv::kBQ)) != CLLO_OK) return rc;

    if (!di->backward_attr_set) {
        CLLO_CUDA_TRY(cudaFuncSetAttribute(bwd_grads_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGradsSmemBytes));
        di->backward_attr_set = true;
    }
    bwd_delta_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(grad_o), static_cast<float*>(workspace),
        rows);
    CLLO_CUDA_TRY(cudaGetLastError());
    bwd_grads_kernel<<<static_cast<unsigned>(blocks_kv + blocks_dq), kThreads, kGradsSmemBytes, stream>>>(
        tm_q, tm_k, tm_v, tm_do, tm_q64, tm_do64, p, static_cast<unsigned>(blocks_kv));
    CLLO_CUDA_TRY(cudaGetLastError());
    if (p.head_splits > 1) {
        bwd_reduce_kernel<<<static_cast<unsigned>(blocks_reduce), 256, 0, stream>>>(p.dkv_partial, p.head_splits, tensor_elems,
                                                                            p.dv, p.dk);
        CLLO_CUDA_TRY(cudaGetLastError());
    }
    return CLLO_OK;
}

}  // namespace backward
}  // namespace cllo
