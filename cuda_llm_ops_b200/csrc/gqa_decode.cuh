// Split-KV single-token GQA decode for sm_100a.
//
// Work decomposition.  A "unit" is one (batch, kv head, block of <=16 query heads).  Its KV range
// is cut into tiles of 64 tokens; all tiles of all units form one flat index space that is divided
// evenly (to within one tile) among W persistent thread blocks ("workers"), so every SM streams the
// same number of bytes whatever the batch / head counts are.  A worker therefore processes a few
// whole units plus at most one partial unit at each end of its range.
//
// Inside a worker.  One producer warp issues TMA tile loads (K and V, 64 tokens x 128 dims each,
// 128-byte swizzled, 32 KB per stage) into a 6-stage ring guarded by full/empty mbarriers.  The eight
// consumer warps form two groups of four; the groups take stages alternately and the four warps of a
// group split a stage's 64 tokens 16 apiece, so a stage is held for a quarter of the time one warp
// would need and goes back to the producer (and to the memory system) sooner.  For ITS 16 tokens and
// ALL query heads of the unit (padded to 16 rows) a warp computes S = Q K^T with mma.sync m16n8k16
// (K fragments via ldmatrix), an online-softmax update of its private running (m, l, O) with quad
// shuffles (O is rescaled only when a maximum actually grew), and O += P V (V fragments via
// ldmatrix.trans, P fed straight from the accumulator registers).  There is no block-wide barrier in
// the streaming loop.  At the end of a unit the eight private states are merged through shared memory
// (log-sum-exp algebra, fixed summation order) and every warp writes its share of either the final
// bf16 output (unit entirely inside this worker) or an fp32 partial (O, m, l) in the workspace.
//
// Second pass, inside the same kernel.  A unit that a worker boundary cut leaves one fp32 partial per worker;
// every worker counts itself in on the unit's arrival counter (after a fence) and the LAST one to arrive merges
// all pieces, always in worker order:  m* = max m_i,  O = sum e^(m_i-m*) O_i / sum e^(m_i-m*) l_i.
// No block ever waits for another one, so any number of workers is safe, and there is no second launch.
//
// Position-sharded mode (kSharded): the KV range of this call is one GPU's share of a longer sequence.  The block
// that holds a unit's merged rows publishes them to every peer GPU and merges the peers' rows of the same unit
// (gqa_shard.cuh), so the exchange of the early units overlaps the decode of the late ones and a whole step of a
// sharded decode is this one kernel.
//
// HBM traffic per launch = K + V once (+ Q, O, and ~1% for partials): the algorithmic minimum.
#pragma once

#include "common.cuh"
#include "gqa_shard.cuh"
#include "host_util.cuh"
#include "rope.cuh"

namespace cllo {
namespace decode {

constexpr int kD = 128;
constexpr int kTok = 64;                     // tokens per stage
#ifndef CLLO_DECODE_STAGES
#define CLLO_DECODE_STAGES 6
#endif
constexpr int kStages = CLLO_DECODE_STAGES;
constexpr int kGroups = 2;                   // consumer groups; kStages must be a multiple of it so that a
                                             // stage buffer is always drained by the same group, in order
constexpr int kWarpsPerGroup = 4;
constexpr int kSubTok = kTok / kWarpsPerGroup;  // tokens per warp per stage
constexpr int kConsumerWarps = kGroups * kWarpsPerGroup;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kHalfBytes = kTok * 128;       // [64 tokens][64 dims] bf16
constexpr int kStageBytes = 4 * kHalfBytes;  // K dims 0-63, K dims 64-127, V dims 0-63, V dims 64-127
constexpr int kStatFloats = kConsumerWarps * 4 * 32;    // per warp, per lane: m0, m1, l0, l1
constexpr int kXchgFloats = kConsumerWarps * 16 * 32;   // per warp, per lane: 16 of the 64 O values
constexpr int kRows = 16;                    // query-head rows per unit (MMA M)
constexpr int kPW = kD + 2;                  // packed partial row width
constexpr int kSlotFloats = kRows * kPW;     // one partial slot in the workspace
constexpr int kSmemStat = kStages * kStageBytes;
constexpr int kSmemXchg = kSmemStat + kStatFloats * 4;
constexpr int kSmemBar = kSmemXchg + kXchgFloats * 4;
constexpr int kSmemBytes = kSmemBar + 2 * kStages * 8 + 16 + 1024;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
static_assert(kStages % kGroups == 0, "a stage buffer must always belong to the same consumer group");
static_assert(kSubTok == 16, "one PV k-step per warp per stage");

struct Params {
    const __nv_bfloat16* q;
    __nv_bfloat16* o;
    float* partial_out;  // nullable
    float* ws;           // [W][2][16][D+2] partial slots
    unsigned* counters;  // [W] arrival counters, zero at kernel start and again at its end
    float scale_log2;    // scale * log2(e)
    int B, S, Hq, Hkv, G, n_gblk, n_t, kv_layout, W;
    long long T;  // total tiles
};

// Decode step with the rotary embedding and the cache append folded in (kRope): the new token's query is rotated as
// its fragments are loaded, and the worker that owns the last KV tile of a (batch, kv head) unit puts the rotated new
// key and the new value into that tile in shared memory -- and into the cache in global memory for later steps --
// before it uses the tile.  A separate rotary pass over Q and K and a separate append kernel disappear from the step.
struct RopeParams {
    const __nv_bfloat16* k_new;  // [B,Hkv,D] un-rotated key of the new token
    const __nv_bfloat16* v_new;  // [B,Hkv,D]
    __nv_bfloat16* k_cache;      // the K/V the tensor maps read; row S-1 of every (batch, kv head) is written here
    __nv_bfloat16* v_cache;
    const int* positions;        // nullable, [B]: rotary position of the new token; default S-1
    long long batch_stride, head_stride, tok_stride;  // of the caches, in elements
    float inv_freq[kD / 2];
};

__host__ __device__ __forceinline__ long long worker_lo(long long w, long long T, long long W) {
    return (w * T) / W;
}
// the worker whose range [worker_lo(w), worker_lo(w+1)) holds tile t
__host__ __device__ __forceinline__ long long worker_of_tile(long long t, long long T, long long W) {
    return ((t + 1) * W - 1) / T;
}

template <bool kSharded, bool kRope>
__global__ void __launch_bounds__(kThreads, 1)
decode_splitkv_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const Params p, const shard::Params sp, const RopeParams rp) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t stage_base = base;
    float* stat = reinterpret_cast<float*>(gen_base + kSmemStat);
    float* xchg = reinterpret_cast<float*>(gen_base + kSmemXchg);
    const uint32_t bar_base = base + kSmemBar;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + kSmemBar + 2 * kStages * 8);
    volatile int* misc = abort_flag + 1;  // [0] this block merges the unit, [1] step number (sharded mode, set once)
    auto full_bar = [&](int s) { return bar_base + s * 8; };
    auto empty_bar = [&](int s) { return bar_base + (kStages + s) * 8; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = blockIdx.x;
    const long long lo = worker_lo(w, p.T, p.W), hi = worker_lo(w + 1, p.T, p.W);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), kWarpsPerGroup);
        }
        *abort_flag = 0;
        if (kSharded) misc[1] = static_cast<int>(shard::read_epoch(sp));
        fence_mbar_init();
    }
    __syncthreads();
    if (lo >= hi) return;

    if (warp == kConsumerWarps) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            // all indices advance incrementally: this one thread paces the whole block, so its loop carries
            // no division
            long long u = lo / p.n_t;
            int tile_in_unit = static_cast<int>(lo - u * p.n_t);
            int gblk = static_cast<int>(u % p.n_gblk);
            int kvh = static_cast<int>((u / p.n_gblk) % p.Hkv);
            int b = static_cast<int>(u / (static_cast<long long>(p.n_gblk) * p.Hkv));
            int slot = 0;
            uint32_t phase = 0;
            const int n_tiles = static_cast<int>(hi - lo);
            const bool bshd = p.kv_layout == CLLO_KV_BSHD;
#pragma unroll 1
            for (int it = 0; it < n_tiles; ++it) {
                mbar_wait(empty_bar(slot), phase ^ 1u, abort_flag, SITE_DECODE_EMPTY, slot);
                const int s0 = tile_in_unit * kTok;
                const int c1 = bshd ? kvh : s0;
                const int c2 = bshd ? s0 : kvh;
                const uint32_t dst = stage_base + slot * kStageBytes;
                mbar_arrive_expect_tx(full_bar(slot), kStageBytes);
                tma_load_4d(dst, &tm_k, full_bar(slot), 0, c1, c2, b);
                tma_load_4d(dst + kHalfBytes, &tm_k, full_bar(slot), 64, c1, c2, b);
                tma_load_4d(dst + 2 * kHalfBytes, &tm_v, full_bar(slot), 0, c1, c2, b);
                tma_load_4d(dst + 3 * kHalfBytes, &tm_v, full_bar(slot), 64, c1, c2, b);
                if (++slot == kStages) {
                    slot = 0;
                    phase ^= 1u;
                }
                if (++tile_in_unit == p.n_t) {
                    tile_in_unit = 0;
                    if (++gblk == p.n_gblk) {
                        gblk = 0;
                        if (++kvh == p.Hkv) {
                            kvh = 0;
                            ++b;
                        }
                    }
                }
            }
            if (*abort_flag) {
                // a wait gave up somewhere: make sure no copy is still landing when the block retires
                const long long n = hi - lo;
                for (long long it = (n > kStages ? n - kStages : 0); it < n; ++it) {
                    const int slot = static_cast<int>(it % kStages);
                    const uint32_t use = static_cast<uint32_t>(it / kStages);
                    const long long t0 = clock64();
                    while (!mbar_try_wait(full_bar(slot), use & 1u)) {
                        if (clock64() - t0 > kWaitLimitCycles / 64) {
                            record_timeout(SITE_DECODE_DRAIN, slot);
                            break;
                        }
                    }
                }
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int g = lane >> 2, tig = lane & 3;
    const int grp = warp / kWarpsPerGroup, sub = warp % kWarpsPerGroup;
    const long long u_first = lo / p.n_t, u_last = (hi - 1) / p.n_t;

#pragma unroll 1
    for (long long u = u_first; u <= u_last; ++u) {
        const long long unit_lo = u * p.n_t, unit_hi = unit_lo + p.n_t;
        const long long seg_lo = lo > unit_lo ? lo : unit_lo;
        const long long seg_hi = hi < unit_hi ? hi : unit_hi;
        const int gblk = static_cast<int>(u % p.n_gblk);
        const int kvh = static_cast<int>((u / p.n_gblk) % p.Hkv);
        const int b = static_cast<int>(u / (static_cast<long long>(p.n_gblk) * p.Hkv));
        const int rows = (p.G - gblk * kRows) < kRows ? (p.G - gblk * kRows) : kRows;
        const long long head0 = static_cast<long long>(b) * p.Hq + static_cast<long long>(kvh) * p.G + gblk * kRows;

        // rotary table of this unit's batch element: (cos, sin) of position * inv_freq for the 64 pairs of a head.
        // It lives in the exchange buffer, which is idle until the end-of-unit merge (whose first barrier every warp
        // reaches only after it has finished reading the table).
        float2* rope_tab = reinterpret_cast<float2*>(xchg);
        if (kRope) {
            named_bar_sync(1, kConsumerWarps * 32);  // the previous unit's merge has finished with the buffer
            if (threadIdx.x < kD / 2) {
                const int pos = rp.positions ? rp.positions[b] : p.S - 1;
                float sn, cs;
                rope::sincos_accurate(static_cast<float>(pos) * rp.inv_freq[threadIdx.x], sn, cs);
                rope_tab[threadIdx.x] = make_float2(cs, sn);
            }
            named_bar_sync(1, kConsumerWarps * 32);
        }
        auto rotate_pair = [&](uint32_t w, int pair) {
            const float2 cs = rope_tab[pair];
            const float even = __uint_as_float(w << 16), odd = __uint_as_float(w & 0xffff0000u);
            return pack_bf16x2(even * cs.x - odd * cs.y, even * cs.y + odd * cs.x);
        };

        // Q fragments of this unit (A operand, rows = query heads of the group, zero padded)
        uint32_t qf[8][4];
        {
            const uint32_t* q0 = reinterpret_cast<const uint32_t*>(p.q + (head0 + g) * kD);
            const uint32_t* q1 = reinterpret_cast<const uint32_t*>(p.q + (head0 + g + 8) * kD);
            const bool v0 = g < rows, v1 = g + 8 < rows;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qf[ks][0] = v0 ? __ldg(q0 + ks * 8 + tig) : 0u;
                qf[ks][1] = v1 ? __ldg(q1 + ks * 8 + tig) : 0u;
                qf[ks][2] = v0 ? __ldg(q0 + ks * 8 + tig + 4) : 0u;
                qf[ks][3] = v1 ? __ldg(q1 + ks * 8 + tig + 4) : 0u;
                if (kRope) {  // a 32-bit word is one (even, odd) pair of the head dimension
                    qf[ks][0] = rotate_pair(qf[ks][0], ks * 8 + tig);
                    qf[ks][1] = rotate_pair(qf[ks][1], ks * 8 + tig);
                    qf[ks][2] = rotate_pair(qf[ks][2], ks * 8 + tig + 4);
                    qf[ks][3] = rotate_pair(qf[ks][3], ks * 8 + tig + 4);
                }
            }
        }

        float o[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        // this group's tiles of the segment: local index (t - lo) congruent to grp modulo kGroups
        const long long first = seg_lo + ((static_cast<long long>(grp) - (seg_lo - lo)) % kGroups + kGroups) % kGroups;
#pragma unroll 1
        for (long long t = first; t < seg_hi; t += kGroups) {
            const int it = static_cast<int>(t - lo);
            const int slot = it % kStages;
            const uint32_t use = static_cast<uint32_t>(it / kStages);
            mbar_wait(full_bar(slot), use & 1u, abort_flag, SITE_DECODE_FULL, slot);
            __syncwarp();
            const uint32_t kb = stage_base + slot * kStageBytes;
            const uint32_t vb = kb + 2 * kHalfBytes;
            const int tok0 = static_cast<int>(t - unit_lo) * kTok + sub * kSubTok;  // first token of this warp
            const int valid = p.S - tok0;  // tokens of this warp's 16 that exist (may be <= 0 or >= 16)

            if (kRope && valid > 0 && valid <= kSubTok) {
                // the new token (position S-1) is one of this warp's 16 rows, and only this warp reads them: put its
                // rotated key and its value into the tile (lane = 4 consecutive dims = 2 pairs), and into the cache
                const uint32_t srow = static_cast<uint32_t>(sub * kSubTok + valid - 1);
                const int d0 = lane * 4;
                const long long src = (static_cast<long long>(b) * p.Hkv + kvh) * kD + d0;
                uint2 kn = *reinterpret_cast<const uint2*>(rp.k_new + src);
                const uint2 vn = *reinterpret_cast<const uint2*>(rp.v_new + src);
                kn.x = rotate_pair(kn.x, lane * 2);
                kn.y = rotate_pair(kn.y, lane * 2 + 1);
                const uint32_t off = static_cast<uint32_t>(d0 >> 6) * kHalfBytes + srow * 128u +
                                     (((static_cast<uint32_t>(d0 & 63) >> 3) ^ (srow & 7u)) << 4) +
                                     static_cast<uint32_t>(d0 & 7) * 2u;
                asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(kb + off), "r"(kn.x), "r"(kn.y) : "memory");
                asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(vb + off), "r"(vn.x), "r"(vn.y) : "memory");
                if (gblk == 0) {
                    const long long dst = static_cast<long long>(b) * rp.batch_stride + kvh * rp.head_stride +
                                          static_cast<long long>(p.S - 1) * rp.tok_stride + d0;
                    *reinterpret_cast<uint2*>(rp.k_cache + dst) = kn;
                    *reinterpret_cast<uint2*>(rp.v_cache + dst) = vn;
                }
                __syncwarp();
            }

            if (valid > 0) {
                // ---- S = Q K^T  (16 heads x 16 tokens) ----
                float s[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
                    const uint32_t row_off = static_cast<uint32_t>(sub * kSubTok + nt * 8 + (lane & 7)) * 128u;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint32_t chunk = static_cast<uint32_t>((kk & 1) * 4 + (lane >> 3));
                        const uint32_t addr = kb + (kk >> 1) * kHalfBytes + row_off + ((chunk ^ (lane & 7)) << 4);
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(addr, b0, b1, b2, b3);
                        mma_bf16_16816(s[nt], qf[2 * kk], b0, b1);
                        mma_bf16_16816(s[nt], qf[2 * kk + 1], b2, b3);
                    }
                }

                // ---- online softmax on this warp's private state ----
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[nt][e] *= p.scale_log2;
                    if (valid < kSubTok) {
                        const int c = nt * 8 + tig * 2;
                        if (c >= valid) s[nt][0] = s[nt][2] = -INFINITY;
                        if (c + 1 >= valid) s[nt][1] = s[nt][3] = -INFINITY;
                    }
                    mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
                    mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
                if (__any_sync(0xffffffffu, (mn0 > m0) || (mn1 > m1))) {
                    // a maximum grew somewhere in the warp: bring O and l to the new reference
                    const float a0 = fast_exp2(m0 - mn0), a1 = fast_exp2(m1 - mn1);
                    l0 *= a0;
                    l1 *= a1;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        o[i][0] *= a0;
                        o[i][1] *= a0;
                        o[i][2] *= a1;
                        o[i][3] *= a1;
                    }
                    m0 = mn0;
                    m1 = mn1;
                }
                uint32_t pa[4];
                {
                    const float p00 = fast_exp2(s[0][0] - m0), p01 = fast_exp2(s[0][1] - m0);
                    const float p02 = fast_exp2(s[0][2] - m1), p03 = fast_exp2(s[0][3] - m1);
                    const float p10 = fast_exp2(s[1][0] - m0), p11 = fast_exp2(s[1][1] - m0);
                    const float p12 = fast_exp2(s[1][2] - m1), p13 = fast_exp2(s[1][3] - m1);
                    l0 += (p00 + p01) + (p10 + p11);
                    l1 += (p02 + p03) + (p12 + p13);
                    pa[0] = pack_bf16x2(p00, p01);
                    pa[1] = pack_bf16x2(p02, p03);
                    pa[2] = pack_bf16x2(p10, p11);
                    pa[3] = pack_bf16x2(p12, p13);
                }

                // ---- O += P V  (16 heads x 128 dims, one 16-token k-step) ----
                const uint32_t tok = static_cast<uint32_t>(sub * kSubTok + (lane & 7) + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int np = 0; np < 8; ++np) {
                    const uint32_t chunk = static_cast<uint32_t>((np & 3) * 2 + (lane >> 4));
                    const uint32_t addr = vb + (np >> 2) * kHalfBytes + tok * 128u + ((chunk ^ (tok & 7u)) << 4);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(addr, b0, b1, b2, b3);
                    mma_bf16_16816(o[2 * np], pa, b0, b1);
                    mma_bf16_16816(o[2 * np + 1], pa, b2, b3);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(slot));
        }

        // ---- merge the eight private states ----
        // 1. publish (m, l); everyone derives the common maximum, its own rescale factor and the total l
        stat[(warp * 4 + 0) * 32 + lane] = m0;
        stat[(warp * 4 + 1) * 32 + lane] = m1;
        stat[(warp * 4 + 2) * 32 + lane] = l0;
        stat[(warp * 4 + 3) * 32 + lane] = l1;
        named_bar_sync(1, kConsumerWarps * 32);
        float ms0 = -INFINITY, ms1 = -INFINITY;
#pragma unroll
        for (int sw = 0; sw < kConsumerWarps; ++sw) {
            ms0 = fmaxf(ms0, stat[(sw * 4 + 0) * 32 + lane]);
            ms1 = fmaxf(ms1, stat[(sw * 4 + 1) * 32 + lane]);
        }
        float lt0 = 0.f, lt1 = 0.f;
#pragma unroll
        for (int sw = 0; sw < kConsumerWarps; ++sw) {
            const float wm0 = stat[(sw * 4 + 0) * 32 + lane], wm1 = stat[(sw * 4 + 1) * 32 + lane];
            lt0 += (wm0 == -INFINITY) ? 0.f : stat[(sw * 4 + 2) * 32 + lane] * fast_exp2(wm0 - ms0);
            lt1 += (wm1 == -INFINITY) ? 0.f : stat[(sw * 4 + 3) * 32 + lane] * fast_exp2(wm1 - ms1);
        }
        lt0 += __shfl_xor_sync(0xffffffffu, lt0, 1);
        lt0 += __shfl_xor_sync(0xffffffffu, lt0, 2);
        lt1 += __shfl_xor_sync(0xffffffffu, lt1, 1);
        lt1 += __shfl_xor_sync(0xffffffffu, lt1, 2);
        const float f0 = (m0 == -INFINITY) ? 0.f : fast_exp2(m0 - ms0);
        const float f1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - ms1);
        // 2. four rounds; in each, every warp posts 16 of its 64 (rescaled) O values and then sums, over
        //    the eight warps in fixed order, the two values it owns.  Warp w ends up owning, for the row
        //    half (w & 1) and the n-tiles congruent to (w >> 1) modulo 4, the two columns of its lanes.
        float acc[4][2];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int idx = r * 16 + i;
                xchg[(warp * 16 + i) * 32 + lane] = o[idx >> 2][idx & 3] * ((idx & 2) ? f1 : f0);
            }
            named_bar_sync(1, kConsumerWarps * 32);
            float a = 0.f, c = 0.f;
#pragma unroll
            for (int sw = 0; sw < kConsumerWarps; ++sw) {
                a += xchg[(sw * 16 + 2 * warp) * 32 + lane];
                c += xchg[(sw * 16 + 2 * warp + 1) * 32 + lane];
            }
            acc[r][0] = a;
            acc[r][1] = c;
            named_bar_sync(1, kConsumerWarps * 32);
        }

        // ---- every warp writes its share ----
        const bool whole = (seg_lo == unit_lo) && (seg_hi == unit_hi);
        const bool direct = whole && !kSharded;  // nothing else to merge with: straight to the output
        {
            const int hrow = warp & 1;             // 0: row g, 1: row g + 8
            const int row = g + 8 * hrow;
            const float mrow = hrow ? ms1 : ms0;
            const float lrow = hrow ? lt1 : lt0;
            if (row < rows) {
                if (direct && p.partial_out == nullptr) {
                    const float inv = 1.f / lrow;
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int col = (r * 4 + (warp >> 1)) * 8 + tig * 2;
                        *reinterpret_cast<uint32_t*>(p.o + (head0 + row) * kD + col) =
                            pack_bf16x2(acc[r][0] * inv, acc[r][1] * inv);
                    }
                } else {
                    float* dst;
                    if (direct) {
                        dst = p.partial_out + (head0 + row) * kPW;
                    } else {
                        const int which = (u == u_first) ? 0 : 1;
                        dst = p.ws + (w * 2 + which) * kSlotFloats + row * kPW;
                    }
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int col = (r * 4 + (warp >> 1)) * 8 + tig * 2;
                        *reinterpret_cast<float2*>(dst + col) = make_float2(acc[r][0], acc[r][1]);
                    }
                    if (tig == 0 && (warp >> 1) == 0) {
                        dst[kD] = mrow * kLn2;
                        dst[kD + 1] = lrow;
                    }
                }
            }
        }
        if (direct) continue;

        // ---- this worker's piece of the unit is in the workspace: count it in; the last one to arrive merges ----
        const long long w_first = worker_of_tile(unit_lo, p.T, p.W), w_last = worker_of_tile(unit_hi - 1, p.T, p.W);
        const int n_pieces = static_cast<int>(w_last - w_first) + 1;
        unsigned* counter = p.counters + w_first;
        // the barrier orders every thread's stores before thread 0's fence, which is cumulative: whoever sees the
        // count sees the piece
        named_bar_sync(1, kConsumerWarps * 32);
        if (threadIdx.x == 0) {
            bool last = n_pieces == 1;
            if (!last) {
                __threadfence();
                last = atomicAdd(counter, 1u) == static_cast<unsigned>(n_pieces - 1);
                __threadfence();
                if (last) *counter = 0u;  // the counters are zero again when the kernel ends
            }
            misc[0] = last ? 1 : 0;
        }
        named_bar_sync(1, kConsumerWarps * 32);
        if (misc[0] == 0) continue;
        {
            const int tid = threadIdx.x, mrow_i = tid >> 4, c8 = (tid & 15) * 8;
            const int which_first = (worker_lo(w_first, p.T, p.W) == unit_lo) ? 0 : 1;
            float mg[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, mm = -INFINITY, ll = 0.f;
            if (mrow_i < rows) {
                auto piece = [&](int i) {
                    return p.ws + ((w_first + i) * 2 + (i == 0 ? which_first : 0)) * kSlotFloats + mrow_i * kPW;
                };
                if (n_pieces <= 4)
                    shard::merge_rows<4>(n_pieces, c8, piece, mg, mm, ll);
                else
                    shard::merge_rows<8>(n_pieces, c8, piece, mg, mm, ll);
            }
            if (kSharded) {
                shard::publish_wait_combine(sp, static_cast<unsigned>(misc[1]), 1, tid, u, head0, rows, mg, mm, ll, p.o);
            } else if (mrow_i < rows) {
                if (p.partial_out)
                    shard::store_packed_row(p.partial_out + (head0 + mrow_i) * kPW, c8, mg, mm, ll);
                else
                    shard::store_bf16_row(p.o + (head0 + mrow_i) * kD, c8, mg, ll);
            }
        }
    }
}

// Public merge of caller-provided partials [nsplit][rows][D+2] -> bf16 [rows][D] (and, when asked, the rows'
// log-sum-exp m + log l in natural-log units).  One warp per row (lane = 4 columns), eight rows per block.
constexpr int kCombineRows = 8;
__global__ void __launch_bounds__(kCombineRows * 32) combine_rows_kernel(const float* __restrict__ partials, int nsplit,
                                                                         long long rows, __nv_bfloat16* __restrict__ o,
                                                                         float* __restrict__ lse) {
    const long long r = static_cast<long long>(blockIdx.x) * kCombineRows + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int c4 = (threadIdx.x & 31) * 4;
    float mstar = -INFINITY;
    for (int i = 0; i < nsplit; ++i) {
        const float2 ml = *reinterpret_cast<const float2*>(partials + (static_cast<long long>(i) * rows + r) * kPW + kD);
        if (ml.y > 0.f) mstar = fmaxf(mstar, ml.x);
    }
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, lsum = 0.f;
    for (int i = 0; i < nsplit; ++i) {
        const float* row = partials + (static_cast<long long>(i) * rows + r) * kPW;
        const float2 ml = *reinterpret_cast<const float2*>(row + kD);
        const float wgt = ml.y > 0.f ? __expf(ml.x - mstar) : 0.f;
        const float2 x = *reinterpret_cast<const float2*>(row + c4);
        const float2 y = *reinterpret_cast<const float2*>(row + c4 + 2);
        a0 += wgt * x.x;
        a1 += wgt * x.y;
        a2 += wgt * y.x;
        a3 += wgt * y.y;
        lsum += wgt * ml.y;
    }
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    uint2 pk;
    pk.x = pack_bf16x2(a0 * inv, a1 * inv);
    pk.y = pack_bf16x2(a2 * inv, a3 * inv);
    *reinterpret_cast<uint2*>(o + r * kD + c4) = pk;
    if (lse && c4 == 0) lse[r] = lsum > 0.f ? mstar + logf(lsum) : -INFINITY;
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
// Workspace layout: kFixedCounters arrival counters at the very start -- a fixed place, so that a workspace that
// serves calls with different worker counts keeps its counters apart from its partial slots -- then the slots; a
// call with more workers than that keeps its counters behind the slots instead.
constexpr int kFixedCounters = 1024;
constexpr size_t kSlotOffsetBytes = kFixedCounters * sizeof(unsigned);

struct Plan {
    Params prm;
    size_t ws_bytes;        // arrival counters + partial slots
    size_t slot_offset;     // byte offset of the partial slots inside the workspace
    size_t counter_offset;  // byte offset of the counters
    size_t counter_bytes;
    bool counters_fixed;    // the counters sit in the fixed area at the start
    bool needs_merge;       // some unit is cut by a worker boundary
    long long units;
};

// How many persistent blocks to launch when the caller leaves the choice to the library.  Measured on B200
// (148 SMs, six 32 KB stages per block): the memory system is saturated from about 0.7 x SMs blocks on, and more
// than about 0.87 x SMs blocks (768 stages in flight) cost 3-7 % again; within that window a count that cuts no
// unit (whole units per worker: no partials, no merge) or, failing that, cuts every unit in the same places (the
// workers of different kv heads then walk the same token positions together, and with K/V [B,S,Hkv,D] those are
// the same DRAM rows) is another ~5 % faster than an arbitrary one.
static long long choose_workers(long long T, long long units, int sm_count) {
    long long hi = (static_cast<long long>(sm_count) * 173) / 200;
    if (hi < 1) hi = 1;
    if (T <= hi) return T;
    long long lo = (static_cast<long long>(sm_count) * 7) / 10;
    if (lo < 1) lo = 1;
    for (long long W = hi; W >= lo; --W)
        if (units % W == 0) return W;
    for (long long W = hi; W >= lo; --W)
        if (W % units == 0) return W;
    return hi;
}

static int make_plan(int B, int S, int Hq, int Hkv, int D, int num_workers, int sm_count, Plan* plan) {
    if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || num_workers < 0) return CLLO_E_BAD_ARG;
    if (Hq % Hkv != 0) return CLLO_E_BAD_ARG;
    if (D != kD) return CLLO_E_UNSUPPORTED;
    Params& p = plan->prm;
    p.B = B;
    p.S = S;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = Hq / Hkv;
    p.n_gblk = (p.G + kRows - 1) / kRows;
    p.n_t = (S + kTok - 1) / kTok;
    plan->units = static_cast<long long>(B) * Hkv * p.n_gblk;
    if (plan->units * kRows > 0x7fffffffLL) return CLLO_E_UNSUPPORTED;
    p.T = plan->units * p.n_t;
    long long W = num_workers > 0 ? num_workers : choose_workers(p.T, plan->units, sm_count);
    if (W > p.T) W = p.T;
    if (W < 1) W = 1;
    p.W = static_cast<int>(W);
    if (p.T / W + 1 > 0x7fffffffLL) return CLLO_E_UNSUPPORTED;  // a worker's tile count is a 32-bit loop index
    const size_t slot_bytes = static_cast<size_t>(W) * 2 * kSlotFloats * sizeof(float);
    plan->slot_offset = kSlotOffsetBytes;
    plan->counter_bytes = static_cast<size_t>(W) * sizeof(unsigned);
    plan->counters_fixed = W <= kFixedCounters;
    plan->counter_offset = plan->counters_fixed ? 0 : kSlotOffsetBytes + slot_bytes;
    plan->ws_bytes = kSlotOffsetBytes + slot_bytes + (plan->counters_fixed ? 0 : plan->counter_bytes);
    plan->needs_merge = false;
    for (long long w = 1; w < W; ++w)
        if (worker_lo(w, p.T, W) % p.n_t != 0) {
            plan->needs_merge = true;
            break;
        }
    return CLLO_OK;
}

// S_cap: the token capacity the cache was allocated with (>= S); rows [S, S_cap) are outside the map and read as zero
static int encode_kv_map(CUtensorMap* map, const void* base, int B, int S, int Hkv, int kv_layout, int S_cap) {
    const uint64_t row = static_cast<uint64_t>(kD) * 2;
    uint64_t dims[4], strides[3];
    uint32_t box[4];
    dims[0] = kD;
    box[0] = 64;
    if (kv_layout == CLLO_KV_BSHD) {  // (D, Hkv, S, B)
        dims[1] = static_cast<uint64_t>(Hkv);
        dims[2] = static_cast<uint64_t>(S);
        strides[0] = row;
        strides[1] = row * Hkv;
        box[1] = 1;
        box[2] = kTok;
    } else {  // (D, S, Hkv, B)
        dims[1] = static_cast<uint64_t>(S);
        dims[2] = static_cast<uint64_t>(Hkv);
        strides[0] = row;
        strides[1] = row * S_cap;
        box[1] = kTok;
        box[2] = 1;
    }
    dims[3] = static_cast<uint64_t>(B);
    strides[2] = row * static_cast<uint64_t>(S_cap) * Hkv;
    box[3] = 1;
    return encode_bf16_4d(map, base, dims, strides, box);
}

}  // namespace decode
}  // namespace cllo
