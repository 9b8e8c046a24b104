// MLA-shaped attention forward for sm_100a: head_dim_qk = 192, head_dim_v = 128 (tcgen05, tensor memory, TMA).
//
// Upstream: flash_mla_forward_bf16_kernel / launch_flash_mla_forward_bf16_kernel,
// src/python/Triton/flash_mla_kernel.py:16-268,315-508 (same attention as the GQA forward with a wider Q/K head).
//
// The GQA forward kernel (gqa_prefill.cuh) keeps two 128-row query tiles per block; with 192-wide Q and K that
// no longer fits shared memory (2 Q tiles + 2 K stages + 2 V stages = 256 KB).  Here a block owns ONE 128-row
// query tile and pipelines over the kv tiles instead, which tensor memory allows once S and P have two homes each:
//     tensor memory (512 columns): C0 (128) | C1 (128) | P0 (64) | P1 (64) | O (128)
//     S(j) = Q K(j)^T lands in C[j % 2] (12 MMAs M128 N128 K16 at a 192-wide head, Q and K K-major from shared memory); the 128 softmax
//     threads copy it to registers at once and hand the region back, so S(j+2) can follow while softmax(j) and
//     softmax(j+1) run; P(j) goes to P[j % 2] as bf16 and O += P(j) V(j) (8 MMAs, A from tensor memory, V MN-major)
//     has until softmax(j+2) wants that region again.
// Shared memory: Q 48 KB (three [128][64] slabs, 128-byte swizzle), K 2 x 48 KB, V 2 x 32 KB.
// The kernel is a template on the Q/K head width; the 128-wide instance serves the GQA forward when all query rows fit
// one tile (Sq <= 128: decode-like chunks), where the two-tile kernel would spend half its work on an empty tile.
// Query chunks of at most 64 rows go further: the heads of a group read the same K/V, so 128 / rows of them share the
// tile (the Q and O tensor maps take a box of rows x heads, whose dense image in shared memory is the same [128][64]
// slab; a thread's row maps to (head, query row) by a shift and a mask).
// Warps: 0-3 softmax (one query row per thread), 4 TMA producer, 5 MMA issuer, 6-7 idle.  Barrier conventions,
// bounded waits and the status word are those of the GQA forward kernel; so are the lazy rescaling, the packed
// fp32 arithmetic and the bulk-store epilogue.
#pragma once

#include "gqa_prefill.cuh"

namespace cllo {
namespace mla {

using prefill::add2;
using prefill::fma2;
using prefill::kIdescPV;
using prefill::kIdescQK;
using prefill::kLn2;
using prefill::kLog2e;
using prefill::kRescaleThreshold;
using prefill::max3;
using prefill::min3;
using prefill::pk2;
using prefill::smem_desc_hi;
using prefill::smem_desc_lo;
using prefill::tc_commit;
using prefill::tc_fence_after;
using prefill::tc_fence_before;
using prefill::tc_mma_ss_lo;
using prefill::tc_mma_ts_lo;
using prefill::tmem_alloc;
using prefill::tmem_dealloc;
using prefill::tmem_ld128_wait;
using prefill::tmem_ld16_wait;
using prefill::tmem_ld32_wait;
using prefill::tmem_relinquish;
using prefill::tmem_st16;
using prefill::tmem_st32;
using prefill::tmem_wait_st;
using prefill::upk2;

constexpr int kDv = 128;
constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kThreads = 256;
constexpr int kSlabBytes = 128 * 128;              // [128 rows][64 dims] bf16, one swizzled slab
constexpr int kVBytes = 2 * kSlabBytes;
constexpr int kNumBars = 16;
// shared-memory map for a Q/K head width of kDqk (a multiple of 64): Q | K x 2 | V x 2 | barriers
template <int kDqk>
struct Smem {
    static constexpr int kSlabs = kDqk / 64;
    static constexpr int kQBytes = kSlabs * kSlabBytes;   // 48 KB at 192
    static constexpr int kKBytes = kSlabs * kSlabBytes;
    static constexpr int kQ = 0;
    static constexpr int kK = kQBytes;
    static constexpr int kV = kK + 2 * kKBytes;
    static constexpr int kBar = kV + 2 * kVBytes;         // 208 KB at 192, 160 KB at 128
    static constexpr int kBytes = kBar + kNumBars * 8 + 32 + 1024;
};
constexpr uint32_t kColC = 0, kColP = 256, kColO = 384;

enum : int {
    SITE_MLA_Q = 56, SITE_MLA_K = 57, SITE_MLA_V = 58, SITE_MLA_S = 59, SITE_MLA_P = 60, SITE_MLA_PV = 61,
    SITE_MLA_C = 62, SITE_MLA_DRAIN = 63,
};

struct Params {
    float* lse;  // nullable
    float scale_log2;
    int B, Sq, Skv, Hq, Hkv, G, causal, n_qt;
    // short query chunks of a group share a tile: the 128 rows are `pack` heads x 2^row_shift query rows (1 x 128 otherwise)
    int pack, row_shift, packs_per_group;
};

template <int kDqk>
__global__ void __launch_bounds__(kThreads, 1)
mla_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    using L = Smem<kDqk>;
    constexpr int kSmemQ = L::kQ, kSmemK = L::kK, kSmemV = L::kV, kSmemBar = L::kBar;
    constexpr int kQBytes = L::kQBytes, kKBytes = L::kKBytes, kSlabs = L::kSlabs;
    const uint32_t bar0 = base + kSmemBar;
    const uint32_t bar_q_full = bar0;
    auto bar_k_full = [&](int s) { return bar0 + 8 * (1 + s); };
    auto bar_v_full = [&](int s) { return bar0 + 8 * (3 + s); };
    auto bar_s_full = [&](int s) { return bar0 + 8 * (5 + s); };    // S landed in C[s]; also: the K tile it read is free
    auto bar_p_full = [&](int s) { return bar0 + 8 * (7 + s); };    // P[s] stored
    auto bar_pv_done = [&](int s) { return bar0 + 8 * (9 + s); };   // O += P[s] V retired: P[s] and the V stage are free
    auto bar_c_free = [&](int s) { return bar0 + 8 * (11 + s); };   // C[s] copied to registers
    const uint32_t bar_drain = bar0 + 8 * 13;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + kSmemBar + kNumBars * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + kSmemBar + kNumBars * 8 + 8);
    // warp index through a shuffle: the compiler then knows it to be the same in every lane
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

    // block -> (batch, kv head, query tile, head in group); heads of one group are neighbours so that they stream
    // the same K/V tiles through L2 together; heavy (late) causal tiles go first
    long long id = blockIdx.x;
    const int g = static_cast<int>(id % p.packs_per_group);
    id /= p.packs_per_group;
    const int qt = p.n_qt - 1 - static_cast<int>(id % p.n_qt);
    id /= p.n_qt;
    const int kvh = static_cast<int>(id % p.Hkv);
    const int b = static_cast<int>(id / p.Hkv);
    const int h = kvh * p.G + g * p.pack;  // first (or only) head of the tile
    const int q0 = qt * kBM;
    const int rows_used = p.pack << p.row_shift;  // 128 unless a small group leaves part of a packed tile empty
    int n_kv = (p.Skv + kBN - 1) / kBN;
    if (p.causal) {
        const int lim = (q0 + kBM - 1) / kBN + 1;
        n_kv = lim < n_kv ? lim : n_kv;
    }

    auto load_k = [&](int j) {
        const int s = j & 1;
        mbar_arrive_expect_tx(bar_k_full(s), kKBytes);
        for (int d = 0; d < kSlabs; ++d)
            tma_load_4d(base + kSmemK + s * kKBytes + d * kSlabBytes, &tm_k, bar_k_full(s), d * 64, j * kBN, kvh, b);
    };
    auto load_v = [&](int j) {
        const int s = j & 1;
        mbar_arrive_expect_tx(bar_v_full(s), kVBytes);
        for (int d = 0; d < 2; ++d)
            tma_load_4d(base + kSmemV + s * kVBytes + d * kSlabBytes, &tm_v, bar_v_full(s), d * 64, j * kBN, kvh, b);
    };

    if (warp == 4 && lane == 0) {
        mbar_init(bar_q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_k_full(s), 1);
            mbar_init(bar_v_full(s), 1);
            mbar_init(bar_s_full(s), 1);
            mbar_init(bar_p_full(s), kBM);
            mbar_init(bar_pv_done(s), 1);
            mbar_init(bar_c_free(s), kBM);
        }
        mbar_init(bar_drain, 1);
        *abort_flag = 0;
        fence_mbar_init();
        // the first copies start before the block has met at its first barrier
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        mbar_arrive_expect_tx(bar_q_full, static_cast<uint32_t>(kSlabs * rows_used * 128));
        for (int d = 0; d < kSlabs; ++d)
            tma_load_4d(base + kSmemQ + d * kSlabBytes, &tm_q, bar_q_full, d * 64, q0, h, b);
        load_k(0);
        load_v(0);
        if (n_kv > 1) load_k(1);
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    if (warp < 4 && static_cast<int>(threadIdx.x) >= rows_used) {
        // rows of the Q tile that the copy does not fill: zeros, so that their scores stay finite
        for (int d = 0; d < kSlabs; ++d)
            for (int c = 0; c < 8; ++c)
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(base + kSmemQ + d * kSlabBytes +
                                                                                static_cast<int>(threadIdx.x) * 128 + c * 16),
                             "r"(0)
                             : "memory");
        fence_async_proxy();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tm_o);
            // K runs one tile ahead of V: K(j+1) is wanted by S(j+1), issued a whole softmax before O += P(j) V(j)
            for (int j = 1; j < n_kv; ++j) {
                if (j + 1 < n_kv) {
                    // stage (j+1) % 2 held K(j-1): free once S(j-1) has retired
                    mbar_wait(bar_s_full((j + 1) & 1), static_cast<uint32_t>((j - 1) >> 1) & 1u, abort_flag, SITE_MLA_K, j);
                    load_k(j + 1);
                }
                if (j >= 2)  // stage j % 2 held V(j-2): free once O += P(j-2) V(j-2) has retired
                    mbar_wait(bar_pv_done(j & 1), static_cast<uint32_t>((j - 2) >> 1) & 1u, abort_flag, SITE_MLA_V, j);
                load_v(j);
            }
            if (*abort_flag) {
                // a wait gave up somewhere: let the copies already issued land before the block retires
                for (int j = (n_kv > 2 ? n_kv - 2 : 0); j < n_kv; ++j) {
                    const long long t0 = clock64();
                    while (!(mbar_try_wait(bar_k_full(j & 1), static_cast<uint32_t>(j >> 1) & 1u) &&
                             mbar_try_wait(bar_v_full(j & 1), static_cast<uint32_t>(j >> 1) & 1u)) &&
                           clock64() - t0 < kWaitLimitCycles / 64) {
                    }
                }
            }
        }
    } else if (warp == 5) {
        // -------------------------------- MMA issuer --------------------------------
        // Lane 0 issues every tcgen05.mma; per kv step one run of 8 + 12 MMAs with one look at the barriers before it
        // (the whole warp looks at once, one barrier per lane) -- see the GQA forward kernel for why.
        const uint32_t hi = smem_desc_hi(1024);
        const uint32_t q_lo = smem_desc_lo(base + kSmemQ, 16);
        const uint32_t k_lo0 = smem_desc_lo(base + kSmemK, 16), k_lo1 = smem_desc_lo(base + kSmemK + kKBytes, 16);
        const uint32_t v_lo0 = smem_desc_lo(base + kSmemV, kSlabBytes);
        const uint32_t v_lo1 = smem_desc_lo(base + kSmemV + kVBytes, kSlabBytes);
        auto issue_s = [&](int j) {  // S(j) -> C[j % 2]
            const uint32_t ka = (j & 1) ? k_lo1 : k_lo0;
            const uint32_t c = tmem_base + kColC + (j & 1) * kBN;
            tc_mma_ss_lo<false>(c, q_lo, ka, hi, kIdescQK);
#pragma unroll
            for (int ks = 1; ks < kDqk / 16; ++ks) {
                const uint32_t off = ((ks >> 2) * kSlabBytes + (ks & 3) * 32) >> 4;
                tc_mma_ss_lo<true>(c, q_lo + off, ka + off, hi, kIdescQK);
            }
        };
        // In the main loop the whole warp runs the issue code and the leader lane's predicate guards the MMAs, so
        // that the operands are warp-uniform values (see tc_mma_ss_lo_if).
        const uint32_t leader = lane == 0 ? 1u : 0u;
        auto issue_s_all = [&](int j) {  // S(j) -> C[j % 2]
            const uint32_t ka = (j & 1) ? k_lo1 : k_lo0;
            const uint32_t c = tmem_base + kColC + (j & 1) * kBN;
            prefill::tc_mma_ss_lo_if<false>(leader, c, q_lo, ka, hi, kIdescQK);
#pragma unroll
            for (int ks = 1; ks < kDqk / 16; ++ks) {
                const uint32_t off = ((ks >> 2) * kSlabBytes + (ks & 3) * 32) >> 4;
                prefill::tc_mma_ss_lo_if<true>(leader, c, q_lo + off, ka + off, hi, kIdescQK);
            }
        };
        auto issue_pv_all = [&](int j) {  // O += P[j % 2] V(j)
            const uint32_t va = (j & 1) ? v_lo1 : v_lo0;
            const uint32_t pa = tmem_base + kColP + (j & 1) * 64;
            const uint32_t oa = tmem_base + kColO;
            prefill::tc_mma_ts_lo_if(leader, oa, pa, va, hi, kIdescPV, j == 0 ? 0u : 1u);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks)
                prefill::tc_mma_ts_lo_if(leader, oa, pa + ks * 8, va + ks * (2048 >> 4), hi, kIdescPV, 1u);
        };
        if (lane == 0) {
            mbar_wait(bar_q_full, 0, abort_flag, SITE_MLA_Q, 0);
            for (int j = 0; j < 2 && j < n_kv; ++j) {
                mbar_wait(bar_k_full(j), 0, abort_flag, SITE_MLA_K, j);
                tc_fence_after();
                issue_s(j);
                tc_commit(bar_s_full(j));
            }
        }
        __syncwarp();
#pragma unroll 1
        for (int j = 0; j < n_kv; ++j) {
            const int s = j & 1;
            const uint32_t par = static_cast<uint32_t>(j >> 1) & 1u;
            const bool more = j + 2 < n_kv;
            // lane 0: P(j) stored; 1: V(j) arrived; 2: C[s] free (S(j) copied out); 3: K(j+2) arrived
            uint32_t my_bar = bar_p_full(s), my_par = par;
            int my_site = SITE_MLA_P;
            if (lane == 1) {
                my_bar = bar_v_full(s);
                my_site = SITE_MLA_V;
            } else if (lane == 2 && more) {
                my_bar = bar_c_free(s);
                my_site = SITE_MLA_C;
            } else if (lane == 3 && more) {
                my_bar = bar_k_full(s);
                my_par = static_cast<uint32_t>((j + 2) >> 1) & 1u;
                my_site = SITE_MLA_K;
            }
            if (!__all_sync(0xffffffffu, mbar_try_wait(my_bar, my_par))) {
                if (lane < 4) mbar_wait(my_bar, my_par, abort_flag, my_site, j);
                __syncwarp();
            }
            tc_fence_after();
            issue_pv_all(j);
            prefill::tc_commit_if(leader, bar_pv_done(s));
            if (more) {
                issue_s_all(j + 2);
                prefill::tc_commit_if(leader, bar_s_full(s));
            }
        }
        __syncwarp();
        if (lane == 0) {
            // everything issued must have retired before tensor memory is released
            tc_commit(bar_drain);
            mbar_wait(bar_drain, 0, abort_flag, SITE_MLA_DRAIN, 0);
            if (*abort_flag) {
                const long long t0 = clock64();
                while (!mbar_try_wait(bar_drain, 0) && clock64() - t0 < kWaitLimitCycles / 64) {
                }
            }
        }
    } else if (warp < 4) {
        // ------------------------- softmax + epilogue (one row per thread) -------------------------
        const int row_in_tile = warp * 32 + lane;
        const int qi = q0 + (row_in_tile & ((1 << p.row_shift) - 1));
        const int h_row = h + (row_in_tile >> p.row_shift);
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t o_addr = tmem_base + lane_base + kColO;
        float m = -INFINITY, l = 0.f;

#pragma unroll 1
        for (int j = 0; j < n_kv; ++j) {
            const int s = j & 1;
            const uint32_t par = static_cast<uint32_t>(j >> 1) & 1u;
            mbar_wait(bar_s_full(s), par, abort_flag, SITE_MLA_S, j);
            __syncwarp();
            tc_fence_after();
            float x[128];
            tmem_ld128_wait(tmem_base + lane_base + kColC + s * kBN, x);
            tc_fence_before();
            mbar_arrive(bar_c_free(s));  // the scores are in registers: C[s] may take S(j+2)

            // mask (diagonal / tail tiles only), then the row extreme of the RAW scores: the scale is folded into the
            // exponent argument below, y = s * c - m with m kept in scaled log2 units
            const bool neg = p.scale_log2 < 0.f;
            const int kv0 = j * kBN;
            const bool need_mask = (kv0 + kBN > p.Skv) || (p.causal && (kv0 + kBN - 1 > q0));
            if (need_mask) {
                int limit = p.Skv - 1 - kv0;
                if (p.causal) {
                    const int cl = qi - kv0;
                    limit = cl < limit ? cl : limit;
                }
                const float masked = neg ? INFINITY : -INFINITY;
#pragma unroll
                for (int c = 0; c < 128; ++c)
                    if (c > limit) x[c] = masked;
            }
            float e0 = neg ? INFINITY : -INFINITY, e1 = e0, e2 = e0, e3 = e0;
            if (neg) {
#pragma unroll
                for (int c = 0; c < 128; c += 8) {
                    e0 = min3(e0, x[c], x[c + 1]);
                    e1 = min3(e1, x[c + 2], x[c + 3]);
                    e2 = min3(e2, x[c + 4], x[c + 5]);
                    e3 = min3(e3, x[c + 6], x[c + 7]);
                }
            } else {
#pragma unroll
                for (int c = 0; c < 128; c += 8) {
                    e0 = max3(e0, x[c], x[c + 1]);
                    e1 = max3(e1, x[c + 2], x[c + 3]);
                    e2 = max3(e2, x[c + 4], x[c + 5]);
                    e3 = max3(e3, x[c + 6], x[c + 7]);
                }
            }
            e0 = neg ? fminf(e0, e1) : fmaxf(e0, e1);
            e2 = neg ? fminf(e2, e3) : fmaxf(e2, e3);
            const float mx = (neg ? fminf(e0, e2) : fmaxf(e0, e2)) * p.scale_log2;

            // raise the running maximum only when it pays (always on the first tile); O is rescaled in tensor memory,
            // which needs every earlier P V product retired
            float alpha = 1.f;
            const bool grow = (j == 0) || (mx > m + kRescaleThreshold);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = fmaxf(m, mx);
                if (j > 0) {
                    alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m - m_new);
                    mbar_wait(bar_pv_done((j - 1) & 1), static_cast<uint32_t>((j - 1) >> 1) & 1u, abort_flag,
                              SITE_MLA_PV, j);
                    __syncwarp();
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < 8; ++c) {
                        uint32_t ou[16];
                        tmem_ld16_wait(o_addr + c * 16, ou);
#pragma unroll
                        for (int e = 0; e < 16; ++e) ou[e] = __float_as_uint(__uint_as_float(ou[e]) * alpha);
                        tmem_st16(o_addr + c * 16, ou);
                    }
                }
                m = m_new;
            }

            const float m_ref = (m == -INFINITY) ? 0.f : m;
            const uint64_t c2 = pk2(p.scale_log2, p.scale_log2), nm2 = pk2(-m_ref, -m_ref);
            uint64_t sum2 = pk2(0.f, 0.f);
            uint32_t pk[64];
#pragma unroll
            for (int e = 0; e < 64; ++e) {
                float y0, y1;
                upk2(fma2(pk2(x[2 * e], x[2 * e + 1]), c2, nm2), y0, y1);
                const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
                sum2 = add2(sum2, pk2(p0, p1));
                pk[e] = pack_bf16x2(p0, p1);
            }
            // P[s] fed O += P(j-2) V(j-2); that product has retired: S(j), whose arrival this step began by waiting
            // for, was issued behind it in the same run, the tensor pipe works in order, and the commit that announced
            // S(j) covers everything issued before it.  (A look at pv_done here costs this thread, which is the
            // critical path of the kernel, 300-600 cycles of shared-memory round trip per step.)
            const uint32_t p_addr = tmem_base + lane_base + kColP + s * 64;
            tmem_st32(p_addr, *reinterpret_cast<const uint32_t(*)[32]>(&pk[0]));
            tmem_st32(p_addr + 32, *reinterpret_cast<const uint32_t(*)[32]>(&pk[32]));
            float s_lo, s_hi;
            upk2(sum2, s_lo, s_hi);
            l = l * alpha + (s_lo + s_hi);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar_p_full(s));
        }

        // epilogue: O / l -> bf16 through the (free) Q slabs and a bulk tensor store, lse = m + log(l)
        mbar_wait(bar_pv_done((n_kv - 1) & 1), static_cast<uint32_t>((n_kv - 1) >> 1) & 1u, abort_flag, SITE_MLA_PV,
                  n_kv);
        __syncwarp();
        tc_fence_after();
        const bool visible = l > 0.f;
        const float inv_l = visible ? 1.f / l : 0.f;
        const uint32_t stage_o = base + kSmemQ;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            float ov[32];
            tmem_ld32_wait(o_addr + c * 32, ov);
            const uint32_t row_base = stage_o + (c >> 1) * kSlabBytes + row_in_tile * 128;
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
                const uint32_t chunk = static_cast<uint32_t>((c & 1) * 4 + (e >> 3));
                const uint32_t dst = row_base + ((chunk ^ (static_cast<uint32_t>(row_in_tile) & 7u)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                             "r"(pack_bf16x2(ov[e + 0] * inv_l, ov[e + 1] * inv_l)),
                             "r"(pack_bf16x2(ov[e + 2] * inv_l, ov[e + 3] * inv_l)),
                             "r"(pack_bf16x2(ov[e + 4] * inv_l, ov[e + 5] * inv_l)),
                             "r"(pack_bf16x2(ov[e + 6] * inv_l, ov[e + 7] * inv_l))
                             : "memory");
            }
        }
        fence_async_proxy();
        named_bar_sync(1, kBM);
        if (row_in_tile == 0) {
            tma_store_4d(&tm_o, stage_o, 0, q0, h, b);
            tma_store_4d(&tm_o, stage_o + kSlabBytes, 64, q0, h, b);
            tma_store_commit_and_wait();
        }
        if (qi < p.Sq && row_in_tile < rows_used && p.lse)
            p.lse[(static_cast<long long>(b) * p.Hq + h_row) * p.Sq + qi] = visible ? (m + log2f(l)) * kLn2 : -INFINITY;
        tc_fence_before();
    }

    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

static int encode_map(CUtensorMap* map, const void* basep, int B, int H, int S, int D, int box_rows = 128,
                      int box_heads = 1) {
    const uint64_t row = static_cast<uint64_t>(D) * 2;
    const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(S), static_cast<uint64_t>(H),
                              static_cast<uint64_t>(B)};
    const uint64_t strides[3] = {row, row * S, row * S * H};
    const uint32_t box[4] = {64, static_cast<uint32_t>(box_rows), static_cast<uint32_t>(box_heads), 1};
    return encode_bf16_4d(map, basep, dims, strides, box);
}

template <int kDqk>
static int launch_width(const void* q, const void* k, const void* v, float scale, int causal, void* o, float* lse, int B,
                        int Sq, int Skv, int Hq, int Hkv, DeviceInfo* di, std::atomic<bool>* attr_set, cudaStream_t stream) {
    Params p;
    p.lse = lse;
    p.scale_log2 = scale * kLog2e;
    p.B = B;
    p.Sq = Sq;
    p.Skv = Skv;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = Hq / Hkv;
    p.causal = causal ? 1 : 0;
    p.n_qt = (Sq + kBM - 1) / kBM;
    // Query chunks of at most 64 rows: the heads of a group read the same K/V, so 128 / rows of them share one tile
    // (rows rounded up to a power of two, heads to a power of two that divides the group).
    p.pack = 1;
    p.row_shift = 7;
    if (Sq <= 64) {
        int shift = 0;
        while ((1 << shift) < Sq) ++shift;
        int pack = 1;
        while (pack * 2 <= (128 >> shift) && p.G % (pack * 2) == 0) pack *= 2;
        if (pack > 1) {
            p.pack = pack;
            p.row_shift = shift;
        }
    }
    p.packs_per_group = p.G / p.pack;
    const int box_rows = 1 << p.row_shift;
    const long long blocks = static_cast<long long>(B) * Hkv * p.packs_per_group * p.n_qt;
    if (blocks > 0x7fffffffLL) return CLLO_E_UNSUPPORTED;

    int rc;
    CUtensorMap tm_q, tm_k, tm_v, tm_o;
    if ((rc = encode_map(&tm_q, q, B, Hq, Sq, kDqk, box_rows, p.pack)) != CLLO_OK) return rc;
    if ((rc = encode_map(&tm_k, k, B, Hkv, Skv, kDqk)) != CLLO_OK) return rc;
    if ((rc = encode_map(&tm_v, v, B, Hkv, Skv, kDv)) != CLLO_OK) return rc;
    if ((rc = encode_map(&tm_o, o, B, Hq, Sq, kDv, box_rows, p.pack)) != CLLO_OK) return rc;
    constexpr int smem = Smem<kDqk>::kBytes;
    if (!*attr_set) {
        CLLO_CUDA_TRY(cudaFuncSetAttribute(mla_fwd_kernel<kDqk>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        *attr_set = true;
    }
    (void)di;
    mla_fwd_kernel<kDqk><<<static_cast<unsigned>(blocks), kThreads, smem, stream>>>(tm_q, tm_k, tm_v, tm_o, p);
    CLLO_CUDA_TRY(cudaGetLastError());
    return CLLO_OK;
}

// Dqk = 192 with Dv = 128 (the MLA shape), or Dqk = Dv = 128 (the GQA forward's one-tile case).
static int launch(const void* q, const void* k, const void* v, float scale, int causal, void* o, float* lse, int B,
                  int Sq, int Skv, int Hq, int Hkv, int Dqk, int Dv, cudaStream_t stream) {
    if (!q || !k || !v || !o) return CLLO_E_BAD_ARG;
    if (!(scale != 0.f) || !isfinite(scale)) return CLLO_E_BAD_ARG;  // masking relies on +-infinity times the scale
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || Dqk <= 0 || Dv <= 0) return CLLO_E_BAD_ARG;
    if (Hq % Hkv != 0) return CLLO_E_BAD_ARG;
    if (!aligned_to(q, 16) || !aligned_to(k, 16) || !aligned_to(v, 16) || !aligned_to(o, 16)) return CLLO_E_BAD_ARG;
    if ((Dqk != 192 && Dqk != 128) || Dv != kDv) return CLLO_E_UNSUPPORTED;
    DeviceInfo* di = nullptr;
    int rc = current_device_info(&di);
    if (rc != CLLO_OK) return rc;
    if (di->cc_major != 10) return CLLO_E_UNSUPPORTED;
    if (Dqk == 192)
        return launch_width<192>(q, k, v, scale, causal, o, lse, B, Sq, Skv, Hq, Hkv, di, &di->mla_attr_set, stream);
    return launch_width<128>(q, k, v, scale, causal, o, lse, B, Sq, Skv, Hq, Hkv, di, &di->one_tile_attr_set, stream);
}

}  // namespace mla
}  // namespace cllo
