// Split-KV single-token GQA decode for sm_100a.
//
// Work decomposition.  A "unit" is one (batch, kv head, block of <=16 query heads).  Its KV range
// is cut into tiles of 64 tokens; all tiles of all units form one flat index space that is divided
// evenly (to within one tile) among W persistent thread blocks ("workers"), so every SM streams the
// same number of bytes whatever the batch / head counts are.  A worker therefore processes a few
// whole units plus at most one partial unit at each end of its range.
//
// Inside a worker.  One producer warp issues TMA tile loads (K and V, 64 tokens x 128 dims each,
// 128-byte swizzled, 32 KB per stage) into a 5-stage ring guarded by full/empty mbarriers.  Eight
// consumer warps take stages round-robin.  Each consumer warp computes, for ITS 64 tokens and ALL
// query heads of the unit (padded to 16 rows): S = Q K^T with mma.sync m16n8k16 (K fragments via
// ldmatrix), an online-softmax update of its private running (m, l, O) with quad shuffles, and
// O += P V (V fragments via ldmatrix.trans, P fed straight from the accumulator registers).  There
// is no block-wide barrier in the streaming loop.  At the end of a unit the eight private states are
// merged pairwise through shared memory (log-sum-exp algebra), and warp 0 writes either the final
// bf16 output (unit entirely inside this worker) or an fp32 partial (O, m, l) to the workspace.
//
// Second pass.  decode_merge_kernel visits every unit that was cut by a worker boundary and merges
// its partials:  m* = max m_i,  O = sum e^(m_i-m*) O_i / sum e^(m_i-m*) l_i.
//
// HBM traffic per launch = K + V once (+ Q, O, and ~1% for partials): the algorithmic minimum.
#pragma once

#include "common.cuh"
#include "host_util.cuh"

namespace cllo {
namespace decode {

constexpr int kD = 128;
constexpr int kTok = 64;
constexpr int kStages = 5;
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kHalfBytes = kTok * 128;       // [64 tokens][64 dims] bf16
constexpr int kStageBytes = 4 * kHalfBytes;  // K dims 0-63, K dims 64-127, V dims 0-63, V dims 64-127
constexpr int kMergeFloats = 68 * 32;        // per lane: 64 O values, m0, m1, l0, l1
constexpr int kMergeBufs = 4;
constexpr int kRows = 16;                    // query-head rows per unit (MMA M)
constexpr int kPW = kD + 2;                  // packed partial row width
constexpr int kSlotFloats = kRows * kPW;     // one partial slot in the workspace
constexpr int kSmemBytes = kStages * kStageBytes + kMergeBufs * kMergeFloats * 4 + 2 * kStages * 8 + 32 + 1024;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct Params {
    const __nv_bfloat16* q;
    __nv_bfloat16* o;
    float* partial_out;  // nullable
    float* ws;           // [W][2][16][D+2]
    float scale_log2;    // scale * log2(e)
    int B, S, Hq, Hkv, G, n_gblk, n_t, kv_layout, W;
    long long T;  // total tiles
};

__host__ __device__ __forceinline__ long long worker_lo(long long w, long long T, long long W) {
    return (w * T) / W;
}
// the worker whose range [worker_lo(w), worker_lo(w+1)) holds tile t
__host__ __device__ __forceinline__ long long worker_of_tile(long long t, long long T, long long W) {
    return ((t + 1) * W - 1) / T;
}

__global__ void __launch_bounds__(kThreads, 1)
decode_splitkv_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t stage_base = base;
    float* merge = reinterpret_cast<float*>(gen_base + kStages * kStageBytes);
    const uint32_t bar_base = base + kStages * kStageBytes + kMergeBufs * kMergeFloats * 4;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + kStages * kStageBytes +
                                                               kMergeBufs * kMergeFloats * 4 + 2 * kStages * 8);
    // number of tiles the producer has issued so far.  A consumer looks at a stage's full barrier only once
    // ITS tile has been issued: the stages are shared by all consumer warps, and a parity wait placed two
    // phases early would be satisfied by the wrong phase.
    volatile long long* issued = reinterpret_cast<volatile long long*>(
        gen_base + kStages * kStageBytes + kMergeBufs * kMergeFloats * 4 + 2 * kStages * 8 + 16);
    auto full_bar = [&](int s) { return bar_base + s * 8; };
    auto empty_bar = [&](int s) { return bar_base + (kStages + s) * 8; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = blockIdx.x;
    const long long lo = worker_lo(w, p.T, p.W), hi = worker_lo(w + 1, p.T, p.W);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        *abort_flag = 0;
        *issued = 0;
        fence_mbar_init();
    }
    __syncthreads();
    if (lo >= hi) return;

    if (warp == kConsumerWarps) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            for (long long t = lo; t < hi; ++t) {
                const long long it = t - lo;
                const int slot = static_cast<int>(it % kStages);
                const uint32_t use = static_cast<uint32_t>(it / kStages);
                mbar_wait(empty_bar(slot), (use & 1u) ^ 1u, abort_flag, SITE_DECODE_EMPTY, slot);
                const long long u = t / p.n_t;
                const int s0 = static_cast<int>(t - u * p.n_t) * kTok;
                const int kvh = static_cast<int>((u / p.n_gblk) % p.Hkv);
                const int b = static_cast<int>(u / (static_cast<long long>(p.n_gblk) * p.Hkv));
                const int c1 = p.kv_layout == CLLO_KV_BSHD ? kvh : s0;
                const int c2 = p.kv_layout == CLLO_KV_BSHD ? s0 : kvh;
                const uint32_t dst = stage_base + slot * kStageBytes;
                mbar_arrive_expect_tx(full_bar(slot), kStageBytes);
                tma_load_4d(dst, &tm_k, full_bar(slot), 0, c1, c2, b);
                tma_load_4d(dst + kHalfBytes, &tm_k, full_bar(slot), 64, c1, c2, b);
                tma_load_4d(dst + 2 * kHalfBytes, &tm_v, full_bar(slot), 0, c1, c2, b);
                tma_load_4d(dst + 3 * kHalfBytes, &tm_v, full_bar(slot), 64, c1, c2, b);
                __threadfence_block();
                *issued = it + 1;
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
            }
        }

        float o[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        const long long first = seg_lo + ((static_cast<long long>(warp) - (seg_lo - lo)) % 8 + 8) % 8;
#pragma unroll 1
        for (long long t = first; t < seg_hi; t += kConsumerWarps) {
            const long long it = t - lo;
            const int slot = static_cast<int>(it % kStages);
            const uint32_t use = static_cast<uint32_t>(it / kStages);
            if (*issued <= it) {
                const long long t0 = clock64();
                while (*issued <= it && !*abort_flag) {
                    if (clock64() - t0 > kWaitLimitCycles) {
                        *abort_flag = 1;
                        record_timeout(SITE_DECODE_ISSUE, slot);
                    }
                }
            }
            mbar_wait(full_bar(slot), use & 1u, abort_flag, SITE_DECODE_FULL, slot);
            __syncwarp();
            const uint32_t kb = stage_base + slot * kStageBytes;
            const uint32_t vb = kb + 2 * kHalfBytes;
            const int tok0 = static_cast<int>(t - unit_lo) * kTok;
            const int valid = (p.S - tok0) < kTok ? (p.S - tok0) : kTok;

            // ---- S = Q K^T  (16 x 64) ----
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
                const uint32_t row_off = static_cast<uint32_t>(nt * 8 + (lane & 7)) * 128u;
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
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] *= p.scale_log2;
                if (valid < kTok) {
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
            const float a0 = fast_exp2(m0 - mn0), a1 = fast_exp2(m1 - mn1);
            m0 = mn0;
            m1 = mn1;
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t pa[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float p0 = fast_exp2(s[nt][0] - mn0), p1 = fast_exp2(s[nt][1] - mn0);
                const float p2 = fast_exp2(s[nt][2] - mn1), p3 = fast_exp2(s[nt][3] - mn1);
                sum0 += p0 + p1;
                sum1 += p2 + p3;
                pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(p0, p1);
                pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
            }
            l0 = l0 * a0 + sum0;
            l1 = l1 * a1 + sum1;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                o[i][0] *= a0;
                o[i][1] *= a0;
                o[i][2] *= a1;
                o[i][3] *= a1;
            }

            // ---- O += P V  (16 x 128) ----
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
                const uint32_t tok = static_cast<uint32_t>(kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int np = 0; np < 8; ++np) {
                    const uint32_t chunk = static_cast<uint32_t>((np & 3) * 2 + (lane >> 4));
                    const uint32_t addr = vb + (np >> 2) * kHalfBytes + tok * 128u + ((chunk ^ (tok & 7u)) << 4);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(addr, b0, b1, b2, b3);
                    mma_bf16_16816(o[2 * np], pa[kt], b0, b1);
                    mma_bf16_16816(o[2 * np + 1], pa[kt], b2, b3);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(slot));
        }

        // ---- merge the eight private states (pairwise tree through shared memory) ----
#pragma unroll 1
        for (int st = 1; st < kConsumerWarps; st <<= 1) {
            const bool writer = (warp % (2 * st)) == st;
            const bool reader = (warp % (2 * st)) == 0;
            float* buf = merge + (warp / (2 * st)) * kMergeFloats;
            if (writer) {
#pragma unroll
                for (int i = 0; i < 64; ++i) buf[i * 32 + lane] = o[i >> 2][i & 3];
                buf[64 * 32 + lane] = m0;
                buf[65 * 32 + lane] = m1;
                buf[66 * 32 + lane] = l0;
                buf[67 * 32 + lane] = l1;
            }
            named_bar_sync(1, kConsumerWarps * 32);
            if (reader) {
                const float om0 = buf[64 * 32 + lane], om1 = buf[65 * 32 + lane];
                const float ol0 = buf[66 * 32 + lane], ol1 = buf[67 * 32 + lane];
                const float mn0 = fmaxf(m0, om0), mn1 = fmaxf(m1, om1);
                const float sa0 = (m0 == -INFINITY) ? 0.f : fast_exp2(m0 - mn0);
                const float sa1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - mn1);
                const float sb0 = (om0 == -INFINITY) ? 0.f : fast_exp2(om0 - mn0);
                const float sb1 = (om1 == -INFINITY) ? 0.f : fast_exp2(om1 - mn1);
                l0 = l0 * sa0 + ol0 * sb0;
                l1 = l1 * sa1 + ol1 * sb1;
                m0 = mn0;
                m1 = mn1;
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const float other = buf[i * 32 + lane];
                    const bool hi_row = (i & 2) != 0;
                    o[i >> 2][i & 3] = o[i >> 2][i & 3] * (hi_row ? sa1 : sa0) + other * (hi_row ? sb1 : sb0);
                }
            }
            named_bar_sync(1, kConsumerWarps * 32);
        }

        // ---- warp 0 owns the merged result ----
        if (warp == 0) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
            l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
            const bool whole = (seg_lo == unit_lo) && (seg_hi == unit_hi);
            if (whole && p.partial_out == nullptr) {
                const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
                for (int nt = 0; nt < 16; ++nt) {
                    const int col = nt * 8 + tig * 2;
                    if (g < rows)
                        *reinterpret_cast<uint32_t*>(p.o + (head0 + g) * kD + col) =
                            pack_bf16x2(o[nt][0] * i0, o[nt][1] * i0);
                    if (g + 8 < rows)
                        *reinterpret_cast<uint32_t*>(p.o + (head0 + g + 8) * kD + col) =
                            pack_bf16x2(o[nt][2] * i1, o[nt][3] * i1);
                }
            } else {
                float* d0;
                float* d1;
                if (whole) {
                    d0 = p.partial_out + (head0 + g) * kPW;
                    d1 = p.partial_out + (head0 + g + 8) * kPW;
                } else {
                    const int which = (u == u_first) ? 0 : 1;
                    float* slot_base = p.ws + (w * 2 + which) * kSlotFloats;
                    d0 = slot_base + g * kPW;
                    d1 = slot_base + (g + 8) * kPW;
                }
#pragma unroll
                for (int nt = 0; nt < 16; ++nt) {
                    const int col = nt * 8 + tig * 2;
                    if (g < rows) *reinterpret_cast<float2*>(d0 + col) = make_float2(o[nt][0], o[nt][1]);
                    if (g + 8 < rows) *reinterpret_cast<float2*>(d1 + col) = make_float2(o[nt][2], o[nt][3]);
                }
                if (tig == 0) {
                    if (g < rows) {
                        d0[kD] = m0 * kLn2;
                        d0[kD + 1] = l0;
                    }
                    if (g + 8 < rows) {
                        d1[kD] = m1 * kLn2;
                        d1[kD + 1] = l1;
                    }
                }
            }
        }
    }
}

// Second pass over the units that a worker boundary cut.  grid = units, block = 128 (one thread per dim).
__global__ void __launch_bounds__(kD) decode_merge_kernel(const Params p) {
    const long long u = blockIdx.x;
    const long long t_first = u * p.n_t, t_last = t_first + p.n_t - 1;
    const long long w_lo = worker_of_tile(t_first, p.T, p.W), w_hi = worker_of_tile(t_last, p.T, p.W);
    if (w_lo == w_hi) return;  // the unit lived inside one worker, which wrote the final result
    const int gblk = static_cast<int>(u % p.n_gblk);
    const int kvh = static_cast<int>((u / p.n_gblk) % p.Hkv);
    const int b = static_cast<int>(u / (static_cast<long long>(p.n_gblk) * p.Hkv));
    const int rows = (p.G - gblk * kRows) < kRows ? (p.G - gblk * kRows) : kRows;
    const long long head0 = static_cast<long long>(b) * p.Hq + static_cast<long long>(kvh) * p.G + gblk * kRows;
    const int which_lo = (worker_lo(w_lo, p.T, p.W) == t_first) ? 0 : 1;
    const int d = threadIdx.x;
    for (int r = 0; r < rows; ++r) {
        float mstar = -INFINITY;
        for (long long w = w_lo; w <= w_hi; ++w) {
            const float* row = p.ws + (w * 2 + (w == w_lo ? which_lo : 0)) * kSlotFloats + r * kPW;
            if (row[kD + 1] > 0.f) mstar = fmaxf(mstar, row[kD]);
        }
        float acc = 0.f, lsum = 0.f;
        for (long long w = w_lo; w <= w_hi; ++w) {
            const float* row = p.ws + (w * 2 + (w == w_lo ? which_lo : 0)) * kSlotFloats + r * kPW;
            const float l = row[kD + 1];
            const float wgt = l > 0.f ? __expf(row[kD] - mstar) : 0.f;
            acc += wgt * row[d];
            lsum += wgt * l;
        }
        if (p.partial_out) {
            float* dst = p.partial_out + (head0 + r) * kPW;
            dst[d] = acc;
            if (d == 0) {
                dst[kD] = mstar;
                dst[kD + 1] = lsum;
            }
        } else {
            p.o[(head0 + r) * kD + d] = __float2bfloat16(lsum > 0.f ? acc / lsum : 0.f);
        }
    }
}

// Public merge of caller-provided partials [nsplit][rows][D+2] -> bf16 [rows][D].  One row per block.
__global__ void __launch_bounds__(kD) combine_rows_kernel(const float* __restrict__ partials, int nsplit,
                                                          long long rows, __nv_bfloat16* __restrict__ o) {
    const long long r = blockIdx.x;
    const int d = threadIdx.x;
    float mstar = -INFINITY;
    for (int i = 0; i < nsplit; ++i) {
        const float* row = partials + (static_cast<long long>(i) * rows + r) * kPW;
        if (row[kD + 1] > 0.f) mstar = fmaxf(mstar, row[kD]);
    }
    float acc = 0.f, lsum = 0.f;
    for (int i = 0; i < nsplit; ++i) {
        const float* row = partials + (static_cast<long long>(i) * rows + r) * kPW;
        const float l = row[kD + 1];
        const float wgt = l > 0.f ? __expf(row[kD] - mstar) : 0.f;
        acc += wgt * row[d];
        lsum += wgt * l;
    }
    o[r * kD + d] = __float2bfloat16(lsum > 0.f ? acc / lsum : 0.f);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct Plan {
    Params prm;
    size_t ws_bytes;
    bool needs_merge;
    long long units;
};

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
    p.T = plan->units * p.n_t;
    long long W = num_workers > 0 ? num_workers : sm_count;
    if (W > p.T) W = p.T;
    if (W < 1) W = 1;
    p.W = static_cast<int>(W);
    plan->ws_bytes = static_cast<size_t>(W) * 2 * kSlotFloats * sizeof(float);
    plan->needs_merge = false;
    for (long long w = 1; w < W; ++w)
        if (worker_lo(w, p.T, W) % p.n_t != 0) {
            plan->needs_merge = true;
            break;
        }
    return CLLO_OK;
}

static int encode_kv_map(CUtensorMap* map, const void* base, int B, int S, int Hkv, int kv_layout) {
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
        strides[1] = row * S;
        box[1] = kTok;
        box[2] = 1;
    }
    dims[3] = static_cast<uint64_t>(B);
    strides[2] = row * static_cast<uint64_t>(S) * Hkv;
    box[3] = 1;
    return encode_bf16_4d(map, base, dims, strides, box);
}

}  // namespace decode
}  // namespace cllo
