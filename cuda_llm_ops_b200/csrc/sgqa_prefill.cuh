// Sparse-index GQA forward for sm_100a: every query token attends to its own list of kv tokens.
//
// Upstream: flash_sgqa_forward_bf16_kernel / launch_flash_sgqa_forward_bf16_kernel,
// src/python/Triton/SparseGQA/flash_sgqa_kernel.py:15-138,202-396 (one Triton program per kv head and query token,
// the index list of a token is shared by the query heads of the group).
//
// The work per (batch, kv head, query token) is a small decode: G <= 16 query heads against num_sparse gathered
// K/V rows of 256 bytes each.  K and V of one kv head are a few megabytes and stay in L2, the lists do not repeat
// from token to token, so the kernel is bound by gathering 512 bytes per list entry out of L2, not by HBM and not
// by the tensor cores.  Hence no tcgen05 here (its M is 128; a token offers 16 rows and no two tokens share an
// operand): ONE WARP owns one token at a time and needs nobody else --
//   * it gathers 16 list entries at a time (16 K rows + 16 V rows = 8 KB) with 16-byte cp.async copies into its
//     private shared-memory ring (two buffers: the next gather is in flight while this one is used), in the swizzled [row][128 B] layout that
//     ldmatrix reads without bank conflicts; entries that are out of range, negative (padding) or above the
//     query position (causal) are zero-filled and masked, a group of 16 without any valid entry is skipped;
//   * S = Q K^T (16 heads x 16 entries) and O += P V by mma.sync m16n8k16 with the online softmax in registers
//     (P rounded to bf16 for the product, the row sum taken from the fp32 values, as upstream does);
//   * O / l leaves through the warp's shared memory as 16-byte stores, one 256-byte row per half warp.
// There is no barrier in the kernel apart from __syncwarp, and no wait that could time out.
#pragma once

#include "common.cuh"
#include "host_util.cuh"

namespace cllo {
namespace sgqa {

constexpr int kD = 128;
constexpr int kRows = 16;        // query heads per mma tile (G <= 16, zero padded)
constexpr int kChunk = 16;       // list entries per gather
constexpr int kDefaultWarps = 12;
constexpr int kDefaultBufs = 2;  // ring of gather buffers per warp: one gather in flight behind the one in use
constexpr int kHalfBytes = kChunk * 128;        // [16 rows][64 dims] bf16
constexpr int kBufBytes = 4 * kHalfBytes;       // K (2 halves) + V (2 halves) = 8 KB
constexpr int smem_bytes(int warps, int bufs) { return warps * bufs * kBufBytes + 1024; }
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct Params {
    const __nv_bfloat16* q;   // [B,Hq,Sq,D]
    const __nv_bfloat16* k;   // [B,Hkv,Skv,D]
    const __nv_bfloat16* v;   // [B,Hkv,Skv,D]
    const int* idx;           // [B,Hkv,Sq,num_sparse]
    __nv_bfloat16* o;         // [B,Hq,Sq,D]
    float* lse;               // [B,Hq,Sq], nullable
    float scale_log2;
    int B, Sq, Skv, Hq, Hkv, G, causal, num_sparse;
    long long n_tokens;       // B * Hkv * Sq
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

template <int kWarps, int kBufs>
__global__ void __launch_bounds__(kWarps * 32, 1) sgqa_fwd_kernel(const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tig = lane & 3;
    const uint32_t ring = base + warp * (kBufs * kBufBytes);
    const int n_chunks = (p.num_sparse + kChunk - 1) / kChunk;
    const long long stride = static_cast<long long>(gridDim.x) * kWarps;
    // gather, per lane: 16-byte piece (lane & 15) of rows (lane >> 4) + 2i; destination offset of row (lane >> 4)
    const uint32_t src_lane = static_cast<uint32_t>((lane & 15) * 16);
    const uint32_t dst_lane = static_cast<uint32_t>(((lane & 15) >> 3) * kHalfBytes + (lane >> 4) * 128);
    const uint32_t xor_lane = static_cast<uint32_t>((lane & 7) ^ (lane >> 4));  // piece index XOR (row & 1)

#pragma unroll 1
    for (long long tok = static_cast<long long>(blockIdx.x) * kWarps + warp; tok < p.n_tokens; tok += stride) {
        const int q_pos = static_cast<int>(tok % p.Sq);
        const int kvh = static_cast<int>((tok / p.Sq) % p.Hkv);
        const int b = static_cast<int>(tok / (static_cast<long long>(p.Sq) * p.Hkv));
        const long long head0 = static_cast<long long>(b) * p.Hq + static_cast<long long>(kvh) * p.G;
        const __nv_bfloat16* kbase = p.k + (static_cast<long long>(b) * p.Hkv + kvh) * p.Skv * kD;
        const __nv_bfloat16* vbase = p.v + (static_cast<long long>(b) * p.Hkv + kvh) * p.Skv * kD;
        const int* list = p.idx + tok * p.num_sparse;
        const long long v_minus_k = reinterpret_cast<const char*>(vbase) - reinterpret_cast<const char*>(kbase);

        // Q fragments (A operand: rows = query heads of the group, zero padded to 16)
        uint32_t qf[8][4];
        {
            const uint32_t* q0 = reinterpret_cast<const uint32_t*>(p.q + ((head0 + g) * p.Sq + q_pos) * kD);
            const uint32_t* q1 = reinterpret_cast<const uint32_t*>(p.q + ((head0 + g + 8) * p.Sq + q_pos) * kD);
            const bool v0 = g < p.G, v1 = g + 8 < p.G;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qf[ks][0] = v0 ? __ldg(q0 + ks * 8 + tig) : 0u;
                qf[ks][1] = v1 ? __ldg(q1 + ks * 8 + tig) : 0u;
                qf[ks][2] = v0 ? __ldg(q0 + ks * 8 + tig + 4) : 0u;
                qf[ks][3] = v1 ? __ldg(q1 + ks * 8 + tig + 4) : 0u;
            }
        }

        // Starts the gather of list entries [16c, 16c+16) into ring buffer c % kBufs and returns the 16-bit mask of
        // the valid ones (0 when c is past the list: nothing is copied then).  Always one commit, so that the
        // group count stays in step with the chunk count.
        auto gather = [&](int c) -> uint32_t {
            uint32_t mask = 0;
            if (c < n_chunks) {
                int e = -1;
                if (lane < kChunk && c * kChunk + lane < p.num_sparse) e = __ldg(list + c * kChunk + lane);
                const bool ok = (e >= 0) && (e < p.Skv) && (!p.causal || e <= q_pos);
                e = ok ? e : -1;
                mask = __ballot_sync(0xffffffffu, ok) & 0xffffu;
                if (mask != 0) {
                    const uint32_t buf = ring + (c % kBufs) * kBufBytes + dst_lane;
                    const char* ksrc = reinterpret_cast<const char*>(kbase) + src_lane;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int src_row = __shfl_sync(0xffffffffu, e, 2 * i + (lane >> 4));
                        // row 2i + (lane >> 4): 256 bytes per step of i, the piece index XOR-ed with row & 7
                        const uint32_t dst = buf + i * 256 + ((xor_lane ^ static_cast<uint32_t>((2 * i) & 7)) << 4);
                        const char* src = ksrc + static_cast<long long>(src_row < 0 ? 0 : src_row) * (kD * 2);
                        const uint32_t bytes = src_row < 0 ? 0u : 16u;  // 0: the 16 bytes are zero-filled
                        cp_async_16(dst, src, bytes);
                        cp_async_16(dst + 2 * kHalfBytes, src + v_minus_k, bytes);
                    }
                }
            }
            cp_async_commit();
            return mask;
        };

        float o[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        // kBufs = 3: two gathers run ahead of the one being consumed; kBufs = 2: one (the gather issued in iteration c
        // is then c + 1, and the mask pipeline is one step shorter)
        uint32_t mask_cur = gather(0), mask_nxt = kBufs == 2 ? 0u : gather(1);
#pragma unroll 1
        for (int c = 0; c < n_chunks; ++c) {
            const uint32_t mask_new = gather(kBufs == 2 ? c + 1 : c + 2);
            cp_async_wait<kBufs == 2 ? 1 : 2>();
            __syncwarp();
            if (mask_cur != 0) {
                const uint32_t kb = ring + (c % kBufs) * kBufBytes;
                const uint32_t vb = kb + 2 * kHalfBytes;
                // ---- S = Q K^T  (16 heads x 16 entries) ----
                // (two accumulators per 8 entries, summed at the end: four independent chains of four MMAs instead
                // of two chains of eight -- a warp has few neighbours to hide the MMA latency behind)
                float s[2][4], s2[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
                    s2[nt][0] = s2[nt][1] = s2[nt][2] = s2[nt][3] = 0.f;
                }
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const uint32_t row_off = static_cast<uint32_t>(nt * 8 + (lane & 7)) * 128u;
                        const uint32_t chunk = static_cast<uint32_t>((kk & 1) * 4 + (lane >> 3));
                        const uint32_t addr = kb + (kk >> 1) * kHalfBytes + row_off + ((chunk ^ (lane & 7)) << 4);
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(addr, b0, b1, b2, b3);
                        mma_bf16_16816(s[nt], qf[2 * kk], b0, b1);
                        mma_bf16_16816(s2[nt], qf[2 * kk + 1], b2, b3);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[nt][e] += s2[nt][e];
                }
                // ---- online softmax ----
                float mx0 = -INFINITY, mx1 = -INFINITY;
                if (mask_cur == 0xffffu) {  // the usual case: all 16 entries count
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) s[nt][e] *= p.scale_log2;
                        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
                        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
                    }
                } else {
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const int col = nt * 8 + tig * 2;
                        const bool ok0 = (mask_cur >> col) & 1u, ok1 = (mask_cur >> (col + 1)) & 1u;
                        s[nt][0] = ok0 ? s[nt][0] * p.scale_log2 : -INFINITY;
                        s[nt][2] = ok0 ? s[nt][2] * p.scale_log2 : -INFINITY;
                        s[nt][1] = ok1 ? s[nt][1] * p.scale_log2 : -INFINITY;
                        s[nt][3] = ok1 ? s[nt][3] * p.scale_log2 : -INFINITY;
                        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
                        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
                    }
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: the chunk has a valid entry
                if (__any_sync(0xffffffffu, (mn0 > m0) || (mn1 > m1))) {
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
                // ---- O += P V  (16 heads x 128 dims, one 16-entry k-step) ----
                const uint32_t trow = static_cast<uint32_t>((lane & 7) + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int np = 0; np < 8; ++np) {
                    const uint32_t chunk = static_cast<uint32_t>((np & 3) * 2 + (lane >> 4));
                    const uint32_t addr = vb + (np >> 2) * kHalfBytes + trow * 128u + ((chunk ^ (trow & 7u)) << 4);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(addr, b0, b1, b2, b3);
                    mma_bf16_16816(o[2 * np], pa, b0, b1);
                    mma_bf16_16816(o[2 * np + 1], pa, b2, b3);
                }
            }
            __syncwarp();  // every lane is done with this buffer before gather(c + 3) overwrites it
            mask_cur = kBufs == 2 ? mask_new : mask_nxt;
            mask_nxt = mask_new;
        }
        cp_async_wait<0>();
        __syncwarp();

        // ---- finish: O / l, lse = m + log l (natural units); rows without a valid entry give 0 and -inf ----
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
        // through the first ring buffer as [16 rows][256 B], 16-byte pieces XOR-ed with the row index
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t a0 = ring + g * 256 + ((i ^ g) << 4) + tig * 4;
            const uint32_t a1 = ring + (g + 8) * 256 + ((i ^ (g + 8)) << 4) + tig * 4;
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(a0), "r"(pack_bf16x2(o[i][0] * inv0, o[i][1] * inv0)) : "memory");
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(a1), "r"(pack_bf16x2(o[i][2] * inv1, o[i][3] * inv1)) : "memory");
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = 2 * i + (lane >> 4);
            const int c16 = lane & 15;
            if (row < p.G) {
                uint4 val;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                             : "r"(ring + row * 256 + ((c16 ^ row) << 4)));
                *reinterpret_cast<uint4*>(p.o + ((head0 + row) * p.Sq + q_pos) * kD + c16 * 8) = val;
            }
        }
        if (p.lse && tig == 0) {
            if (g < p.G) p.lse[(head0 + g) * p.Sq + q_pos] = l0 > 0.f ? (m0 + log2f(l0)) * kLn2 : -INFINITY;
            if (g + 8 < p.G) p.lse[(head0 + g + 8) * p.Sq + q_pos] = l1 > 0.f ? (m1 + log2f(l1)) * kLn2 : -INFINITY;
        }
        __syncwarp();  // the staging rows are read before the next token's first gather lands in this buffer
    }
}

static int launch(const void* q, const void* k, const void* v, const int* idx, int num_sparse, float scale, int causal,
                  void* o, float* lse, int B, int Sq, int Skv, int Hq, int Hkv, int D, cudaStream_t stream) {
    if (!q || !k || !v || !idx || !o) return CLLO_E_BAD_ARG;
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || num_sparse <= 0) return CLLO_E_BAD_ARG;
    if (Hq % Hkv != 0) return CLLO_E_BAD_ARG;
    if (!aligned_to(q, 16) || !aligned_to(k, 16) || !aligned_to(v, 16) || !aligned_to(o, 16) || !aligned_to(idx, 4))
        return CLLO_E_BAD_ARG;
    if (D != kD || Hq / Hkv > kRows) return CLLO_E_UNSUPPORTED;
    DeviceInfo* di = nullptr;
    int rc = current_device_info(&di);
    if (rc != CLLO_OK) return rc;
    if (di->cc_major != 10) return CLLO_E_UNSUPPORTED;

    Params p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k = static_cast<const __nv_bfloat16*>(k);
    p.v = static_cast<const __nv_bfloat16*>(v);
    p.idx = idx;
    p.o = static_cast<__nv_bfloat16*>(o);
    p.lse = lse;
    p.scale_log2 = scale * kLog2e;
    p.B = B;
    p.Sq = Sq;
    p.Skv = Skv;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = Hq / Hkv;
    p.causal = causal ? 1 : 0;
    p.num_sparse = num_sparse;
    p.n_tokens = static_cast<long long>(B) * Hkv * Sq;

    // 12 warps x 2 ring buffers (192 KB) measured best at upstream's shape: 8 x 3 1041 us, 10 x 2 1197, 12 x 2 838,
    // 14 x 2 1039 (128 registers per thread: spills)
    constexpr int warps = kDefaultWarps, bufs = kDefaultBufs, smem = smem_bytes(kDefaultWarps, kDefaultBufs);
    if (!di->sgqa_attr_set) {
        CLLO_CUDA_TRY(cudaFuncSetAttribute(sgqa_fwd_kernel<warps, bufs>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        di->sgqa_attr_set = true;
    }
    const long long want = (p.n_tokens + warps - 1) / warps;
    const long long cap = static_cast<long long>(di->sm_count) * 8;  // a few rounds per SM: lists differ in length
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    sgqa_fwd_kernel<warps, bufs><<<grid, warps * 32, smem, stream>>>(p);
    CLLO_CUDA_TRY(cudaGetLastError());
    return CLLO_OK;
}

}  // namespace sgqa
}  // namespace cllo
