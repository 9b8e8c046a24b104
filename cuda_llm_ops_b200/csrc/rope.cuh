// Rotary position embedding, bf16, interleaved pairs over the whole hidden dimension: the operator that
// precedes attention in a decoder (upstream: RopeBf16Kernel, src/cplusplus/RoPE/rope_kernel.cu:33-107).
//
// HBM-bound: 2 * B * S * hidden * 2 bytes per call.  Every thread rotates 4 pairs (one 16-byte load, one
// 16-byte store).  Results follow the CPU reference of upstream's test (examples/cplusplus/test_rope.cu:69-101)
// rather than upstream's kernel, which uses the fast-math __sincosf on angles of up to 5e5 radians:
//   * the inverse frequencies powf(base, -2i/hidden) are computed on the HOST, with the same libm call as the
//     reference, and travel as a kernel argument (hidden <= 1024);
//   * the angle is the fp32 product token * invFreq, as in the reference;
//   * sine and cosine of that fp32 angle are evaluated accurately for any magnitude: exact range reduction in
//     integer arithmetic, then fp32 minimax polynomials on [-pi/4, pi/4].
#pragma once

#include "common.cuh"
#include "host_util.cuh"

#include <cmath>

namespace cllo {
namespace rope {

constexpr int kMaxHalf = 512;  // hidden <= 1024
constexpr int kThreads = 256;

struct Params {
    const uint4* in;
    uint4* out;
    long long n_vec;  // number of 8-element vectors
    int hidden, seq_len;
    float inv_freq[kMaxHalf];
};

// sine and cosine of an fp32 angle x >= 0, accurate to about an fp32 ulp for any magnitude.
// Range reduction: below 786432 rad (every angle of a 512K-token sequence) an eight-constant Cody-Waite scheme in
// fp32; up to 2^25 an integer scheme (x = m * 2^(e-23) with a 24-bit m, 2/pi as a 64-bit fixed-point constant, a
// 64-bit window of the 128-bit product holds the quadrant and 62 fraction bits); beyond that double precision.
// Then fp32 minimax polynomials on [-pi/4, pi/4].
__device__ __forceinline__ void sincos_accurate(float x, float& s, float& c) {
    const uint32_t ix = __float_as_uint(x);
    const int e = static_cast<int>(ix >> 23) - 127;
    int q = 0;
    float z = x;
    if (x < 786432.0f) {
        // Cody-Waite with pi/2 cut into 6-bit pieces: k < 2^19, so every product k * piece is exact inside the
        // fused multiply-add and every difference is representable (the operands agree in their leading bits).
        const float k = rintf(x * 0.63661977236758134f);
        z = fmaf(-k, 1.5625f, x);
        z = fmaf(-k, 0.008056640625f, z);
        z = fmaf(-k, 0.00023651123046875f, z);
        z = fmaf(-k, 3.1590461730957031e-06f, z);
        z = fmaf(-k, 1.5832483768463135e-08f, z);
        z = fmaf(-k, 6.0026650317013264e-11f, z);
        z = fmaf(-k, 7.3896444519050419e-13f, z);
        z = fmaf(-k, 5.3290705182007514e-15f, z);
        q = static_cast<int>(k) & 3;
    } else if (e <= 24) {  // up to 2^25: exact reduction in integer arithmetic
        const unsigned long long m = (ix & 0x7fffffu) | 0x800000u;
        const unsigned long long two_over_pi = 0xA2F9836E4E441529ull;  // 2/pi * 2^64
        const unsigned long long hi = __umul64hi(m, two_over_pi), lo = m * two_over_pi;
        const int sh = 25 - e;  // 1..26: drops all but 62 fraction bits
        unsigned long long w = (hi << (64 - sh)) | (lo >> sh);
        w += 1ull << 61;  // round to the nearest quarter turn
        q = static_cast<int>(w >> 62);
        const long long frac = static_cast<long long>(w & ((1ull << 62) - 1)) - (1ll << 61);  // in [-2^61, 2^61)
        z = static_cast<float>(static_cast<int>(frac >> 30)) * (1.5707963267948966f * 2.3283064365386963e-10f);
    } else if (e > 24) {  // astronomically large angles: double-precision reduction, rarely taken
        const double xd = static_cast<double>(x);
        const double kd = rint(xd * 0.63661977236758134308);
        double r = fma(-kd, 1.57079632679489655800, xd);
        r = fma(-kd, 6.12323399573676603587e-17, r);
        q = static_cast<int>(static_cast<long long>(kd) & 3);
        z = static_cast<float>(r);
    }
    const float z2 = z * z;
    const float sp = z + z * z2 * (-1.6666654611e-1f + z2 * (8.3321608736e-3f + z2 * -1.9515295891e-4f));
    const float cp = 1.0f - 0.5f * z2 + z2 * z2 * (4.166664568298827e-2f + z2 * (-1.388731625493765e-3f + z2 * 2.443315711809948e-5f));
    const float ss = (q & 1) ? cp : sp, cc = (q & 1) ? sp : cp;
    s = (q & 2) ? -ss : ss;
    c = ((q + 1) & 2) ? -cc : cc;
}

template <typename Index>
__device__ __forceinline__ void rope_loop(const Params& p, const float* inv_freq) {
    const Index n = static_cast<Index>(p.n_vec), stride = static_cast<Index>(gridDim.x) * kThreads;
    const Index vecs_per_row = static_cast<Index>(p.hidden / 8);
    for (Index v = static_cast<Index>(blockIdx.x) * kThreads + threadIdx.x; v < n; v += stride) {
        const Index row = v / vecs_per_row;
        const int pair0 = static_cast<int>(v - row * vecs_per_row) * 4;
        const int token = static_cast<int>(row % static_cast<Index>(p.seq_len));
        const uint4 raw = p.in[v];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float angle = static_cast<float>(token) * inv_freq[pair0 + i];
            float s, c;
            sincos_accurate(angle, s, c);
            const float even = __uint_as_float(w[i] << 16), odd = __uint_as_float(w[i] & 0xffff0000u);
            r[i] = pack_bf16x2(even * c - odd * s, even * s + odd * c);
        }
        p.out[v] = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

__global__ void __launch_bounds__(kThreads) rope_bf16_kernel(const __grid_constant__ Params p) {
    // the table goes to shared memory: lanes of a warp read different entries, which the constant bank that
    // holds kernel arguments would serialise
    __shared__ float inv_freq[kMaxHalf];
    for (int i = threadIdx.x; i < p.hidden / 2; i += kThreads) inv_freq[i] = p.inv_freq[i];
    __syncthreads();
    if (p.n_vec < 0x7fffffffLL - static_cast<long long>(gridDim.x) * kThreads)
        rope_loop<unsigned>(p, inv_freq);  // 32-bit index arithmetic (the common case)
    else
        rope_loop<long long>(p, inv_freq);
}

static int launch(const void* input, void* output, int B, int S, int hidden, float base, cudaStream_t stream) {
    if (!input || !output || B <= 0 || S <= 0 || hidden <= 0) return CLLO_E_BAD_ARG;
    if (!aligned_to(input, 16) || !aligned_to(output, 16)) return CLLO_E_BAD_ARG;
    if ((hidden % 8) != 0 || hidden > 2 * kMaxHalf) return CLLO_E_UNSUPPORTED;
    DeviceInfo* di = nullptr;
    int rc = current_device_info(&di);
    if (rc != CLLO_OK) return rc;
    Params p;
    p.in = static_cast<const uint4*>(input);
    p.out = static_cast<uint4*>(output);
    p.n_vec = static_cast<long long>(B) * S * hidden / 8;
    p.hidden = hidden;
    p.seq_len = S;
    const float hidden_inv = 1.0f / static_cast<float>(hidden);
    for (int i = 0; i < hidden / 2; ++i) p.inv_freq[i] = std::pow(base, -2.0f * static_cast<float>(i) * hidden_inv);
    for (int i = hidden / 2; i < kMaxHalf; ++i) p.inv_freq[i] = 0.f;
    long long blocks = (p.n_vec + kThreads - 1) / kThreads;
    const long long cap = static_cast<long long>(di->sm_count) * 16;  // grid-stride beyond 16 blocks per SM
    if (blocks > cap) blocks = cap;
    rope_bf16_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(p);
    CLLO_CUDA_TRY(cudaGetLastError());
    return CLLO_OK;
}

}  // namespace rope
}  // namespace cllo
