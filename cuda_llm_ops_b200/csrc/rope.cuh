// Rotary position embedding, bf16, interleaved pairs over the whole hidden dimension: the operator that
// precedes attention in a decoder (upstream: RopeBf16Kernel, src/cplusplus/RoPE/rope_kernel.cu:33-107).
//
// HBM-bound: 2 * B * S * hidden * 2 bytes per call.  Every thread rotates 4 pairs (one 16-byte load, one
// 16-byte store).  Results follow the CPU reference of upstream's test (examples/cplusplus/test_rope.cu:69-101)
// rather than upstream's kernel, which uses the fast-math __sincosf on angles of up to 5e5 radians:
//   * the inverse frequencies powf(base, -2i/hidden) are computed on the HOST, with the same libm call as the
//     reference, and travel as a kernel argument (hidden <= 1024);
//   * the angle is the fp32 product token * invFreq, as in the reference;
//   * sine and cosine of that fp32 angle are evaluated accurately for any magnitude: two-constant Cody-Waite
//     reduction in double precision (exact enough for |angle| < 2^22), then fp32 minimax polynomials on
//     [-pi/4, pi/4].
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

__device__ __forceinline__ void sincos_accurate(float x, float& s, float& c) {
    const double xd = static_cast<double>(x);
    const double kd = rint(xd * 0.63661977236758134308);  // 2/pi
    double r = fma(-kd, 1.57079632679489655800, xd);       // pi/2, high part
    r = fma(-kd, 6.12323399573676603587e-17, r);           // pi/2, low part
    const int q = static_cast<int>(kd);
    const float z = static_cast<float>(r), z2 = z * z;
    const float sp = z + z * z2 * (-1.6666654611e-1f + z2 * (8.3321608736e-3f + z2 * -1.9515295891e-4f));
    const float cp = 1.0f - 0.5f * z2 + z2 * z2 * (4.166664568298827e-2f + z2 * (-1.388731625493765e-3f + z2 * 2.443315711809948e-5f));
    const float ss = (q & 1) ? cp : sp, cc = (q & 1) ? sp : cp;
    s = (q & 2) ? -ss : ss;
    c = ((q + 1) & 2) ? -cc : cc;
}

__global__ void __launch_bounds__(kThreads) rope_bf16_kernel(const __grid_constant__ Params p) {
    const long long stride = static_cast<long long>(gridDim.x) * kThreads;
    for (long long v = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; v < p.n_vec; v += stride) {
        const long long e0 = v * 8;
        const int dim0 = static_cast<int>(e0 % p.hidden);
        const int token = static_cast<int>((e0 / p.hidden) % p.seq_len);
        const uint4 raw = p.in[v];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float angle = static_cast<float>(token) * p.inv_freq[dim0 / 2 + i];
            float s, c;
            sincos_accurate(angle, s, c);
            const float even = __uint_as_float(w[i] << 16), odd = __uint_as_float(w[i] & 0xffff0000u);
            r[i] = pack_bf16x2(even * c - odd * s, even * s + odd * c);
        }
        p.out[v] = make_uint4(r[0], r[1], r[2], r[3]);
    }
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
