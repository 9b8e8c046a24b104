// C++ bench harness for the decode path: the timing half of upstream's examples/cplusplus/test_decode_flash_gqa.cu
// (which times one cold launch, :295-309) redone with warm-up, repeated launches and decimal units, calling the
// library through upstream's own launcher signature and through the explicit C ABI.
//
//   nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -I include/cplusplus -I include \
//        examples/cplusplus/bench_flash_gqa.cu -L cuda_llm_ops_b200 -lcllo_flash_gqa \
//        -Xlinker -rpath=$PWD/cuda_llm_ops_b200 -o build/bench_flash_gqa
//   ./build/bench_flash_gqa [B S Hq Hkv iters]
//
// Correctness is not checked here (the parity tests do that against the CPU oracle); inputs are a fixed pattern.
#include "cuda_llm_ops.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#define CHECK(x)                                                                              \
    do {                                                                                      \
        cudaError_t e_ = (x);                                                                 \
        if (e_ != cudaSuccess) {                                                              \
            std::fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));              \
            return 1;                                                                         \
        }                                                                                     \
    } while (0)

__global__ void fill_pattern(__nv_bfloat16* p, size_t n, unsigned seed) {
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (; i < n; i += stride) {
        unsigned h = static_cast<unsigned>(i) * 2654435761u + seed;
        h ^= h >> 15;
        h *= 2246822519u;
        h ^= h >> 13;
        p[i] = __float2bfloat16((static_cast<float>(h & 0xffff) / 32768.f) - 1.f);
    }
}

int main(int argc, char** argv) {
    const int B = argc > 1 ? std::atoi(argv[1]) : 60, S = argc > 2 ? std::atoi(argv[2]) : 4096;
    const int Hq = argc > 3 ? std::atoi(argv[3]) : 128, Hkv = argc > 4 ? std::atoi(argv[4]) : 8;
    const int iters = argc > 5 ? std::atoi(argv[5]) : 50, D = 128;
    const size_t nq = static_cast<size_t>(B) * Hq * D, nkv = static_cast<size_t>(B) * S * Hkv * D;
    __nv_bfloat16 *q, *k, *v, *o;
    float* inter;
    CHECK(cudaMalloc(&q, nq * 2));
    CHECK(cudaMalloc(&k, nkv * 2));
    CHECK(cudaMalloc(&v, nkv * 2));
    CHECK(cudaMalloc(&o, nq * 2));
    CHECK(cudaMalloc(&inter, nq * 4));
    fill_pattern<<<1184, 256>>>(q, nq, 1u);
    fill_pattern<<<1184, 256>>>(k, nkv, 2u);
    fill_pattern<<<1184, 256>>>(v, nkv, 3u);
    const float scale = 0.08838834764831845f;
    const size_t ws_bytes = cllo_gqa_decode_workspace_bytes(B, S, Hq, Hkv, D, 0);
    void* ws;
    CHECK(cudaMalloc(&ws, ws_bytes));
    cudaStream_t stream;
    CHECK(cudaStreamCreate(&stream));
    cudaEvent_t t0, t1;
    CHECK(cudaEventCreate(&t0));
    CHECK(cudaEventCreate(&t1));
    const double bytes = 2.0 * nkv * 2 + 2.0 * nq * 2;

    // (1) upstream's launcher signature (default stream)
    for (int i = 0; i < 5; ++i) LaunchFlashGqaBf16Kernel(q, k, v, scale, o, inter, B, S, Hq, Hkv, D);
    CHECK(cudaDeviceSynchronize());
    CHECK(cudaEventRecord(t0));
    for (int i = 0; i < iters; ++i) LaunchFlashGqaBf16Kernel(q, k, v, scale, o, inter, B, S, Hq, Hkv, D);
    CHECK(cudaEventRecord(t1));
    CHECK(cudaEventSynchronize(t1));
    float ms = 0.f;
    CHECK(cudaEventElapsedTime(&ms, t0, t1));
    std::printf("LaunchFlashGqaBf16Kernel   B=%d S=%d Hq=%d Hkv=%d: %.1f us, %.3f TB/s\n", B, S, Hq, Hkv,
                ms / iters * 1e3, bytes / (ms / iters * 1e-3) / 1e12);

    // (2) explicit C ABI: caller-owned workspace and stream
    for (int i = 0; i < 5; ++i) {
        const int rc = cllo_gqa_decode_bf16(q, k, v, scale, o, ws, ws_bytes, B, S, Hq, Hkv, D, CLLO_KV_BSHD, 0, nullptr,
                                            stream);
        if (rc != CLLO_OK) {
            std::fprintf(stderr, "cllo_gqa_decode_bf16: %s\n", cllo_status_string(rc));
            return 1;
        }
    }
    CHECK(cudaStreamSynchronize(stream));
    CHECK(cudaEventRecord(t0, stream));
    for (int i = 0; i < iters; ++i)
        (void)cllo_gqa_decode_bf16(q, k, v, scale, o, ws, ws_bytes, B, S, Hq, Hkv, D, CLLO_KV_BSHD, 0, nullptr, stream);
    CHECK(cudaEventRecord(t1, stream));
    CHECK(cudaEventSynchronize(t1));
    CHECK(cudaEventElapsedTime(&ms, t0, t1));
    std::printf("cllo_gqa_decode_bf16       B=%d S=%d Hq=%d Hkv=%d: %.1f us, %.3f TB/s\n", B, S, Hq, Hkv,
                ms / iters * 1e3, bytes / (ms / iters * 1e-3) / 1e12);
    int detail[4];
    const int st = cllo_device_status(detail);
    std::printf("device status: %s\n", cllo_status_string(st));
    cllo_shutdown();
    return st == CLLO_OK ? 0 : 2;
}
