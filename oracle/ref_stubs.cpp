// TEST INFRASTRUCTURE ONLY -- link-time stand-ins that let the upstream benchmark programs
// examples/cplusplus/test_decode_flash_gqa.cu and examples/cplusplus/test_rope.cu run, unmodified, on a machine
// without a GPU.
//
// The upstream program fills Q/K/V with random values, runs its CPU reference loop (:184-255),
// copies the tensors "to the device", calls LaunchFlashGqaBf16Kernel and prints the relative
// error between the kernel's output and its CPU reference.  Here the CUDA runtime calls are
// replaced by host-memory equivalents and the launcher is replaced by this repository's C
// restatement of the same loop (gqa_oracle.c).  "O error = 0" in the program's output therefore
// proves that the restatement is bit-identical to the upstream loop on upstream's own inputs,
// and "CPU time = ..." is the upstream loop timed on this machine's cores.
//
// Nothing here is part of the product; it is built only into oracle/_ref/.
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

extern "C" int cllo_oracle_gqa_decode_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, float scale,
                                           uint16_t* o, float* o_unnorm, float* m_out, float* l_out, int B, int S,
                                           int Hq, int Hkv, int D, int kv_layout, int s_begin, int s_end, int tile,
                                           int par_heads);

extern "C" int cllo_oracle_rope_bf16(const uint16_t* input, uint16_t* output, int B, int S, int hidden, float base);

static double g_launch_ms = 0.0;
static bool g_output_cleared = true;  // set by cudaMemset: the next launcher call has to produce the result again

// Replaces the upstream launcher declared in include/cplusplus/FlashGQA/decode_flash_gqa_kernel.cuh:28-38.
void LaunchFlashGqaBf16Kernel(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, float scale,
                              __nv_bfloat16* o, float* /*oIntermediate*/, int batchSize, int seqLength,
                              int numQueryHeads, int numKvHeads, int headDim) {
    const auto t0 = std::chrono::steady_clock::now();
    const int rc = cllo_oracle_gqa_decode_bf16(
        reinterpret_cast<const uint16_t*>(q), reinterpret_cast<const uint16_t*>(k),
        reinterpret_cast<const uint16_t*>(v), scale, reinterpret_cast<uint16_t*>(o), nullptr, nullptr, nullptr,
        batchSize, seqLength, numQueryHeads, numKvHeads, headDim, /*kv_layout=*/0, 0, seqLength, /*tile=*/128,
        /*par_heads=*/0);
    g_launch_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    std::fprintf(stderr, "[ref_stubs] restated oracle rc=%d, %.3f s\n", rc, g_launch_ms / 1e3);
}

// Replaces the upstream launcher declared in include/cplusplus/RoPE/rope_kernel.cuh:22 (examples/cplusplus/test_rope.cu
// calls it 110 times; the restatement runs on the first call and on the first call after the output was cleared).
void LaunchRopeBf16Kernel(const __nv_bfloat16* input, __nv_bfloat16* output, int batchSize, int seqLen, int hiddenDim,
                          float base) {
    if (!g_output_cleared) return;
    const auto t0 = std::chrono::steady_clock::now();
    const int rc = cllo_oracle_rope_bf16(reinterpret_cast<const uint16_t*>(input), reinterpret_cast<uint16_t*>(output),
                                         batchSize, seqLen, hiddenDim, base);
    g_launch_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    g_output_cleared = false;
    std::fprintf(stderr, "[ref_stubs] restated rope oracle rc=%d, %.3f s\n", rc, g_launch_ms / 1e3);
}

extern "C" {

void** __cudaRegisterFatBinary(void*) {
    static void* handle = nullptr;
    return &handle;
}
void __cudaRegisterFatBinaryEnd(void**) {}
void __cudaUnregisterFatBinary(void**) {}

cudaError_t cudaMalloc(void** p, size_t n) {
    *p = std::malloc(n ? n : 1);
    return *p ? cudaSuccess : cudaErrorMemoryAllocation;
}
cudaError_t cudaMemcpy(void* dst, const void* src, size_t n, cudaMemcpyKind) {
    std::memcpy(dst, src, n);
    return cudaSuccess;
}
cudaError_t cudaMemset(void* p, int value, size_t n) {
    std::memset(p, value, n);
    g_output_cleared = true;
    return cudaSuccess;
}
cudaError_t cudaFree(void* p) {
    std::free(p);
    return cudaSuccess;
}
cudaError_t cudaGetLastError(void) { return cudaSuccess; }
const char* cudaGetErrorString(cudaError_t) { return "stubbed CUDA runtime"; }
cudaError_t cudaEventDestroy(cudaEvent_t) { return cudaSuccess; }
cudaError_t cudaEventCreate(cudaEvent_t* e) {
    *e = nullptr;
    return cudaSuccess;
}
cudaError_t cudaEventRecord(cudaEvent_t, cudaStream_t) { return cudaSuccess; }
cudaError_t cudaEventSynchronize(cudaEvent_t) { return cudaSuccess; }
cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t, cudaEvent_t) {
    *ms = static_cast<float>(g_launch_ms);
    return cudaSuccess;
}

}  // extern "C"
