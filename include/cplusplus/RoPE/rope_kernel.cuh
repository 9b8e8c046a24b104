// Source-compatible stand-in for upstream's include/cplusplus/RoPE/rope_kernel.cuh (launcher at line 22 there):
// same launcher name and arguments, implemented over the C ABI of libcllo_flash_gqa.so.
#pragma once

#include <cuda_bf16.h>

#include "../../cllo_flash_gqa.h"

constexpr int kRopeValuesPerThread = 8;    // exported by upstream's header
constexpr int kRopeThreadsPerBlock = 256;  // exported by upstream's header

// input/output [batchSize, seqLen, hiddenDim] bf16; default stream; silent on refused sizes like upstream.
inline void LaunchRopeBf16Kernel(const __nv_bfloat16* input, __nv_bfloat16* output, int batchSize, int seqLen,
                                 int hiddenDim, float base = 10000.0f) {
    (void)cllo_rope_bf16(input, output, batchSize, seqLen, hiddenDim, base, nullptr);
}
