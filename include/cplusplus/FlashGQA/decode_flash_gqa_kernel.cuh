// Source-compatible stand-in for upstream's include/cplusplus/FlashGQA/decode_flash_gqa_kernel.cuh:
// same launcher name and argument list (there: lines 28-38), implemented over the C ABI of
// libcllo_flash_gqa.so instead of upstream's wmma kernel.  Link with -lcllo_flash_gqa.
#pragma once

#include <cuda_bf16.h>

#include "../../cllo_flash_gqa.h"
#include "../Utils/utils.cuh"

constexpr int WARP_SIZE = 32;  // exported by upstream's header and used by its test program

// Single-token GQA decode, Q [B,Hq,D], K/V [B,S,Hkv,D], O [B,Hq,D] bf16; oIntermediate is a caller-owned
// fp32 [B,Hq,D] scratch (used as workspace when large enough).  Default stream, current device.
// Returns nothing and stays silent when the shape is refused, which is upstream's behaviour
// (decode_flash_gqa_kernel.cu:416-437); here only headDim != 128 and indivisible head counts are refused.
inline void LaunchFlashGqaBf16Kernel(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                                     float scale, __nv_bfloat16* o, float* oIntermediate, int batchSize,
                                     int seqLength, int numQueryHeads, int numKvHeads, int headDim) {
    (void)cllo_gqa_decode_bf16_compat(q, k, v, scale, o, oIntermediate, batchSize, seqLength, numQueryHeads,
                                      numKvHeads, headDim);
}
