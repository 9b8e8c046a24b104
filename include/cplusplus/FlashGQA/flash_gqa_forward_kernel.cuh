// C++ launcher for the prefill (multi-token) GQA forward.  Upstream has this operator only as a Triton
// kernel (src/python/Triton/flash_gqa_kernel.py:185-338); this header gives it the same calling style as
// upstream's C++ operators: raw device pointers, int dimensions, default stream, void.
#pragma once

#include <cuda_bf16.h>

#include "../../cllo_flash_gqa.h"

// q, o [B,Hq,Sq,D]; k, v [B,Hkv,Skv,D] bf16; lse [B,Hq,Sq] fp32 or nullptr; causal keeps kv <= q.
inline void LaunchFlashGqaForwardBf16Kernel(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                                            float scale, bool causal, __nv_bfloat16* o, float* lse, int batchSize,
                                            int seqLengthQ, int seqLengthKv, int numQueryHeads, int numKvHeads,
                                            int headDim) {
    (void)cllo_gqa_prefill_fwd_bf16(q, k, v, scale, causal ? 1 : 0, o, lse, batchSize, seqLengthQ, seqLengthKv,
                                    numQueryHeads, numKvHeads, headDim, nullptr);
}
