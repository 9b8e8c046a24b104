// Umbrella header under upstream's name (include/cplusplus/cuda_llm_ops.h there): only the operators this
// library implements.  Inside the upstream tree keep upstream's umbrella and swap the FlashGQA header.
#pragma once

#include "FlashGQA/decode_flash_gqa_kernel.cuh"
#include "FlashGQA/flash_gqa_forward_kernel.cuh"
#include "RoPE/rope_kernel.cuh"
#include "Utils/utils.cuh"
