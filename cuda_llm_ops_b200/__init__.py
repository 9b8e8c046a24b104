"""B200 (sm_100a) flash grouped-query attention: drop-in for the GQA path of cuda_llm_ops.

The product is the C-ABI shared library built from ``csrc/`` (declared in ``include/cllo_flash_gqa.h``);
this package is the thin host side that mirrors upstream's launcher functions on top of it.
"""
from .flash_gqa import (  # noqa: F401
    HEAD_DIM,
    KV_BHSD,
    KV_BSHD,
    PARTIAL_WIDTH,
    LaunchFlashGqaBf16Kernel,
    LaunchRopeBf16Kernel,
    decode_workspace_bytes,
    device_status,
    gqa_combine,
    gqa_decode,
    gqa_decode_rope_append,
    gqa_decode_sharded,
    launch_decode_flash_gqa_bf16_kernel,
    launch_flash_gqa_backward_bf16_kernel,
    launch_flash_gqa_forward_bf16_kernel,
    launch_flash_mla_forward_bf16_kernel,
    launch_flash_sgqa_forward_bf16_kernel,
    launch_flash_swa_backward_bf16_kernel,
    launch_flash_swa_forward_bf16_kernel,
    set_exchange_wait_limit,
)
from .sharded import (  # noqa: F401
    KVShardedDecoder,
    shard_batch,
    shard_kv_positions,
)
