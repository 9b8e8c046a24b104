"""Host-side mirror of upstream's launchers: argument checks and sharding arithmetic (no GPU)."""
import pytest
import torch

import cuda_llm_ops_b200 as ops


def _t(*shape, dtype=torch.bfloat16):
    return torch.zeros(*shape, dtype=dtype)


def test_triton_decode_launcher_error_behaviour_matches_upstream():
    # same checks, same exception type as src/python/Triton/decode_flash_gqa_kernel.py:153-171
    with pytest.raises(ValueError, match="bf16"):
        ops.launch_decode_flash_gqa_bf16_kernel(_t(1, 4, 1, 128, dtype=torch.float16), _t(1, 1, 8, 128), _t(1, 1, 8, 128))
    with pytest.raises(ValueError, match="contiguous"):
        ops.launch_decode_flash_gqa_bf16_kernel(_t(1, 4, 1, 256)[..., ::2], _t(1, 1, 8, 128), _t(1, 1, 8, 128))
    with pytest.raises(ValueError, match="batch"):
        ops.launch_decode_flash_gqa_bf16_kernel(_t(2, 4, 1, 128), _t(1, 1, 8, 128), _t(1, 1, 8, 128))
    with pytest.raises(ValueError, match="sequence length"):
        ops.launch_decode_flash_gqa_bf16_kernel(_t(1, 4, 1, 128), _t(1, 1, 8, 128), _t(1, 1, 9, 128))
    with pytest.raises(ValueError, match="divisible"):
        ops.launch_decode_flash_gqa_bf16_kernel(_t(1, 3, 1, 128), _t(1, 2, 8, 128), _t(1, 2, 8, 128))


def test_triton_prefill_launcher_error_behaviour_matches_upstream():
    # src/python/Triton/flash_gqa_kernel.py:226-252
    with pytest.raises(ValueError, match="bf16"):
        ops.launch_flash_gqa_forward_bf16_kernel(_t(4, 8, 128, dtype=torch.float32), _t(1, 8, 128), _t(1, 8, 128))
    with pytest.raises(ValueError, match="3D or 4D"):
        ops.launch_flash_gqa_forward_bf16_kernel(_t(8, 128), _t(8, 128), _t(8, 128))
    with pytest.raises(ValueError, match="matching ranks"):
        ops.launch_flash_gqa_forward_bf16_kernel(_t(4, 8, 128), _t(1, 1, 8, 128), _t(1, 8, 128))


def test_sparse_and_mla_launcher_error_behaviour_matches_upstream():
    """Argument checks of the sparse-index and MLA launchers, in upstream's order and wording, before any device work."""
    import torch
    import cuda_llm_ops_b200 as ops
    q = torch.zeros((1, 4, 8, 128), dtype=torch.bfloat16)
    k = torch.zeros((1, 2, 8, 128), dtype=torch.bfloat16)
    idx = torch.zeros((1, 2, 8, 4), dtype=torch.int32)
    with pytest.raises(ValueError, match="expects bf16 inputs"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q.float(), k, k, idx, 4)
    with pytest.raises(ValueError, match="must be int32"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k, k, idx.long(), 4)
    with pytest.raises(ValueError, match="must be 4D"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k, k, idx[0], 4)
    with pytest.raises(ValueError, match="num_sparse_kv must be an int"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k, k, idx, 4.0)
    with pytest.raises(ValueError, match="block_sparse_sub"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k, k, idx, 4, block_sparse_sub=0)
    with pytest.raises(ValueError, match="matching ranks"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k[0], k, idx, 4)
    with pytest.raises(ValueError, match="must have shape"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k, k, idx, 3)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k, k, idx, 4)

    qm = torch.zeros((4, 8, 192), dtype=torch.bfloat16)
    km = torch.zeros((2, 8, 192), dtype=torch.bfloat16)
    vm = torch.zeros((2, 8, 128), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="expects bf16 inputs"):
        ops.launch_flash_mla_forward_bf16_kernel(qm.float(), km, vm)
    with pytest.raises(ValueError, match="share head_dim_qk"):
        ops.launch_flash_mla_forward_bf16_kernel(qm, km[..., :128], vm)
    with pytest.raises(ValueError, match="share sequence length"):
        ops.launch_flash_mla_forward_bf16_kernel(qm, km, vm[:, :4])
    with pytest.raises(ValueError, match="number of KV heads"):
        ops.launch_flash_mla_forward_bf16_kernel(qm, km, vm[:1])
    with pytest.raises(ValueError, match="divisible by KV heads"):
        ops.launch_flash_mla_forward_bf16_kernel(qm[:3], km, vm)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.launch_flash_mla_forward_bf16_kernel(qm, km, vm)


def test_no_cpu_path():
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.gqa_decode(_t(1, 4, 128), _t(1, 1, 8, 128), _t(1, 1, 8, 128))
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.launch_flash_gqa_forward_bf16_kernel(_t(4, 8, 128), _t(1, 8, 128), _t(1, 8, 128))


def test_cpp_launcher_mirror_rejects_silently_like_upstream():
    # decode_flash_gqa_kernel.cu:416-437 returns without launching on shapes it refuses
    assert ops.LaunchFlashGqaBf16Kernel(None, None, None, 1.0, None, None, 0, 128, 16, 1, 128) is None
    assert ops.LaunchFlashGqaBf16Kernel(None, None, None, 1.0, None, None, 1, 128, 16, 1, 64) is None
    assert ops.LaunchFlashGqaBf16Kernel(None, None, None, 1.0, None, None, 1, 128, 5, 2, 128) is None


@pytest.mark.parametrize("batch,world", [(60, 1), (60, 2), (60, 4), (60, 8), (3, 8), (8, 8)])
def test_shard_batch_partitions(batch, world):
    spans = [ops.shard_batch(batch, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == batch
    assert all(a[1] == b[0] for a, b in zip(spans[:-1], spans[1:]))
    sizes = [e - b for b, e in spans]
    assert max(sizes) - min(sizes) <= 1


def test_shard_batch_60_over_8_matches_the_stated_split():
    assert [e - b for b, e in (ops.shard_batch(60, 8, r) for r in range(8))] == [8, 8, 8, 8, 7, 7, 7, 7]


@pytest.mark.parametrize("seq,world", [(1 << 20, 8), (1000, 4), (64, 4), (1, 2), (130, 3)])
def test_shard_kv_positions_partitions(seq, world):
    spans = [ops.shard_kv_positions(seq, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == seq
    assert all(a[1] == b[0] for a, b in zip(spans[:-1], spans[1:]))
    assert all(b % 64 == 0 for b, _ in spans if b < seq)
