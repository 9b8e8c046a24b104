"""Helpers shared by the GPU parity tests: move bf16 bit patterns between numpy and CUDA tensors."""
import numpy as np
import torch


def to_dev(bits):
    """uint16 bf16 bit patterns (numpy) -> CUDA bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def to_bits(t):
    """CUDA/CPU bf16 tensor -> uint16 numpy bit patterns."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def assert_clean_status():
    import cuda_llm_ops_b200 as ops
    rc, detail = ops.device_status()
    assert rc == 0, "device status %d detail %s" % (rc, detail)
