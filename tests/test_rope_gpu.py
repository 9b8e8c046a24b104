"""Rotary position embedding kernel against the CPU oracle (which is bit-identical to upstream's CPU reference)."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import to_bits, to_dev

pytestmark = pytest.mark.gpu


def _run(x, base=10000.0):
    import cuda_llm_ops_b200 as ops
    B, S, hidden = x.shape
    xin = to_dev(x)
    out = torch.zeros_like(xin)
    ops.LaunchRopeBf16Kernel(xin, out, B, S, hidden, base)
    torch.cuda.synchronize()
    return to_bits(out)


@pytest.mark.parametrize("B,S,hidden,base", [(1, 4096, 128, 10000.0), (3, 777, 64, 10000.0), (2, 100, 1024, 500000.0),
                                             (1, 1, 8, 10000.0)])
def test_parity_with_cpu_oracle(B, S, hidden, base):
    x = ol.randn_bf16((B, S, hidden), 501)
    got, want = _run(x, base), ol.rope(x, base)
    mx, mean, rel = ol.errors(got, want)
    # fp32 sine/cosine within an ulp of libm, rounded to bf16: at most a rounding flip here and there
    assert rel <= 1e-3 and mx <= 2e-2, (mx, mean, rel)
    assert (got != want).mean() <= 1e-3


def test_large_positions_of_upstream_benchmark_shape():
    """Upstream's shape (B=1, S=512K, hidden=128): angles reach 5e5 rad, where a fast-math sincos is useless."""
    S = 512 * 1024
    x = ol.randn_bf16((1, S, 128), 502)
    got = _run(x)
    tail = slice(S - 4096, S)  # the largest angles
    want = ol.rope(x)
    mx, mean, rel = ol.errors(got[:, tail], want[:, tail])
    assert rel <= 1e-3 and mx <= 2e-2, (mx, mean, rel)
    mx, mean, rel = ol.errors(got, want)
    assert rel <= 1e-3, (mx, mean, rel)


def test_in_place():
    import cuda_llm_ops_b200 as ops
    x = ol.randn_bf16((2, 300, 128), 503)
    t = to_dev(x)
    ops.LaunchRopeBf16Kernel(t, t, 2, 300, 128)
    torch.cuda.synchronize()
    assert np.array_equal(to_bits(t), _run(x))
