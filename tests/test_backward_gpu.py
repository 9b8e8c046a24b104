"""GQA attention backward (tcgen05 dQ and dK/dV kernels) against upstream's golden vectors and the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import assert_clean_status, to_bits, to_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def _forward_then_backward(q, k, v, grad_o, causal):
    import cuda_llm_ops_b200 as ops
    qd, kd, vd, god = to_dev(q), to_dev(k), to_dev(v), to_dev(grad_o)
    o, lse = ops.launch_flash_gqa_forward_bf16_kernel(qd, kd, vd, causal=causal)
    dq, dk, dv = ops.launch_flash_gqa_backward_bf16_kernel(qd, kd, vd, o, lse, god, causal=causal)
    torch.cuda.synchronize()
    return to_bits(o), to_bits(dq), to_bits(dk), to_bits(dv)


def test_golden_vectors_from_upstream_torch_oracle(golden):
    import cuda_llm_ops_b200 as ops
    name = "bwd_g2"
    # upstream's un-batched convention, with upstream's own O and lse as inputs
    t = {key: to_dev(golden[name + "/" + key]) for key in ("q", "k", "v", "o", "grad_o")}
    lse = torch.from_numpy(golden[name + "/lse"]).cuda()
    dq, dk, dv = ops.launch_flash_gqa_backward_bf16_kernel(t["q"], t["k"], t["v"], t["o"], lse, t["grad_o"])
    torch.cuda.synchronize()
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        ol.assert_grad_parity(to_bits(got), golden[name + "/" + key], key)
    assert_clean_status()


# (B, Hq, Hkv, Sq, Skv)
CASES = [
    (1, 2, 1, 128, 128),
    (1, 4, 2, 256, 256),
    (2, 4, 1, 200, 200),      # group 4 summed into one kv head, ragged tails
    (1, 2, 2, 384, 384),
    (1, 2, 1, 70, 300),       # Sq != Skv
    (1, 2, 1, 300, 70),
    (1, 8, 1, 512, 512),
]


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv", CASES)
def test_parity_with_cpu_oracle(B, Hq, Hkv, Sq, Skv, causal):
    q = ol.randn_bf16((B, Hq, Sq, 128), 401)
    k = ol.randn_bf16((B, Hkv, Skv, 128), 402)
    v = ol.randn_bf16((B, Hkv, Skv, 128), 403)
    grad_o = ol.randn_bf16((B, Hq, Sq, 128), 404)
    o, dq, dk, dv = _forward_then_backward(q, k, v, grad_o, causal)
    want_q, want_k, want_v = ol.backward(q, k, v, o, grad_o, SCALE, causal)
    what = "B%d Hq%d Hkv%d Sq%d Skv%d causal%d " % (B, Hq, Hkv, Sq, Skv, causal)
    ol.assert_grad_parity(dq, want_q, what + "dq")
    ol.assert_grad_parity(dk, want_k, what + "dk")
    ol.assert_grad_parity(dv, want_v, what + "dv")
    assert_clean_status()


def test_deterministic():
    q = ol.randn_bf16((1, 4, 384, 128), 411)
    k = ol.randn_bf16((1, 1, 384, 128), 412)
    v = ol.randn_bf16((1, 1, 384, 128), 413)
    g = ol.randn_bf16((1, 4, 384, 128), 414)
    first = _forward_then_backward(q, k, v, g, True)
    for _ in range(3):
        again = _forward_then_backward(q, k, v, g, True)
        assert all(np.array_equal(a, b) for a, b in zip(first, again))


def _gpu_case(B, Hq, Hkv, S, seed):
    import cuda_llm_ops_b200 as ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((B, Hq, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((B, Hkv, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((B, Hkv, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    grad_o = torch.randn((B, Hq, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    o, lse = ops.launch_flash_gqa_forward_bf16_kernel(q, k, v, causal=True)
    dq, dk, dv = ops.launch_flash_gqa_backward_bf16_kernel(q, k, v, o, lse, grad_o, causal=True)
    torch.cuda.synchronize()
    return q, k, v, grad_o, o, dq, dk, dv


def test_upstream_shape_whole_tensors():
    """Upstream's benchmark shape (B=1, S=4096, 16 query heads on one kv head, causal): here the 16 heads of the group
    are divided among blocks and a reduction kernel sums their fp32 partials.  Whole gradients against the oracle."""
    q, k, v, grad_o, o, dq, dk, dv = _gpu_case(1, 16, 1, 4096, 431)
    want_q, want_k, want_v = ol.backward(to_bits(q), to_bits(k), to_bits(v), to_bits(o), to_bits(grad_o), SCALE, True)
    ol.assert_grad_parity(to_bits(dq), want_q, "upstream shape dq")
    ol.assert_grad_parity(to_bits(dk), want_k, "upstream shape dk")
    ol.assert_grad_parity(to_bits(dv), want_v, "upstream shape dv")
    assert_clean_status()


def test_large_shape_slices():
    """B=2, S=8192, Hq=32, Hkv=4, causal (the other shape whose throughput is quoted); the oracle would need minutes
    for it.  A (batch, kv head) slice is a closed problem -- its 8 query heads see only that kv head -- so (1) the
    same slice run alone (another grid, another division of the heads among blocks) must give the same gradients,
    and (2) under the causal mask the first n query rows see only the first n keys, so their grad_q is checked
    against the oracle on that prefix."""
    import cuda_llm_ops_b200 as ops
    B, Hq, Hkv, S = 2, 32, 4, 8192
    G = Hq // Hkv
    q, k, v, grad_o, o, dq, dk, dv = _gpu_case(B, Hq, Hkv, S, 432)
    for b, h in [(1, 3), (0, 0)]:
        hs = slice(h * G, (h + 1) * G)
        qs, ks, vs = q[b:b + 1, hs].contiguous(), k[b:b + 1, h:h + 1].contiguous(), v[b:b + 1, h:h + 1].contiguous()
        gs = grad_o[b:b + 1, hs].contiguous()
        o_s, lse_s = ops.launch_flash_gqa_forward_bf16_kernel(qs, ks, vs, causal=True)
        dq_s, dk_s, dv_s = ops.launch_flash_gqa_backward_bf16_kernel(qs, ks, vs, o_s, lse_s, gs, causal=True)
        torch.cuda.synchronize()
        ol.assert_grad_parity(to_bits(dq[b:b + 1, hs]), to_bits(dq_s), "slice (%d,%d) dq vs slice alone" % (b, h))
        ol.assert_grad_parity(to_bits(dk[b:b + 1, h:h + 1]), to_bits(dk_s), "slice (%d,%d) dk vs slice alone" % (b, h))
        ol.assert_grad_parity(to_bits(dv[b:b + 1, h:h + 1]), to_bits(dv_s), "slice (%d,%d) dv vs slice alone" % (b, h))
    n = 1280
    b, h = 1, 3
    hs = slice(h * G, (h + 1) * G)
    want_q, _, _ = ol.backward(to_bits(q[b:b + 1, hs, :n]), to_bits(k[b:b + 1, h:h + 1, :n]),
                               to_bits(v[b:b + 1, h:h + 1, :n]), to_bits(o[b:b + 1, hs, :n]),
                               to_bits(grad_o[b:b + 1, hs, :n]), SCALE, True)
    ol.assert_grad_parity(to_bits(dq[b:b + 1, hs, :n]), want_q, "first %d rows dq vs oracle" % n)
    assert_clean_status()
