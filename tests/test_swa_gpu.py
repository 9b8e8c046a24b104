"""Sliding-window + sink forward (the mask variant of the prefill kernel) against upstream's golden vectors and the oracle."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import assert_clean_status, to_bits, to_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def _run(q, k, v, window, sink):
    import cuda_llm_ops_b200 as ops
    out, lse = ops.launch_flash_swa_forward_bf16_kernel(to_dev(q), to_dev(k), to_dev(v), window_size=window,
                                                        sink_value=torch.from_numpy(np.asarray(sink)).cuda())
    torch.cuda.synchronize()
    return to_bits(out), lse.cpu().numpy()


@pytest.mark.parametrize("name", ["swa_g4_w48", "swa_g2_w130"])
def test_golden_vectors_from_upstream_torch_oracle(golden, name):
    got_o, got_lse = _run(golden[name + "/q"], golden[name + "/k"], golden[name + "/v"], int(golden[name + "/window"]),
                          golden[name + "/sink"])
    ol.assert_parity(got_o, golden[name + "/o"], name)
    assert np.allclose(got_lse, golden[name + "/lse"], atol=2e-3)
    assert_clean_status()


# (B, Hq, Hkv, Sq, Skv, window): windows inside one tile, across tile edges, wider than the sequence, of one token
CASES = [
    (1, 4, 1, 512, 512, 64),
    (1, 2, 2, 700, 700, 129),
    (2, 8, 2, 384, 384, 256),
    (1, 4, 2, 300, 300, 1),
    (1, 2, 1, 260, 260, 4096),
    (1, 2, 1, 1024, 1024, 300),
    (1, 2, 1, 400, 200, 100),     # more queries than keys: the last rows see nothing
]


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,window", CASES)
def test_parity_with_cpu_oracle(B, Hq, Hkv, Sq, Skv, window):
    q = ol.randn_bf16((B, Hq, Sq, 128), 201)
    k = ol.randn_bf16((B, Hkv, Skv, 128), 202)
    v = ol.randn_bf16((B, Hkv, Skv, 128), 203)
    sink = np.linspace(0.0, 3.0, Hq).astype(np.float32)
    want_o, want_lse = ol.swa_prefill(q, k, v, SCALE, window, sink)
    got_o, got_lse = _run(q, k, v, window, sink)
    ol.assert_parity(got_o, want_o, "B%d Hq%d Hkv%d Sq%d Skv%d w%d" % (B, Hq, Hkv, Sq, Skv, window))
    assert np.allclose(got_lse, want_lse, atol=2e-3), np.abs(got_lse - want_lse).max()
    assert_clean_status()


def test_long_sequence_with_upstream_window_sampled_rows():
    """Upstream's benchmark shape family (window 512) at S=8192: only ~5 KV tiles per block are visited."""
    import cuda_llm_ops_b200 as ops
    Hq, S, window = 8, 8192, 512
    g = torch.Generator(device="cuda").manual_seed(77)
    q = torch.randn((1, Hq, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((1, 1, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((1, 1, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    sink = torch.full((Hq,), 0.5, device="cuda")
    out, lse = ops.launch_flash_swa_forward_bf16_kernel(q, k, v, window_size=window, sink_value=sink)
    torch.cuda.synchronize()
    got = to_bits(out)
    for r0 in (0, 500, 4090, 8160):
        sl = slice(max(0, r0 - window), r0 + 32)  # everything rows r0..r0+31 can see
        off = r0 - sl.start
        want_o, want_lse = ol.swa_prefill(to_bits(q[:, :, sl]), to_bits(k[:, :, sl]), to_bits(v[:, :, sl]), SCALE, window,
                                          sink.cpu().numpy())
        ol.assert_parity(got[:, :, r0:r0 + 32], want_o[:, :, off:off + 32], "rows %d" % r0)
        assert np.allclose(lse.cpu().numpy()[:, :, r0:r0 + 32], want_lse[:, :, off:off + 32], atol=2e-3)
    assert_clean_status()


def test_backward_golden_vectors_from_upstream_torch_oracle(golden):
    import cuda_llm_ops_b200 as ops
    name = "swa_bwd_g2_w100"
    t = {key: to_dev(golden[name + "/" + key]) for key in ("q", "k", "v", "o", "grad_o")}
    lse = torch.from_numpy(golden[name + "/lse"]).cuda()
    dq, dk, dv = ops.launch_flash_swa_backward_bf16_kernel(t["q"], t["k"], t["v"], t["o"], lse, t["grad_o"],
                                                           window_size=int(golden[name + "/window"]))
    torch.cuda.synchronize()
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        ol.assert_grad_parity(to_bits(got), golden[name + "/" + key], key)
    assert_clean_status()


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,window", [(1, 4, 1, 512, 512, 64), (1, 2, 2, 700, 700, 129), (2, 4, 2, 384, 384, 256),
                                                    (1, 2, 1, 300, 300, 1), (1, 2, 1, 260, 260, 4096), (1, 2, 1, 400, 200, 100)])
def test_backward_parity_with_cpu_oracle(B, Hq, Hkv, Sq, Skv, window):
    import cuda_llm_ops_b200 as ops
    q = ol.randn_bf16((B, Hq, Sq, 128), 211)
    k = ol.randn_bf16((B, Hkv, Skv, 128), 212)
    v = ol.randn_bf16((B, Hkv, Skv, 128), 213)
    g = ol.randn_bf16((B, Hq, Sq, 128), 214)
    sink = np.linspace(0.2, 2.0, Hq).astype(np.float32)
    qd, kd, vd, gd = to_dev(q), to_dev(k), to_dev(v), to_dev(g)
    o, lse = ops.launch_flash_swa_forward_bf16_kernel(qd, kd, vd, window_size=window, sink_value=torch.from_numpy(sink).cuda())
    dq, dk, dv = ops.launch_flash_swa_backward_bf16_kernel(qd, kd, vd, o, lse, gd, window_size=window)
    torch.cuda.synchronize()
    want = ol.swa_backward(q, k, v, to_bits(o), g, SCALE, window, sink)
    what = "B%d Hq%d Hkv%d Sq%d Skv%d w%d " % (B, Hq, Hkv, Sq, Skv, window)
    for got, ref, key in zip((dq, dk, dv), want, ("dq", "dk", "dv")):
        ol.assert_grad_parity(to_bits(got), ref, what + key)
    assert_clean_status()
