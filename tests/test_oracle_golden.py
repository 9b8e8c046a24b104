"""The CPU oracle against upstream's own code: golden vectors from the upstream torch oracles, the
bit-identity run of the unmodified upstream C++ benchmark, and the oracle's internal consistency."""
import os
import re
import subprocess

import numpy as np
import pytest

import oracle_lib as ol

SCALE = 1.0 / np.sqrt(128.0)


def _case(golden, name):
    return {k: golden[name + "/" + k] for k in ("q", "k", "v", "o")}


@pytest.mark.parametrize("name", ["decode_g4", "decode_g16_rag", "decode_g8_tiny", "decode_g1"])
def test_decode_oracle_matches_upstream_torch_oracle(golden, name):
    c = _case(golden, name)
    q = c["q"][:, :, 0, :]
    got = ol.decode(q, c["k"], c["v"], SCALE, kv_layout=1)
    mx, mean, rel = ol.errors(got, c["o"][:, :, 0, :])
    # two fp32 formulations of the same tiled softmax: they may differ by an output ulp, no more
    assert mx <= 4e-3 and mean <= 2e-4 and rel <= 4e-3, (mx, mean, rel)


def test_decode_oracle_layouts_agree(golden):
    c = _case(golden, "decode_g4")
    q = c["q"][:, :, 0, :]
    a = ol.decode(q, c["k"], c["v"], SCALE, kv_layout=1)
    kb = np.ascontiguousarray(c["k"].transpose(0, 2, 1, 3))
    vb = np.ascontiguousarray(c["v"].transpose(0, 2, 1, 3))
    b = ol.decode(q, kb, vb, SCALE, kv_layout=0)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("name,causal", [("causal_g4", True), ("causal_g1", True), ("noncausal_g2", False)])
def test_prefill_oracle_matches_upstream_torch_oracle(golden, name, causal):
    c = _case(golden, name)
    q, k, v, o = c["q"], c["k"], c["v"], c["o"]
    if q.ndim == 3:
        q, k, v, o = q[None], k[None], v[None], o[None]
    got_o, got_lse = ol.prefill(q, k, v, SCALE, causal)
    mx, mean, rel = ol.errors(got_o, o)
    assert mx <= 4e-3 and mean <= 2e-4 and rel <= 4e-3, (mx, mean, rel)
    if causal:
        want_lse = golden[name + "/lse"]
        assert np.allclose(got_lse[0], want_lse, atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("name", ["swa_g4_w48", "swa_g2_w130"])
def test_swa_oracle_matches_upstream_torch_oracle(golden, name):
    q, k, v, o = (golden[name + "/" + t][None] for t in ("q", "k", "v", "o"))
    got_o, got_lse = ol.swa_prefill(q, k, v, SCALE, int(golden[name + "/window"]), golden[name + "/sink"])
    mx, mean, rel = ol.errors(got_o, o)
    assert mx <= 4e-3 and mean <= 2e-4 and rel <= 4e-3, (mx, mean, rel)
    assert np.allclose(got_lse[0], golden[name + "/lse"], atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("name", ["mla_g1", "mla_g2"])
def test_mla_oracle_matches_upstream_torch_oracle(golden, name):
    q, k, v, o = (golden[name + "/" + t][None] for t in ("q", "k", "v", "o"))
    got_o, got_lse = ol.mla_prefill(q, k, v, 1.0 / np.sqrt(192.0), True)
    mx, mean, rel = ol.errors(got_o, o)
    assert mx <= 4e-3 and mean <= 2e-4 and rel <= 4e-3, (mx, mean, rel)
    assert np.allclose(got_lse[0], golden[name + "/lse"], atol=2e-5, rtol=1e-5)


def test_mla_oracle_with_equal_head_dims_is_the_gqa_oracle():
    q = ol.randn_bf16((1, 4, 70, 128), 51)
    k = ol.randn_bf16((1, 2, 70, 128), 52)
    v = ol.randn_bf16((1, 2, 70, 128), 53)
    a_o, a_lse = ol.mla_prefill(q, k, v, SCALE, True)
    b_o, b_lse = ol.prefill(q, k, v, SCALE, True)
    assert np.array_equal(a_o, b_o) and np.array_equal(a_lse, b_lse)


@pytest.mark.parametrize("name", ["sgqa_g4_n40", "sgqa_g2_n16"])
def test_sgqa_oracle_matches_upstream_torch_oracle(golden, name):
    q, k, v, o = (golden[name + "/" + t][None] for t in ("q", "k", "v", "o"))
    got_o, got_lse = ol.sgqa_prefill(q, k, v, golden[name + "/idx"], SCALE, bool(golden[name + "/causal"]))
    mx, mean, rel = ol.errors(got_o, o)
    assert mx <= 4e-3 and mean <= 2e-4 and rel <= 4e-3, (mx, mean, rel)
    want_lse = golden[name + "/lse"]
    finite = np.isfinite(want_lse)
    assert np.array_equal(np.isfinite(got_lse[0]), finite)            # the empty list gives -inf in both
    assert np.allclose(got_lse[0][finite], want_lse[finite], atol=2e-5, rtol=1e-5)
    assert not finite.all()


def test_sgqa_oracle_with_the_full_causal_list_is_causal_attention():
    B, Hq, Hkv, S = 1, 4, 2, 40
    q = ol.randn_bf16((B, Hq, S, 128), 41)
    k = ol.randn_bf16((B, Hkv, S, 128), 42)
    v = ol.randn_bf16((B, Hkv, S, 128), 43)
    idx = np.broadcast_to(np.arange(S, dtype=np.int32)[::-1], (B, Hkv, S, S)).copy()   # every token, any order
    o_sparse, lse_sparse = ol.sgqa_prefill(q, k, v, idx, SCALE, causal=True)
    o_dense, lse_dense = ol.prefill(q, k, v, SCALE, True)
    mx, mean, rel = ol.errors(o_sparse, o_dense)
    assert mx <= 4e-3 and mean <= 2e-4, (mx, mean, rel)
    assert np.allclose(lse_sparse, lse_dense, atol=2e-5, rtol=1e-5)


def test_swa_oracle_with_a_window_wider_than_the_sequence_is_causal_attention_plus_sink():
    q = ol.randn_bf16((1, 2, 50, 128), 14)
    k = ol.randn_bf16((1, 1, 50, 128), 15)
    v = ol.randn_bf16((1, 1, 50, 128), 16)
    o_swa, lse_swa = ol.swa_prefill(q, k, v, SCALE, 1000, np.zeros(2, dtype=np.float32))
    o_c, lse_c = ol.prefill(q, k, v, SCALE, True)
    assert np.array_equal(o_swa, o_c) and np.allclose(lse_swa, lse_c, atol=1e-6)


def test_backward_oracle_matches_upstream_torch_oracle(golden):
    name = "bwd_g2"
    t = {key: golden[name + "/" + key][None] for key in ("q", "k", "v", "o", "grad_o", "dq", "dk", "dv")}
    gq, gk, gv = ol.backward(t["q"], t["k"], t["v"], t["o"], t["grad_o"], SCALE, True)
    for got, want, what in ((gq, t["dq"], "dq"), (gk, t["dk"], "dk"), (gv, t["dv"], "dv")):
        mx, mean, rel = ol.errors(got, want)
        assert rel <= 4e-3, (what, mx, mean, rel)  # two fp32 evaluation orders of the same formula, bf16 outputs


def test_swa_backward_oracle_matches_upstream_torch_oracle(golden):
    name = "swa_bwd_g2_w100"
    t = {key: golden[name + "/" + key][None] for key in ("q", "k", "v", "o", "grad_o", "dq", "dk", "dv")}
    gq, gk, gv = ol.swa_backward(t["q"], t["k"], t["v"], t["o"], t["grad_o"], SCALE, int(golden[name + "/window"]),
                                 golden[name + "/sink"])
    for got, want, what in ((gq, t["dq"], "dq"), (gk, t["dk"], "dk"), (gv, t["dv"], "dv")):
        mx, mean, rel = ol.errors(got, want)
        assert rel <= 4e-3, (what, mx, mean, rel)


def test_partials_combine_to_full_result():
    B, Hq, Hkv, S = 2, 8, 2, 300
    q = ol.randn_bf16((B, Hq, 128), 1)
    k = ol.randn_bf16((B, S, Hkv, 128), 2)
    v = ol.randn_bf16((B, S, Hkv, 128), 3)
    full = ol.decode(q, k, v, SCALE, 0)
    cuts = [0, 64, 64, 200, 300]  # includes an empty range
    parts = []
    for a, b in zip(cuts[:-1], cuts[1:]):
        _, ou, m, l = ol.decode(q, k, v, SCALE, 0, s_begin=a, s_end=b, want_partial=True)
        parts.append(ol.pack_partial(ou, m, l))
    merged, _ = ol.combine(np.stack(parts))
    mx, mean, rel = ol.errors(merged, full)
    assert mx <= 4e-3 and rel <= 5e-3, (mx, mean, rel)  # P is rounded to bf16 per tile; cuts move tile edges


def test_combine_ignores_empty_and_all_empty_rows():
    part = np.zeros((3, 1, 2, 130), dtype=np.float32)
    part[..., 128] = -np.inf
    part[1, 0, 0, :128] = 4.0
    part[1, 0, 0, 128] = 0.5
    part[1, 0, 0, 129] = 2.0
    o, of = ol.combine(part)
    assert np.allclose(of[0, 0], 2.0) and np.all(of[0, 1] == 0.0)


def test_causal_first_row_is_v0():
    q = ol.randn_bf16((1, 2, 5, 128), 4)
    k = ol.randn_bf16((1, 1, 5, 128), 5)
    v = ol.randn_bf16((1, 1, 5, 128), 6)
    o, lse = ol.prefill(q, k, v, SCALE, True)
    assert np.array_equal(o[0, :, 0, :], np.broadcast_to(v[0, 0, 0], (2, 128)))


@pytest.mark.skipif(not os.path.exists(ol.REF_BIN), reason="oracle/_ref not built (needs the upstream checkout)")
def test_unmodified_upstream_benchmark_agrees_bit_for_bit():
    """The upstream C++ program computes its CPU reference, then 'launches' -- through link-time stubs --
    this repository's restatement on the same random inputs and prints their relative error."""
    out = subprocess.run([ol.REF_BIN], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr
    m = re.search(r"O error = (\S+)", out.stdout)
    assert m, out.stdout
    assert float(m.group(1)) == 0.0, out.stdout
    assert re.search(r"CPU time = ", out.stdout)


@pytest.mark.skipif(not os.path.exists(ol.REF_ROPE_BIN), reason="oracle/_ref not built (needs the upstream checkout)")
def test_unmodified_upstream_rope_benchmark_agrees_bit_for_bit():
    """Upstream's test_rope.cu computes its CPU reference (B=1, S=512K, hidden=128) and compares it with what the
    'kernel' -- through link-time stubs, this repository's restatement -- produced."""
    out = subprocess.run([ol.REF_ROPE_BIN], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr
    m = re.search(r"RopeKernel error = (\S+)", out.stdout)
    assert m and float(m.group(1)) == 0.0, out.stdout


def test_rope_oracle_rotates_pairs_and_keeps_token_zero():
    x = ol.randn_bf16((2, 5, 16), 31)
    y = ol.rope(x)
    assert np.array_equal(y[:, 0], x[:, 0])  # angle 0
    xf, yf = ol.bf16_bits_to_f32(x), ol.bf16_bits_to_f32(y)
    # a rotation keeps the norm of every pair (up to bf16 rounding)
    assert np.allclose(xf[..., 0::2] ** 2 + xf[..., 1::2] ** 2, yf[..., 0::2] ** 2 + yf[..., 1::2] ** 2, rtol=2e-2, atol=1e-3)
