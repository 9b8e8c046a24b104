"""Parity of the tcgen05 prefill kernel (through the C ABI) with the CPU oracle and upstream's golden vectors."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import assert_clean_status, to_bits, to_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)
LSE_TOL = 2e-3  # fp32 log-sum-exp, absolute


def _run(q, k, v, causal, scale=None):
    import cuda_llm_ops_b200 as ops
    out, lse = ops.launch_flash_gqa_forward_bf16_kernel(to_dev(q), to_dev(k), to_dev(v), scale=scale, causal=causal)
    torch.cuda.synchronize()
    return to_bits(out), lse.cpu().numpy()


@pytest.mark.parametrize("name,causal", [("causal_g4", True), ("causal_g1", True)])
def test_golden_causal_vectors_from_upstream_torch_oracle(golden, name, causal):
    # upstream's un-batched 3-D calling convention
    got_o, got_lse = _run(golden[name + "/q"], golden[name + "/k"], golden[name + "/v"], causal)
    ol.assert_parity(got_o, golden[name + "/o"], name)
    assert np.allclose(got_lse, golden[name + "/lse"], atol=LSE_TOL)
    assert_clean_status()


def test_golden_noncausal_vectors_from_upstream_torch_oracle(golden):
    name = "noncausal_g2"
    got_o, _ = _run(golden[name + "/q"], golden[name + "/k"], golden[name + "/v"], False)
    ol.assert_parity(got_o, golden[name + "/o"], name)


# (B, Hq, Hkv, Sq, Skv)
CASES = [
    (1, 4, 1, 256, 256),
    (1, 2, 2, 128, 128),
    (2, 8, 2, 384, 384),      # odd number of 128-row tiles
    (1, 4, 2, 200, 200),      # ragged query and kv tails
    (1, 2, 1, 1, 1),
    (1, 3, 1, 70, 300),       # Sq != Skv
    (1, 16, 1, 640, 640),     # group 16, like the headline prefill config
    (1, 2, 1, 1024, 1024),
    # query chunks of at most 64 rows: heads of a group share one tile
    (2, 8, 2, 64, 500),       # 2 heads x 64 rows
    (1, 16, 1, 16, 300),      # 8 heads x 16 rows
    (1, 16, 1, 1, 700),       # 16 heads x 1 row: part of the tile stays empty
    (1, 6, 1, 33, 257),       # group of 6: 2 heads x 64 rows, rows 33..63 of each head beyond the chunk
    (2, 4, 2, 5, 130),        # group of 2: 2 heads x 8 rows
    (1, 3, 1, 20, 200),       # odd group: no sharing
    (3, 32, 2, 7, 129),       # 16 heads x 8 rows
]


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv", CASES)
def test_parity_with_cpu_oracle(B, Hq, Hkv, Sq, Skv, causal):
    q = ol.randn_bf16((B, Hq, Sq, 128), 101)
    k = ol.randn_bf16((B, Hkv, Skv, 128), 102)
    v = ol.randn_bf16((B, Hkv, Skv, 128), 103)
    want_o, want_lse = ol.prefill(q, k, v, SCALE, causal)
    got_o, got_lse = _run(q, k, v, causal)
    ol.assert_parity(got_o, want_o, "B%d Hq%d Hkv%d Sq%d Skv%d causal%d" % (B, Hq, Hkv, Sq, Skv, causal))
    assert np.allclose(got_lse, want_lse, atol=LSE_TOL), np.abs(got_lse - want_lse).max()
    assert_clean_status()


def test_peaked_scores_exercise_the_rescale_path():
    # growing keys make the running maximum jump by more than the lazy-rescale threshold many times
    B, Hq, Hkv, S = 1, 2, 1, 1024
    q = ol.randn_bf16((B, Hq, S, 128), 111, std=2.0)
    kf = np.random.default_rng(112).standard_normal((B, Hkv, S, 128)).astype(np.float32)
    kf *= np.linspace(0.2, 4.0, S, dtype=np.float32)[None, None, :, None]
    k = ol.f32_to_bf16_bits(kf)
    v = ol.randn_bf16((B, Hkv, S, 128), 113)
    for causal in (False, True):
        want_o, want_lse = ol.prefill(q, k, v, SCALE, causal)
        got_o, got_lse = _run(q, k, v, causal)
        ol.assert_parity(got_o, want_o, "peaked causal=%d" % causal)
        assert np.allclose(got_lse, want_lse, atol=5e-3, rtol=1e-4)
    assert_clean_status()


@pytest.mark.parametrize("causal", [False, True])
def test_negative_scale_turns_the_row_maximum_into_a_minimum(causal):
    """The kernel takes the row extreme on the raw scores; with a negative scale that is the minimum."""
    B, Hq, Hkv, Sq, Skv = 1, 4, 2, 384, 500
    q = ol.randn_bf16((B, Hq, Sq, 128), 121)
    k = ol.randn_bf16((B, Hkv, Skv, 128), 122)
    v = ol.randn_bf16((B, Hkv, Skv, 128), 123)
    want_o, want_lse = ol.prefill(q, k, v, -SCALE, causal)
    got_o, got_lse = _run(q, k, v, causal, scale=-SCALE)
    ol.assert_parity(got_o, want_o, "negative scale causal=%d" % causal)
    assert np.allclose(got_lse, want_lse, atol=LSE_TOL), np.abs(got_lse - want_lse).max()
    assert_clean_status()


def test_headline_prefill_shape_sampled_rows():
    """Baseline config 3 (B=1, S=4096, Hq=16, Hkv=1, non-causal) at full size; rows sampled for the oracle."""
    import cuda_llm_ops_b200 as ops
    Hq, S = 16, 4096
    g = torch.Generator(device="cuda").manual_seed(4321)
    q = torch.randn((1, Hq, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((1, 1, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((1, 1, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    for causal in (False, True):
        out, lse = ops.launch_flash_gqa_forward_bf16_kernel(q, k, v, causal=causal)
        torch.cuda.synchronize()
        got = to_bits(out)
        qb, kb, vb = to_bits(q), to_bits(k), to_bits(v)
        for r0 in (0, 127, 1920, 4064):
            want_o, want_lse = ol.prefill(qb, kb, vb, SCALE, causal, row_begin=r0, row_end=r0 + 32)
            ol.assert_parity(got[:, :, r0:r0 + 32], want_o[:, :, r0:r0 + 32], "rows %d causal=%d" % (r0, causal))
            assert np.allclose(lse.cpu().numpy()[:, :, r0:r0 + 32], want_lse[:, :, r0:r0 + 32], atol=LSE_TOL)
    assert_clean_status()


def test_long_causal_shape_at_full_size_sampled_rows():
    """Baseline config 5 (B=8, S=16384, Hq=64, Hkv=8, causal) whole on one GPU: Q and O are 2 GiB each, so the last
    sequence sits beyond the reach of 32-bit byte offsets.  Sampled row windows of the first and last sequence (the
    first rows, a 128-row tile boundary, the middle, the last rows) are checked against the oracle."""
    import cuda_llm_ops_b200 as ops
    B, Hq, Hkv, S = 8, 64, 8, 16384
    g = torch.Generator(device="cuda").manual_seed(555)
    q = torch.empty((B, Hq, S, 128), dtype=torch.bfloat16, device="cuda")
    k = torch.empty((B, Hkv, S, 128), dtype=torch.bfloat16, device="cuda")
    v = torch.empty((B, Hkv, S, 128), dtype=torch.bfloat16, device="cuda")
    for b in range(B):   # one sequence at a time keeps the fp32 temporaries small
        q[b] = torch.randn((Hq, S, 128), generator=g, device="cuda").to(torch.bfloat16)
        k[b] = torch.randn((Hkv, S, 128), generator=g, device="cuda").to(torch.bfloat16)
        v[b] = torch.randn((Hkv, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    out, lse = ops.launch_flash_gqa_forward_bf16_kernel(q, k, v, causal=True)
    torch.cuda.synchronize()
    assert_clean_status()
    for b in (0, B - 1):
        qb, kb, vb = to_bits(q[b:b + 1]), to_bits(k[b:b + 1]), to_bits(v[b:b + 1])
        for r0 in (0, 124, 8188, S - 8):
            want_o, want_lse = ol.prefill(qb, kb, vb, SCALE, True, row_begin=r0, row_end=r0 + 8)
            got_o = to_bits(out[b:b + 1, :, r0:r0 + 8].contiguous())
            got_lse = lse[b:b + 1, :, r0:r0 + 8].cpu().numpy()
            ol.assert_parity(got_o, want_o[:, :, r0:r0 + 8], "sequence %d rows %d" % (b, r0))
            assert np.allclose(got_lse, want_lse[:, :, r0:r0 + 8], atol=LSE_TOL)


# Query chunks against a long cache (non-causal): the heads of a group become extra rows of the two-tile kernel and,
# with a workspace, the kv range is shared out among blocks and merged.  (B, Hq, Hkv, Sq, Skv)
CHUNK_CASES = [
    (2, 16, 2, 64, 4096),     # 8 heads x 64 rows = 512 rows per kv head, kv range cut four ways
    (1, 8, 2, 100, 2500),     # rows 400..511 of the merged tile pair empty, ragged kv tail, two shares
    (1, 4, 4, 200, 3000),     # no grouping: shares only
    (1, 32, 1, 8, 6000),      # 32 heads x 8 rows = 256 rows, many shares
    (32, 16, 2, 64, 1024),    # enough (batch, kv head) pairs to fill the GPU: merged rows, no shares
]


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv", CHUNK_CASES)
def test_query_chunk_against_long_cache(B, Hq, Hkv, Sq, Skv):
    import cuda_llm_ops_b200 as ops
    from cuda_llm_ops_b200 import _lib
    q = ol.randn_bf16((B, Hq, Sq, 128), 151)
    k = ol.randn_bf16((B, Hkv, Skv, 128), 152)
    v = ol.randn_bf16((B, Hkv, Skv, 128), 153)
    want_o, want_lse = ol.prefill(q, k, v, SCALE, False)
    # through the launcher (brings its own scratch) ...
    got_o, got_lse = _run(q, k, v, False)
    ol.assert_parity(got_o, want_o, "chunk, launcher")
    assert np.allclose(got_lse, want_lse, atol=LSE_TOL), np.abs(got_lse - want_lse).max()
    # ... through the C ABI with a caller-owned workspace of the size the library asks for, and without one
    lib = _lib.load()
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    need = int(lib.cllo_gqa_prefill_workspace_bytes(B, Sq, Skv, Hq, Hkv, 0))
    for with_ws in (True, False):
        o = torch.zeros((B, Hq, Sq, 128), dtype=torch.bfloat16, device="cuda")
        lse = torch.zeros((B, Hq, Sq), dtype=torch.float32, device="cuda")
        ws = torch.full((max(need, 16),), 0xFF, dtype=torch.uint8, device="cuda")  # NaN patterns: nothing may be read unwritten
        rc = lib.cllo_gqa_prefill_fwd_ws_bf16(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), SCALE, 0, o.data_ptr(),
                                              lse.data_ptr(), ws.data_ptr() if with_ws else None, need if with_ws else 0,
                                              B, Sq, Skv, Hq, Hkv, 128, None)
        assert rc == 0
        torch.cuda.synchronize()
        ol.assert_parity(to_bits(o), want_o, "chunk, C ABI, workspace=%s" % with_ws)
        assert np.allclose(lse.cpu().numpy(), want_lse, atol=LSE_TOL)
    # a workspace that is too small is simply not used
    rc = lib.cllo_gqa_prefill_fwd_ws_bf16(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), SCALE, 0, o.data_ptr(),
                                          lse.data_ptr(), ws.data_ptr(), 16, B, Sq, Skv, Hq, Hkv, 128, None)
    assert rc == 0
    torch.cuda.synchronize()
    ol.assert_parity(to_bits(o), want_o, "chunk, C ABI, tiny workspace")
    assert_clean_status()
