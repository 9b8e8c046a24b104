"""MLA-shaped forward (head_dim_qk = 192, head_dim_v = 128) against upstream's golden vectors and the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import assert_clean_status, to_bits, to_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(192.0)


def _run(q, k, v, causal=True, squeeze=False, scale=None):
    import cuda_llm_ops_b200 as ops
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    if squeeze:
        qd, kd, vd = qd[0], kd[0], vd[0]
    out, lse = ops.launch_flash_mla_forward_bf16_kernel(qd, kd, vd, scale=scale, causal=causal)
    torch.cuda.synchronize()
    if squeeze:
        out, lse = out[None], lse[None]
    return to_bits(out), lse.cpu().numpy()


@pytest.mark.parametrize("name", ["mla_g1", "mla_g2"])
def test_golden_vectors_from_upstream_torch_oracle(golden, name):
    q, k, v = (golden[name + "/" + t][None] for t in ("q", "k", "v"))
    got_o, got_lse = _run(q, k, v, True, squeeze=True)
    ol.assert_parity(got_o[0], golden[name + "/o"], name)
    assert np.allclose(got_lse[0], golden[name + "/lse"], atol=2e-3)
    assert_clean_status()


# (B, Hq, Hkv, Sq, Skv, causal): one kv tile, two (the prologue only), three and more (the steady loop), ragged tails,
# more keys than queries and the reverse, grouped heads
CASES = [
    (1, 2, 2, 64, 64, True),
    (1, 2, 2, 128, 128, True),
    (1, 2, 1, 256, 256, True),
    (1, 4, 4, 384, 384, True),
    (2, 4, 2, 700, 700, True),
    (1, 16, 16, 1024, 1024, True),       # upstream's head layout (16 heads, no grouping)
    (1, 2, 2, 300, 520, False),
    (1, 2, 1, 520, 300, False),
    (1, 8, 2, 200, 1000, False),
    (1, 2, 2, 450, 130, True),           # rows beyond the last key see every key
    (2, 8, 2, 40, 300, False),           # short query chunk: 2 heads of a group x 64 rows share the tile
    (1, 16, 1, 3, 200, True),            # 16 heads x 4 rows
    (1, 16, 2, 16, 129, False),          # 8 heads x 16 rows
]


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal", CASES)
def test_parity_with_cpu_oracle(B, Hq, Hkv, Sq, Skv, causal):
    q = ol.randn_bf16((B, Hq, Sq, 192), 401)
    k = ol.randn_bf16((B, Hkv, Skv, 192), 402)
    v = ol.randn_bf16((B, Hkv, Skv, 128), 403)
    want_o, want_lse = ol.mla_prefill(q, k, v, SCALE, causal)
    got_o, got_lse = _run(q, k, v, causal)
    tag = "B%d Hq%d Hkv%d Sq%d Skv%d causal%d" % (B, Hq, Hkv, Sq, Skv, causal)
    ol.assert_parity(got_o, want_o, tag)
    assert np.allclose(got_lse, want_lse, atol=2e-3), (tag, np.abs(got_lse - want_lse).max())
    assert_clean_status()


def test_large_scores_exercise_the_rescaling_of_o():
    """Scores that keep growing along the sequence force the running maximum up again and again."""
    B, Hq, Hkv, S = 1, 2, 2, 640
    q = ol.randn_bf16((B, Hq, S, 192), 411)
    k = ol.randn_bf16((B, Hkv, S, 192), 412)
    v = ol.randn_bf16((B, Hkv, S, 128), 413)
    scale = 0.6                                   # logits of tens of units
    want_o, want_lse = ol.mla_prefill(q, k, v, scale, True)
    got_o, got_lse = _run(q, k, v, True, scale=scale)
    ol.assert_parity(got_o, want_o, "large scores")
    assert np.allclose(got_lse, want_lse, atol=2e-2, rtol=1e-4)
    assert_clean_status()


@pytest.mark.parametrize("causal", [False, True])
def test_negative_scale(causal):
    B, Hq, Hkv, Sq, Skv = 1, 4, 2, 300, 420
    q = ol.randn_bf16((B, Hq, Sq, 192), 421)
    k = ol.randn_bf16((B, Hkv, Skv, 192), 422)
    v = ol.randn_bf16((B, Hkv, Skv, 128), 423)
    want_o, want_lse = ol.mla_prefill(q, k, v, -SCALE, causal)
    got_o, got_lse = _run(q, k, v, causal, scale=-SCALE)
    ol.assert_parity(got_o, want_o, "negative scale causal=%d" % causal)
    assert np.allclose(got_lse, want_lse, atol=2e-3), np.abs(got_lse - want_lse).max()
    assert_clean_status()


def test_upstream_shape_sampled_rows():
    """Upstream's benchmark shape (S = 4096, 16 heads, no grouping), rows checked by sampling."""
    import cuda_llm_ops_b200 as ops
    H, S = 16, 4096
    g = torch.Generator(device="cuda").manual_seed(93)
    q = torch.randn((1, H, S, 192), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((1, H, S, 192), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((1, H, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    out, lse = ops.launch_flash_mla_forward_bf16_kernel(q, k, v, causal=True)
    torch.cuda.synchronize()
    rows = [0, 1, 127, 128, 129, 1000, 2047, 2048, 4095]
    qn, kn, vn = to_bits(q), to_bits(k), to_bits(v)
    for row in rows:
        # a causal row depends on the keys up to it only: the oracle gets the prefix
        want_o, want_lse = ol.mla_prefill(qn[:, :, row:row + 1], kn[:, :, :row + 1], vn[:, :, :row + 1], SCALE, False)
        ol.assert_parity(to_bits(out)[:, :, row:row + 1], want_o, "row %d" % row)
        assert np.allclose(lse.cpu().numpy()[:, :, row:row + 1], want_lse, atol=2e-3)
    assert_clean_status()


def test_launcher_checks_like_upstream():
    import cuda_llm_ops_b200 as ops
    q = torch.zeros((1, 4, 8, 192), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((1, 2, 8, 192), dtype=torch.bfloat16, device="cuda")
    v = torch.zeros((1, 2, 8, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="bf16"):
        ops.launch_flash_mla_forward_bf16_kernel(q.float(), k, v)
    with pytest.raises(ValueError, match="share head_dim_qk"):
        ops.launch_flash_mla_forward_bf16_kernel(q, k[..., :128].contiguous(), v)
    with pytest.raises(ValueError, match="divisible"):
        ops.launch_flash_mla_forward_bf16_kernel(q[:, :3], k, v)
    with pytest.raises(ValueError, match="sequence length"):
        ops.launch_flash_mla_forward_bf16_kernel(q, k, v[:, :, :4].contiguous())
