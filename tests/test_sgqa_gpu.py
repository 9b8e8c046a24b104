"""Sparse-index GQA forward against upstream's golden vectors and the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import assert_clean_status, to_bits, to_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def _run(q, k, v, idx, causal=True, squeeze=False):
    import cuda_llm_ops_b200 as ops
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    if squeeze:
        qd, kd, vd = qd[0], kd[0], vd[0]
    idx_d = torch.from_numpy(np.ascontiguousarray(idx, dtype=np.int32)).cuda()
    out, lse = ops.launch_flash_sgqa_forward_bf16_kernel(qd, kd, vd, idx_d, int(idx.shape[-1]), causal=causal)
    torch.cuda.synchronize()
    if squeeze:
        out, lse = out[None], lse[None]
    return to_bits(out), lse.cpu().numpy()


def _check_lse(got, want, tag):
    finite = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), finite), tag
    assert np.all(got[~finite] == -np.inf), tag
    assert np.allclose(got[finite], want[finite], atol=2e-3), (tag, np.abs(got[finite] - want[finite]).max())


@pytest.mark.parametrize("name", ["sgqa_g4_n40", "sgqa_g2_n16"])
def test_golden_vectors_from_upstream_torch_oracle(golden, name):
    q, k, v = (golden[name + "/" + t][None] for t in ("q", "k", "v"))
    got_o, got_lse = _run(q, k, v, golden[name + "/idx"], bool(golden[name + "/causal"]), squeeze=True)
    ol.assert_parity(got_o[0], golden[name + "/o"], name)
    _check_lse(got_lse[0], golden[name + "/lse"], name)
    assert_clean_status()


def _lists(rng, B, Hkv, Sq, Skv, n, causal, pad_share=0.2):
    """Random lists: unique valid entries, then padding; some hostile entries on top."""
    idx = np.full((B, Hkv, Sq, n), -1, dtype=np.int32)
    for b in range(B):
        for h in range(Hkv):
            for i in range(Sq):
                hi = min(i, Skv - 1) if causal else Skv - 1
                take = min(n, hi + 1)
                take = max(0, take - int(rng.integers(0, max(1, int(pad_share * n)))))
                idx[b, h, i, :take] = rng.permutation(hi + 1)[:take]
    flat = idx.reshape(-1, n)
    rows = rng.integers(0, flat.shape[0], size=max(4, flat.shape[0] // 10))
    for r in rows[0::4]:
        flat[r, rng.integers(0, n)] = Skv + int(rng.integers(0, 1000))     # out of range
    for r in rows[1::4]:
        flat[r, rng.integers(0, n)] = flat[r, 0]                            # a repeated entry
    for r in rows[2::4]:
        flat[r, :] = -1                                                     # an empty list
    for r in rows[3::4]:
        flat[r, rng.integers(0, n)] = -5                                    # negative but not -1
    return idx


# (B, Hq, Hkv, Sq, Skv, n_sparse, causal)
CASES = [
    (1, 16, 1, 200, 200, 64, True),      # upstream's head layout (16 query heads on one kv head)
    (2, 8, 2, 96, 160, 48, False),       # G = 4, two kv heads, more keys than queries, no causal filter
    (1, 4, 4, 130, 130, 17, True),       # G = 1, list length 17: a second gather with a single entry
    (1, 2, 1, 64, 64, 1, True),          # one entry per token
    (1, 32, 2, 80, 300, 100, True),      # G = 16 with two kv heads, list length not a multiple of 16
    (1, 6, 2, 50, 50, 512, True),        # upstream's list length; G = 3; most of every list is padding
]


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,n,causal", CASES)
def test_parity_with_cpu_oracle(B, Hq, Hkv, Sq, Skv, n, causal):
    rng = np.random.default_rng(1000 + n + Sq)
    q = ol.randn_bf16((B, Hq, Sq, 128), 301)
    k = ol.randn_bf16((B, Hkv, Skv, 128), 302)
    v = ol.randn_bf16((B, Hkv, Skv, 128), 303)
    idx = _lists(rng, B, Hkv, Sq, Skv, n, causal)
    want_o, want_lse = ol.sgqa_prefill(q, k, v, idx, SCALE, causal)
    got_o, got_lse = _run(q, k, v, idx, causal)
    tag = "B%d Hq%d Hkv%d Sq%d Skv%d n%d causal%d" % (B, Hq, Hkv, Sq, Skv, n, causal)
    ol.assert_parity(got_o, want_o, tag)
    _check_lse(got_lse, want_lse, tag)
    assert_clean_status()


def test_full_causal_list_reproduces_the_dense_prefill_kernel():
    """With every visible token listed, the sparse kernel and the dense causal kernel compute the same attention."""
    import cuda_llm_ops_b200 as ops
    B, Hq, Hkv, S = 1, 8, 2, 256
    q = ol.randn_bf16((B, Hq, S, 128), 311)
    k = ol.randn_bf16((B, Hkv, S, 128), 312)
    v = ol.randn_bf16((B, Hkv, S, 128), 313)
    idx = np.broadcast_to(np.arange(S, dtype=np.int32), (B, Hkv, S, S)).copy()
    got_o, got_lse = _run(q, k, v, idx, True)
    dense_o, dense_lse = ops.launch_flash_gqa_forward_bf16_kernel(to_dev(q), to_dev(k), to_dev(v), causal=True)
    torch.cuda.synchronize()
    ol.assert_parity(got_o, to_bits(dense_o), "sparse vs dense")
    assert np.allclose(got_lse, dense_lse.cpu().numpy(), atol=2e-3)


def test_upstream_shape_family_sampled_rows():
    """Upstream's benchmark family (16 query heads on one kv head, lists of 512) at S = 4096, rows checked by sampling."""
    import cuda_llm_ops_b200 as ops
    Hq, S, n = 16, 4096, 512
    g = torch.Generator(device="cuda").manual_seed(91)
    q = torch.randn((1, Hq, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((1, 1, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((1, 1, S, 128), generator=g, device="cuda").to(torch.bfloat16)
    pos = torch.arange(S, device="cuda").view(1, 1, S, 1)
    idx = (torch.rand((1, 1, S, n), generator=g, device="cuda") * (pos + 1)).to(torch.int32)
    idx = torch.minimum(idx, pos.to(torch.int32))
    idx[..., :16] = torch.clamp(pos - torch.arange(16, device="cuda").view(1, 1, 1, 16), min=-1).to(torch.int32)
    out, lse = ops.launch_flash_sgqa_forward_bf16_kernel(q, k, v, idx.contiguous(), n, causal=True)
    torch.cuda.synchronize()
    rows = [0, 1, 15, 16, 17, 511, 512, 2047, 4095]
    qn, kn, vn = to_bits(q)[:, :, rows], to_bits(k), to_bits(v)
    idx_rows = idx.cpu().numpy()[:, :, rows]
    # the oracle takes the query position from the row number: give it the sampled rows one at a time
    for r, row in enumerate(rows):
        q_pad = np.zeros((1, Hq, row + 1, 128), dtype=np.uint16)
        q_pad[:, :, row] = qn[:, :, r]
        idx_pad = np.full((1, 1, row + 1, n), -1, dtype=np.int32)
        idx_pad[:, :, row] = idx_rows[:, :, r]
        want_o, want_lse = ol.sgqa_prefill(q_pad, kn, vn, idx_pad, SCALE, True)
        ol.assert_parity(to_bits(out)[:, :, row], want_o[:, :, row], "row %d" % row)
        assert np.allclose(lse.cpu().numpy()[:, :, row], want_lse[:, :, row], atol=2e-3)
    assert_clean_status()


def test_launcher_checks_like_upstream():
    import cuda_llm_ops_b200 as ops
    q = torch.zeros((1, 4, 8, 128), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((1, 2, 8, 128), dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros((1, 2, 8, 4), dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="int32"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k, k, idx.long(), 4)
    with pytest.raises(ValueError, match="num_sparse_kv must be >= 1"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k, k, idx, 0)
    with pytest.raises(ValueError, match="must have shape"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q, k, k, idx, 5)
    with pytest.raises(ValueError, match="bf16"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q.float(), k, k, idx, 4)
    with pytest.raises(ValueError, match="divisible"):
        ops.launch_flash_sgqa_forward_bf16_kernel(q[:, :3], k, k, idx, 4)
