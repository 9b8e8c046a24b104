"""The decode step with rotary embedding and cache append folded in, against the composition of the two oracles
(upstream's RoPE reference on the new token's Q and K, then upstream's decode reference over the appended cache)."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import assert_clean_status, to_bits, to_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def _rope_at(vecs, pos, base=10000.0):
    """Rotate bf16 vectors [..., 128] as token `pos` of a sequence (the oracle rotates row s of [B,S,hidden] by s)."""
    flat = vecs.reshape(-1, 128)
    out = np.zeros_like(flat)
    for i in range(flat.shape[0]):
        x = np.zeros((1, pos + 1, 128), dtype=np.uint16)
        x[0, pos] = flat[i]
        out[i] = ol.rope(x, base)[0, pos]
    return out.reshape(vecs.shape)


# (B, S, S_capacity, Hq, Hkv, layout, per-sequence positions?)
CASES = [
    (2, 300, 300, 16, 2, 0, False),      # the new token fills the cache exactly
    (3, 1000, 1024, 32, 4, 1, False),    # capacity beyond the sequence, [B,Hkv,S,D]
    (1, 65, 4096, 8, 8, 0, True),        # the new token starts a tile; positions given
    (2, 2049, 2304, 40, 2, 1, True),     # group 20: two 16-row blocks patch the same key row
    (4, 1, 16, 4, 1, 0, False),          # first token of a sequence
    (1, 5000, 5000, 64, 8, 0, False),    # every unit cut between workers
]


@pytest.mark.parametrize("B,S,S_cap,Hq,Hkv,layout,with_pos", CASES)
def test_step_matches_rope_then_decode(B, S, S_cap, Hq, Hkv, layout, with_pos):
    import cuda_llm_ops_b200 as ops
    q = ol.randn_bf16((B, Hq, 128), 701)
    k_new, v_new = ol.randn_bf16((B, Hkv, 128), 702), ol.randn_bf16((B, Hkv, 128), 703)
    shape = (B, S_cap, Hkv, 128) if layout == 0 else (B, Hkv, S_cap, 128)
    k_cache, v_cache = ol.randn_bf16(shape, 704), ol.randn_bf16(shape, 705)
    pos = [S - 1 + 7 * b for b in range(B)] if with_pos else [S - 1] * B
    # expected: rotate, append, attend over the first S positions
    q_rot = np.stack([_rope_at(q[b], pos[b]) for b in range(B)])
    k_rot = np.stack([_rope_at(k_new[b], pos[b]) for b in range(B)])
    k_want, v_want = k_cache.copy(), v_cache.copy()
    if layout == 0:
        k_want[:, S - 1], v_want[:, S - 1] = k_rot, v_new
        want = ol.decode(q_rot, k_want[:, :S], v_want[:, :S], SCALE, 0)
    else:
        k_want[:, :, S - 1], v_want[:, :, S - 1] = k_rot, v_new
        want = ol.decode(q_rot, k_want[:, :, :S], v_want[:, :, :S], SCALE, 1)
    kd, vd = to_dev(k_cache), to_dev(v_cache)
    positions = torch.tensor(pos, dtype=torch.int32, device="cuda") if with_pos else None
    out = ops.gqa_decode_rope_append(to_dev(q), to_dev(k_new), to_dev(v_new), kd, vd, S, positions=positions,
                                     scale=SCALE, kv_layout=layout)
    torch.cuda.synchronize()
    ol.assert_parity(to_bits(out), want, "rope+append+decode")
    # the caches: the new row appended (rotated key within one bf16 ulp of the oracle's), nothing else touched
    got_k, got_v = to_bits(kd), to_bits(vd)
    assert np.array_equal(got_v, v_want)
    diff = got_k != k_want
    row = (slice(None), S - 1) if layout == 0 else (slice(None), slice(None), S - 1)
    mask = np.zeros_like(diff)
    mask[row] = True
    assert not (diff & ~mask).any(), "a cache row other than the appended one changed"
    mx, _, rel = ol.errors(got_k[row], k_want[row])
    assert rel <= 4e-3, (mx, rel)
    # a plain decode over the updated cache with the rotated query gives the same output
    plain = ops.gqa_decode(to_dev(q_rot), kd[:, :S].contiguous() if layout == 0 else kd[:, :, :S].contiguous(),
                           vd[:, :S].contiguous() if layout == 0 else vd[:, :, :S].contiguous(), scale=SCALE,
                           kv_layout=layout)
    torch.cuda.synchronize()
    mx, _, rel = ol.errors(to_bits(out), to_bits(plain))
    assert mx <= 4e-3 and rel <= 5e-3, (mx, rel)
    assert_clean_status()


def test_argument_checks():
    import cuda_llm_ops_b200 as ops
    q = torch.zeros((1, 8, 128), dtype=torch.bfloat16, device="cuda")
    kn = torch.zeros((1, 2, 128), dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros((1, 64, 2, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="seq_len"):
        ops.gqa_decode_rope_append(q, kn, kn, cache, cache.clone(), 65, kv_layout=0)
    with pytest.raises(ValueError, match="k_new"):
        ops.gqa_decode_rope_append(q, kn[:, :1], kn, cache, cache.clone(), 10, kv_layout=0)
    with pytest.raises(ValueError, match="positions"):
        ops.gqa_decode_rope_append(q, kn, kn, cache, cache.clone(), 10, kv_layout=0,
                                   positions=torch.zeros(1, dtype=torch.int64, device="cuda"))
