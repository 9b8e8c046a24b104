"""Generate the golden vectors in this directory from the UPSTREAM torch oracles.

Run once, in a container that has the upstream checkout (it is not needed to run the tests):

    python tests/golden/make_golden.py --reference <path of the upstream checkout>

It imports, unmodified,
  * ``flash_gqa_reference``          examples/python/Triton/test_decode_flash_gqa_kernel.py:26-79
    (tiled, non-causal, any number of query rows), and
  * ``flash_gqa_forward_reference``  examples/python/Triton/test_flash_gqa_kernel.py:27-94
    (full softmax, causal, returns the log-sum-exp),
  * ``flash_swa_forward_reference``  examples/python/Triton/test_flash_swa_kernel.py:28-118
    (sliding window + sink term),
  * ``flash_sgqa_forward_reference`` examples/python/Triton/test_flash_sgqa_kernel.py:102-216
    (sparse-index GQA; the list length is a module constant there, 512, which the script sets to the small
    length of its cases before calling the function),
  * ``flash_mla_forward_reference``  examples/python/Triton/test_flash_mla_kernel.py:27-94
    (head_dim_qk = 192, head_dim_v = 128, causal),
feeds them small seeded N(0,1) bf16 tensors and stores inputs and outputs (bf16 as uint16 bit
patterns) in ``gqa_golden.npz``.  The tests compare both the C oracle and the CUDA kernels with
these files, so the oracle is pinned to upstream's own code rather than to itself.
"""
import argparse
import os
import sys

import numpy as np
import torch


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the upstream checkout")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "examples", "python", "Triton"))
    from test_decode_flash_gqa_kernel import flash_gqa_reference  # noqa: E402
    from test_flash_gqa_kernel import flash_gqa_forward_reference  # noqa: E402

    out = {}
    meta = []

    # --- decode (one query row) and non-causal multi-row cases: layout [B,H,S,D] -------------
    decode_cases = [
        # name,            B, Hq, Hkv, Sq, Skv, std
        ("decode_g4",      2, 8, 2, 1, 192, 1.0),
        ("decode_g16_rag", 1, 16, 1, 1, 200, 1.0),   # ragged last tile (200 = 128 + 72)
        ("decode_g8_tiny", 1, 8, 1, 1, 77, 1.0),     # shorter than one tile
        ("decode_g1",      1, 2, 2, 1, 130, 0.5),
        ("noncausal_g2",   1, 4, 2, 48, 160, 1.0),   # pins the non-causal prefill path
    ]
    for i, (name, B, Hq, Hkv, Sq, Skv, std) in enumerate(decode_cases):
        g = torch.Generator().manual_seed(1000 + i)
        q = (torch.randn(B, Hq, Sq, 128, generator=g) * std).to(torch.bfloat16)
        k = (torch.randn(B, Hkv, Skv, 128, generator=g) * std).to(torch.bfloat16)
        v = (torch.randn(B, Hkv, Skv, 128, generator=g) * std).to(torch.bfloat16)
        o = flash_gqa_reference(q, k, v)
        out[name + "/q"], out[name + "/k"], out[name + "/v"], out[name + "/o"] = map(_bits, (q, k, v, o))
        meta.append(name)

    # --- causal prefill with log-sum-exp: upstream takes un-batched [H,S,D] -------------------
    prefill_cases = [
        ("causal_g4", 4, 1, 160),
        ("causal_g1", 2, 2, 96),
    ]
    for i, (name, Hq, Hkv, S) in enumerate(prefill_cases):
        g = torch.Generator().manual_seed(2000 + i)
        q = torch.randn(Hq, S, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(Hkv, S, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(Hkv, S, 128, generator=g).to(torch.bfloat16)
        o, lse = flash_gqa_forward_reference(q, k, v, return_lse=True)
        out[name + "/q"], out[name + "/k"], out[name + "/v"], out[name + "/o"] = map(_bits, (q, k, v, o))
        out[name + "/lse"] = lse.numpy().astype(np.float32)
        meta.append(name)

    # --- sliding window + sink (upstream un-batched [H,S,D]; reference of test_flash_swa_kernel.py:28-118) ---
    from test_flash_swa_kernel import flash_swa_forward_reference  # noqa: E402
    swa_cases = [
        ("swa_g4_w48", 4, 1, 160, 48),
        ("swa_g2_w130", 2, 1, 260, 130),
    ]
    for i, (name, Hq, Hkv, S, window) in enumerate(swa_cases):
        g = torch.Generator().manual_seed(3000 + i)
        q = torch.randn(Hq, S, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(Hkv, S, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(Hkv, S, 128, generator=g).to(torch.bfloat16)
        sink = torch.rand(Hq, generator=g) * 2.0 + 0.1
        o, lse = flash_swa_forward_reference(q, k, v, return_lse=True, window_size=window, sink_value=sink)
        out[name + "/q"], out[name + "/k"], out[name + "/v"], out[name + "/o"] = map(_bits, (q, k, v, o))
        out[name + "/lse"] = lse.numpy().astype(np.float32)
        out[name + "/sink"] = sink.numpy().astype(np.float32)
        out[name + "/window"] = np.array(window)
        meta.append(name)

    # --- backward (upstream flash_gqa_backward_reference, test_flash_gqa_kernel.py:97-173; causal, un-batched) ---
    from test_flash_gqa_kernel import flash_gqa_backward_reference  # noqa: E402
    for i, (name, Hq, Hkv, S) in enumerate([("bwd_g2", 2, 1, 144)]):
        g = torch.Generator().manual_seed(4000 + i)
        q = torch.randn(Hq, S, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(Hkv, S, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(Hkv, S, 128, generator=g).to(torch.bfloat16)
        grad_o = torch.randn(Hq, S, 128, generator=g).to(torch.bfloat16)
        o, lse = flash_gqa_forward_reference(q, k, v, return_lse=True)
        dq, dk, dv = flash_gqa_backward_reference(q, k, v, o, grad_o)
        for key, t in (("q", q), ("k", k), ("v", v), ("o", o), ("grad_o", grad_o), ("dq", dq), ("dk", dk), ("dv", dv)):
            out[name + "/" + key] = _bits(t)
        out[name + "/lse"] = lse.numpy().astype(np.float32)
        meta.append(name)

    # --- sliding-window backward (upstream flash_swa_backward_reference, test_flash_swa_kernel.py:121-220) ---
    from test_flash_swa_kernel import flash_swa_backward_reference  # noqa: E402
    for i, (name, Hq, Hkv, S, window) in enumerate([("swa_bwd_g2_w100", 2, 1, 176, 100)]):
        g = torch.Generator().manual_seed(5000 + i)
        q = torch.randn(Hq, S, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(Hkv, S, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(Hkv, S, 128, generator=g).to(torch.bfloat16)
        grad_o = torch.randn(Hq, S, 128, generator=g).to(torch.bfloat16)
        sink = torch.rand(Hq, generator=g) * 2.0 + 0.1
        o, lse = flash_swa_forward_reference(q, k, v, return_lse=True, window_size=window, sink_value=sink)
        dq, dk, dv = flash_swa_backward_reference(q, k, v, o, grad_o, window_size=window, sink_value=sink)
        for key, t in (("q", q), ("k", k), ("v", v), ("o", o), ("grad_o", grad_o), ("dq", dq), ("dk", dk), ("dv", dv)):
            out[name + "/" + key] = _bits(t)
        out[name + "/lse"] = lse.numpy().astype(np.float32)
        out[name + "/sink"] = sink.numpy().astype(np.float32)
        out[name + "/window"] = np.array(window)
        meta.append(name)

    # --- sparse-index GQA forward (upstream flash_sgqa_forward_reference, test_flash_sgqa_kernel.py:102-216) ---
    import test_flash_sgqa_kernel as sg  # noqa: E402
    sgqa_cases = [
        # name,          Hq, Hkv, Sq, Skv, n_sparse, causal
        ("sgqa_g4_n40",   4,  1,  96,  96,  40, True),    # list length not a multiple of 16; early rows are padded with -1
        ("sgqa_g2_n16",   4,  2,  48,  80,  16, False),   # two kv heads with lists of their own; entries above q allowed
    ]
    for i, (name, Hq, Hkv, Sq, Skv, n_sparse, causal) in enumerate(sgqa_cases):
        g = torch.Generator().manual_seed(6000 + i)
        q = torch.randn(Hq, Sq, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(Hkv, Skv, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(Hkv, Skv, 128, generator=g).to(torch.bfloat16)
        idx = torch.full((1, Hkv, Sq, n_sparse), -1, dtype=torch.int32)
        for h in range(Hkv):
            for qi in range(Sq):
                hi = min(qi, Skv - 1) if causal else Skv - 1
                take = min(n_sparse, hi + 1)
                perm = torch.randperm(hi + 1, generator=g)[:take].to(torch.int32)
                idx[0, h, qi, :take] = perm
        # a few hostile entries: out of range, above the query position, repeated, and one empty list
        idx[0, 0, 5, 0] = Skv + 7
        idx[0, 0, 6, 1] = idx[0, 0, 6, 0]
        idx[0, 0, 7, :] = -1
        if causal:
            idx[0, 0, 9, 2] = 50
        sg.NUM_SPARSE_KV = n_sparse
        o, lse = sg.flash_sgqa_forward_reference(q, k, v, idx, return_lse=True, causal=causal)
        out[name + "/q"], out[name + "/k"], out[name + "/v"], out[name + "/o"] = map(_bits, (q, k, v, o))
        out[name + "/lse"] = lse.numpy().astype(np.float32)
        out[name + "/idx"] = idx.numpy().astype(np.int32)
        out[name + "/causal"] = np.array(1 if causal else 0)
        meta.append(name)

    # --- MLA-shaped forward (upstream flash_mla_forward_reference, test_flash_mla_kernel.py:27-94; causal) ---
    from test_flash_mla_kernel import flash_mla_forward_reference  # noqa: E402
    for i, (name, Hq, Hkv, S) in enumerate([("mla_g1", 2, 2, 200), ("mla_g2", 4, 2, 130)]):
        g = torch.Generator().manual_seed(7000 + i)
        q = torch.randn(Hq, S, 192, generator=g).to(torch.bfloat16)
        k = torch.randn(Hkv, S, 192, generator=g).to(torch.bfloat16)
        v = torch.randn(Hkv, S, 128, generator=g).to(torch.bfloat16)
        o, lse = flash_mla_forward_reference(q, k, v, return_lse=True)
        out[name + "/q"], out[name + "/k"], out[name + "/v"], out[name + "/o"] = map(_bits, (q, k, v, o))
        out[name + "/lse"] = lse.numpy().astype(np.float32)
        meta.append(name)

    out["cases"] = np.array(meta)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gqa_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", "torch", torch.__version__)


if __name__ == "__main__":
    main()
