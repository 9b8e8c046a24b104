#!/usr/bin/env python
"""Python bench script for the GQA path, in the style of upstream's examples/python/Triton/test_decode_flash_gqa_kernel.py
and test_flash_gqa_kernel.py: seeded inputs at upstream's benchmark shapes, a plain torch fp32 reference, the
launcher timed with CUDA events after warm-up, and one line per operator with time, rate (decimal units) and the
relative L2 error against the reference.  Inputs are N(0,1) rather than upstream's U(0,1): with all-positive inputs
the softmax is nearly uniform and grad_q is a difference of nearly equal terms, whose relative error says little.

    python examples/python/bench_flash_gqa.py [--iters 50]

The launchers are the drop-in mirrors of upstream's (same names, arguments and tensor layouts).
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import cuda_llm_ops_b200 as ops  # noqa: E402


def reference_attention(q, k, v, causal):
    """softmax(q k^T / sqrt(D)) v in fp32, heads of a group sharing their kv head.  q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D]."""
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().view(B, Hkv, g, Sq, D)
    s = torch.einsum("bhgqd,bhkd->bhgqk", qf, k.float()) / math.sqrt(D)
    if causal:
        mask = torch.ones(Sq, Skv, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhgqk,bhkd->bhgqd", p, v.float()).reshape(B, Hq, Sq, D)


def rel_l2(got, want):
    got, want = got.float(), want.float()
    return float((got - want).norm() / want.norm())


def time_us(fn, iters):
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=50)
    args = ap.parse_args()
    torch.manual_seed(0)
    dev = torch.device("cuda")

    # decode, upstream's shape (test_decode_flash_gqa_kernel.py: B=60, Hq=128, Hkv=8, S=4096, D=128, [B,H,S,D])
    B, Hq, Hkv, S, D = 60, 128, 8, 4096, 128
    q = torch.randn((B, Hq, 1, D), device=dev).to(torch.bfloat16)
    k = torch.randn((B, Hkv, S, D), device=dev).to(torch.bfloat16)
    v = torch.randn((B, Hkv, S, D), device=dev).to(torch.bfloat16)
    out = ops.launch_decode_flash_gqa_bf16_kernel(q, k, v)
    want = torch.cat([reference_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], False) for b in range(B)])
    us = time_us(lambda: ops.launch_decode_flash_gqa_bf16_kernel(q, k, v, out=out), args.iters)
    nbytes = 2 * k.numel() * 2 + 2 * q.numel() * 2
    print("decode_flash_gqa   B=%d Hq=%d Hkv=%d S=%d: %8.1f us  %6.3f TB/s  rel. L2 error %.2e"
          % (B, Hq, Hkv, S, us, nbytes / us / 1e6, rel_l2(out, want)))
    del k, v, want

    # prefill forward and backward, upstream's shape (test_flash_gqa_kernel.py: S=4096, Hq=16, Hkv=1, causal, un-batched)
    Hq, Hkv, S = 16, 1, 4096
    q = torch.randn((Hq, S, D), device=dev).to(torch.bfloat16)
    k = torch.randn((Hkv, S, D), device=dev).to(torch.bfloat16)
    v = torch.randn((Hkv, S, D), device=dev).to(torch.bfloat16)
    o, lse = ops.launch_flash_gqa_forward_bf16_kernel(q, k, v)
    want = reference_attention(q[None], k[None], v[None], True)[0]
    us = time_us(lambda: ops.launch_flash_gqa_forward_bf16_kernel(q, k, v, out=o, lse=lse), args.iters)
    flops = 4.0 * Hq * S * S * D / 2
    print("flash_gqa_forward  Hq=%d Hkv=%d S=%d causal: %8.1f us  %6.1f TFLOP/s  rel. L2 error %.2e"
          % (Hq, Hkv, S, us, flops / us / 1e6, rel_l2(o, want)))

    grad_o = torch.randn((Hq, S, D), device=dev).to(torch.bfloat16)
    qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
    reference_attention(qr[None], kr[None], vr[None], True)[0].backward(grad_o.float())
    dq, dk, dv = ops.launch_flash_gqa_backward_bf16_kernel(q, k, v, o, lse, grad_o)
    us = time_us(lambda: ops.launch_flash_gqa_backward_bf16_kernel(q, k, v, o, lse, grad_o), args.iters)
    flops = 2.0 * Hq * S * S * (3 * D + 2 * D) / 2  # upstream's count: five products, halved for causality
    print("flash_gqa_backward Hq=%d Hkv=%d S=%d causal: %8.1f us  %6.1f TFLOP/s  rel. L2 error dq %.2e dk %.2e dv %.2e"
          % (Hq, Hkv, S, us, flops / us / 1e6, rel_l2(dq, qr.grad), rel_l2(dk, kr.grad), rel_l2(dv, vr.grad)))
    rc, detail = ops.device_status()
    print("device status:", rc, detail)
    return 0 if rc == 0 else 2


if __name__ == "__main__":
    sys.exit(main())
