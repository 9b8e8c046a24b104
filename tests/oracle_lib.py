"""Test-side binding of the CPU oracle (oracle/gqa_oracle.c) plus bf16 <-> numpy helpers.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "_build", "libgqa_oracle.so")
REF_BIN = os.path.join(ORACLE_DIR, "_ref", "ref_decode_cpu")
REF_ROPE_BIN = os.path.join(ORACLE_DIR, "_ref", "ref_rope_cpu")

MAX_ABS_TOL = 2e-2   # parity gate stated for this path: max-abs error of the bf16 output
MEAN_ABS_TOL = 2e-3  # and mean-abs error, both against the CPU reference on identical inputs

_lib = None
_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def build_oracle(with_ref=False):
    src = os.path.join(ORACLE_DIR, "gqa_oracle.c")
    if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", ORACLE_DIR, "all"], check=True, capture_output=True)
    if with_ref and not os.path.exists(REF_BIN):
        subprocess.run(["make", "-C", ORACLE_DIR, "_ref"], check=True, capture_output=True)
    return ORACLE_SO


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build_oracle())
        _lib.cllo_oracle_gqa_decode_bf16.restype = ctypes.c_int
        _lib.cllo_oracle_gqa_combine.restype = ctypes.c_int
        _lib.cllo_oracle_gqa_prefill_bf16.restype = ctypes.c_int
        _lib.cllo_oracle_num_threads.restype = ctypes.c_int
        _lib.cllo_oracle_swa_prefill_bf16.restype = ctypes.c_int
        _lib.cllo_oracle_gqa_backward_bf16.restype = ctypes.c_int
        _lib.cllo_oracle_swa_backward_bf16.restype = ctypes.c_int
        _lib.cllo_oracle_rope_bf16.restype = ctypes.c_int
    return _lib


def f32_to_bf16_bits(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def randn_bf16(shape, seed, std=1.0):
    rng = np.random.default_rng(seed)
    return f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


def _ptr(a, ct):
    return a.ctypes.data_as(ctypes.POINTER(ct)) if a is not None else None


def decode(q, k, v, scale, kv_layout, s_begin=0, s_end=None, tile=128, want_partial=False, par_heads=True):
    """q [B,Hq,D] uint16; k,v per layout (0: [B,S,Hkv,D], 1: [B,Hkv,S,D]).  Returns o bits (and O,m,l)."""
    q, k, v = (np.ascontiguousarray(a, dtype=np.uint16) for a in (q, k, v))
    B, Hq, D = q.shape
    if kv_layout == 0:
        _, S, Hkv, _ = k.shape
    else:
        _, Hkv, S, _ = k.shape
    if s_end is None:
        s_end = S
    o = np.zeros((B, Hq, D), dtype=np.uint16)
    ou = np.zeros((B, Hq, D), dtype=np.float32) if want_partial else None
    m = np.zeros((B, Hq), dtype=np.float32) if want_partial else None
    l = np.zeros((B, Hq), dtype=np.float32) if want_partial else None
    rc = lib().cllo_oracle_gqa_decode_bf16(
        _ptr(q, ctypes.c_uint16), _ptr(k, ctypes.c_uint16), _ptr(v, ctypes.c_uint16), ctypes.c_float(scale),
        _ptr(o, ctypes.c_uint16), _ptr(ou, ctypes.c_float), _ptr(m, ctypes.c_float), _ptr(l, ctypes.c_float),
        B, S, Hq, Hkv, D, kv_layout, s_begin, s_end, tile, 1 if par_heads else 0)
    assert rc == 0, rc
    if want_partial:
        return o, ou, m, l
    return o


def pack_partial(ou, m, l):
    """[B,Hq,D], [B,Hq], [B,Hq] -> [B,Hq,D+2] in the library's packed layout."""
    return np.concatenate([ou, m[..., None], l[..., None]], axis=-1).astype(np.float32)


def combine(partials):
    """partials [nsplit, rows..., D+2] fp32 -> (o bits [rows..., D], o fp32)."""
    partials = np.ascontiguousarray(partials, dtype=np.float32)
    nsplit = partials.shape[0]
    D = partials.shape[-1] - 2
    rows = int(np.prod(partials.shape[1:-1]))
    o = np.zeros(partials.shape[1:-1] + (D,), dtype=np.uint16)
    of = np.zeros(partials.shape[1:-1] + (D,), dtype=np.float32)
    rc = lib().cllo_oracle_gqa_combine(_ptr(partials, ctypes.c_float), nsplit, ctypes.c_int64(rows), D,
                                       _ptr(o, ctypes.c_uint16), _ptr(of, ctypes.c_float))
    assert rc == 0, rc
    return o, of


def prefill(q, k, v, scale, causal, row_begin=0, row_end=None):
    """q [B,Hq,Sq,D], k,v [B,Hkv,Skv,D] uint16 -> (o bits, lse fp32)."""
    q, k, v = (np.ascontiguousarray(a, dtype=np.uint16) for a in (q, k, v))
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    if row_end is None:
        row_end = Sq
    o = np.zeros((B, Hq, Sq, D), dtype=np.uint16)
    lse = np.zeros((B, Hq, Sq), dtype=np.float32)
    rc = lib().cllo_oracle_gqa_prefill_bf16(
        _ptr(q, ctypes.c_uint16), _ptr(k, ctypes.c_uint16), _ptr(v, ctypes.c_uint16), ctypes.c_float(scale),
        1 if causal else 0, _ptr(o, ctypes.c_uint16), _ptr(lse, ctypes.c_float),
        B, Sq, Skv, Hq, Hkv, D, row_begin, row_end)
    assert rc == 0, rc
    return o, lse


def swa_prefill(q, k, v, scale, window, sink):
    """Sliding-window + sink forward: q [B,Hq,Sq,D], k,v [B,Hkv,Skv,D] uint16, sink [Hq] fp32 -> (o bits, lse)."""
    q, k, v = (np.ascontiguousarray(a, dtype=np.uint16) for a in (q, k, v))
    sink = np.ascontiguousarray(sink, dtype=np.float32)
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    o = np.zeros((B, Hq, Sq, D), dtype=np.uint16)
    lse = np.zeros((B, Hq, Sq), dtype=np.float32)
    rc = lib().cllo_oracle_swa_prefill_bf16(
        _ptr(q, ctypes.c_uint16), _ptr(k, ctypes.c_uint16), _ptr(v, ctypes.c_uint16), ctypes.c_float(scale),
        int(window), _ptr(sink, ctypes.c_float), _ptr(o, ctypes.c_uint16), _ptr(lse, ctypes.c_float),
        B, Sq, Skv, Hq, Hkv, D)
    assert rc == 0, rc
    return o, lse


def mla_prefill(q, k, v, scale, causal=True):
    """MLA-shaped forward: q [B,Hq,Sq,Dqk], k [B,Hkv,Skv,Dqk], v [B,Hkv,Skv,Dv] uint16 -> (o [B,Hq,Sq,Dv] bits, lse)."""
    q, k, v = (np.ascontiguousarray(a, dtype=np.uint16) for a in (q, k, v))
    B, Hq, Sq, Dqk = q.shape
    _, Hkv, Skv, _ = k.shape
    Dv = v.shape[3]
    o = np.zeros((B, Hq, Sq, Dv), dtype=np.uint16)
    lse = np.zeros((B, Hq, Sq), dtype=np.float32)
    rc = lib().cllo_oracle_mla_prefill_bf16(
        _ptr(q, ctypes.c_uint16), _ptr(k, ctypes.c_uint16), _ptr(v, ctypes.c_uint16), ctypes.c_float(scale),
        1 if causal else 0, _ptr(o, ctypes.c_uint16), _ptr(lse, ctypes.c_float), B, Sq, Skv, Hq, Hkv, Dqk, Dv)
    assert rc == 0, rc
    return o, lse


def sgqa_prefill(q, k, v, sparse_idx, scale, causal=True):
    """Sparse-index GQA forward: q [B,Hq,Sq,D], k,v [B,Hkv,Skv,D] uint16, sparse_idx int32 [B,Hkv,Sq,n] -> (o, lse)."""
    q, k, v = (np.ascontiguousarray(a, dtype=np.uint16) for a in (q, k, v))
    sparse_idx = np.ascontiguousarray(sparse_idx, dtype=np.int32)
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    assert sparse_idx.shape[:3] == (B, Hkv, Sq), sparse_idx.shape
    o = np.zeros((B, Hq, Sq, D), dtype=np.uint16)
    lse = np.zeros((B, Hq, Sq), dtype=np.float32)
    rc = lib().cllo_oracle_sgqa_prefill_bf16(
        _ptr(q, ctypes.c_uint16), _ptr(k, ctypes.c_uint16), _ptr(v, ctypes.c_uint16), _ptr(sparse_idx, ctypes.c_int32),
        int(sparse_idx.shape[3]), ctypes.c_float(scale), 1 if causal else 0, _ptr(o, ctypes.c_uint16),
        _ptr(lse, ctypes.c_float), B, Sq, Skv, Hq, Hkv, D)
    assert rc == 0, rc
    return o, lse


def backward(q, k, v, o, grad_o, scale, causal):
    """q,o,grad_o [B,Hq,Sq,D], k,v [B,Hkv,Skv,D] uint16 -> (grad_q, grad_k, grad_v) bits."""
    q, k, v, o, grad_o = (np.ascontiguousarray(a, dtype=np.uint16) for a in (q, k, v, o, grad_o))
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    gq, gk, gv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    u16 = ctypes.c_uint16
    rc = lib().cllo_oracle_gqa_backward_bf16(_ptr(q, u16), _ptr(k, u16), _ptr(v, u16), _ptr(o, u16), _ptr(grad_o, u16),
                                             ctypes.c_float(scale), 1 if causal else 0, _ptr(gq, u16), _ptr(gk, u16),
                                             _ptr(gv, u16), B, Sq, Skv, Hq, Hkv, D)
    assert rc == 0, rc
    return gq, gk, gv


def swa_backward(q, k, v, o, grad_o, scale, window, sink):
    """Sliding-window + sink backward -> (grad_q, grad_k, grad_v) bits."""
    q, k, v, o, grad_o = (np.ascontiguousarray(a, dtype=np.uint16) for a in (q, k, v, o, grad_o))
    sink = np.ascontiguousarray(sink, dtype=np.float32)
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    gq, gk, gv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    u16 = ctypes.c_uint16
    rc = lib().cllo_oracle_swa_backward_bf16(_ptr(q, u16), _ptr(k, u16), _ptr(v, u16), _ptr(o, u16), _ptr(grad_o, u16),
                                             ctypes.c_float(scale), int(window), _ptr(sink, ctypes.c_float),
                                             _ptr(gq, u16), _ptr(gk, u16), _ptr(gv, u16), B, Sq, Skv, Hq, Hkv, D)
    assert rc == 0, rc
    return gq, gk, gv


def rope(x, base=10000.0):
    """x [B,S,hidden] uint16 -> rotated bits."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    B, S, hidden = x.shape
    out = np.zeros_like(x)
    rc = lib().cllo_oracle_rope_bf16(_ptr(x, ctypes.c_uint16), _ptr(out, ctypes.c_uint16), B, S, hidden, ctypes.c_float(base))
    assert rc == 0, rc
    return out


def assert_grad_parity(got_bits, want_bits, what=""):
    """Gradients have no fixed scale, so the gate is relative: relative L2 <= 2e-2 (upstream's own metric) and a
    max-abs error below 2e-2 of the largest reference magnitude."""
    mx, mean, rel = errors(got_bits, want_bits)
    ref_max = float(np.abs(bf16_bits_to_f32(want_bits)).max())
    assert np.isfinite(bf16_bits_to_f32(got_bits)).all(), what + ": non-finite gradient"
    assert rel <= 2e-2 and mx <= 2e-2 * max(ref_max, 1e-6), "%s: max-abs %.3e (ref max %.3e) rel-L2 %.3e" % (what, mx, ref_max, rel)
    return mx, mean, rel


def errors(got_bits, want_bits):
    """(max-abs, mean-abs, relative-L2) between two bf16 bit arrays."""
    g = bf16_bits_to_f32(got_bits).astype(np.float64)
    w = bf16_bits_to_f32(want_bits).astype(np.float64)
    d = np.abs(g - w)
    rel = float(np.sqrt((d * d).sum()) / max(np.sqrt((w * w).sum()), 1e-30))
    return float(d.max()), float(d.mean()), rel


def assert_parity(got_bits, want_bits, what=""):
    mx, mean, rel = errors(got_bits, want_bits)
    assert np.isfinite(bf16_bits_to_f32(got_bits)).all(), what + ": non-finite output"
    assert mx <= MAX_ABS_TOL and mean <= MEAN_ABS_TOL, "%s: max-abs %.3e mean-abs %.3e rel-L2 %.3e" % (what, mx, mean, rel)
    # the stated gate is loose next to the output scale; relative L2 (upstream's own metric) catches real bugs
    assert rel <= 2e-2, "%s: relative L2 %.3e" % (what, rel)
    return mx, mean, rel
