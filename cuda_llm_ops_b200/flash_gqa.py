"""Host-side mirror of upstream's GQA operator interface, on top of the C ABI.

Upstream (LiuYiyang-Canton/cuda_llm_ops) exposes this path three ways; each has a same-named function here
with the same argument meaning and error behaviour:

* ``LaunchFlashGqaBf16Kernel``                 C++ launcher, include/cplusplus/FlashGQA/decode_flash_gqa_kernel.cuh:28-38
  (Q [B,Hq,D], K/V [B,S,Hkv,D], O [B,Hq,D]; silently does nothing on shapes it cannot handle,
  src/cplusplus/FlashGQA/decode_flash_gqa_kernel.cu:416-437)
* ``launch_decode_flash_gqa_bf16_kernel``      Triton launcher, src/python/Triton/decode_flash_gqa_kernel.py:137-196
  (Q [B,Hq,Sq,D], K/V [B,Hkv,S,D]; raises ValueError on bad inputs; only query row 0 is used)
* ``launch_flash_gqa_forward_bf16_kernel``     Triton launcher, src/python/Triton/flash_gqa_kernel.py:185-338
  (3-D or 4-D tensors, causal=True default, returns (out, lse))

torch is used for device memory and streams only.  Nothing here computes attention on the host and there
is no fallback: without the compiled library or on a non-CUDA tensor these functions raise.
"""
import math
import threading

import torch

from . import _lib

KV_BSHD = _lib.KV_BSHD
KV_BHSD = _lib.KV_BHSD
HEAD_DIM = 128
PARTIAL_WIDTH = HEAD_DIM + 2

_workspaces = {}
_workspaces_lock = threading.Lock()


def _stream_ptr():
    return torch.cuda.current_stream().cuda_stream


_ws_bytes_cache = {}


def decode_workspace_bytes(B, S, Hq, Hkv, D=HEAD_DIM, num_workers=0):
    # asked on every decode call: remembered per shape (and device, whose SM count enters the library's choice)
    key = (B, S, Hq, Hkv, D, num_workers, torch.cuda.current_device() if torch.cuda.is_available() else -1)
    n = _ws_bytes_cache.get(key)
    if n is None:
        n = int(_lib.load().cllo_gqa_decode_workspace_bytes(B, S, Hq, Hkv, D, num_workers))
        if len(_ws_bytes_cache) > 4096:
            _ws_bytes_cache.clear()
        _ws_bytes_cache[key] = n
    return n


def _workspace(device, nbytes, kind="decode"):
    """A per-device scratch tensor per kind of use, grown on demand (torch owns the memory).  The decode scratch is
    kept apart from any other: its first 4 KB are arrival counters that the decode calls vouch for.

    It is shared by every call on that device that does not bring its own ``workspace``: calls issued on different
    streams that may overlap on the GPU must each pass their own.
    """
    key = (kind, device.type, device.index if device.index is not None else torch.cuda.current_device())
    with _workspaces_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            # zeroed once: the decode kernel leaves its arrival counters zero, so calls on this tensor may vouch
            # for them (WS_COUNTERS_ZERO) and skip the memset in front of every kernel
            ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            _workspaces[key] = ws
    return ws


def _require_cuda_bf16(name, t):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor: this library has no CPU path" % name)
    if t.dtype != torch.bfloat16:
        raise ValueError("%s must be bf16" % name)


def _decode_shapes(q, k, v, kv_layout):
    for name, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(name, t)
    if q.dim() != 3 or k.dim() != 4 or v.shape != k.shape:
        raise ValueError("expected q [B,Hq,D] and k, v of identical 4-D shape")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise ValueError("q, k and v must be contiguous")
    B, Hq, D = q.shape
    if kv_layout == KV_BSHD:
        Bk, S, Hkv, Dk = k.shape
    elif kv_layout == KV_BHSD:
        Bk, Hkv, S, Dk = k.shape
    else:
        raise ValueError("unknown kv_layout")
    if Bk != B or Dk != D:
        raise ValueError("q, k and v must share batch and head_dim")
    if Hq % Hkv != 0:
        raise ValueError("Query heads must be divisible by KV heads")
    return B, S, Hq, Hkv, D


def gqa_decode(q, k, v, scale=None, kv_layout=KV_BHSD, out=None, partial_out=None, num_workers=0, workspace=None):
    """Split-KV decode through ``cllo_gqa_decode_bf16``.

    q [B,Hq,D]; k, v [B,S,Hkv,D] (KV_BSHD) or [B,Hkv,S,D] (KV_BHSD); returns out [B,Hq,D] bf16, or, when
    ``partial_out`` ([B,Hq,D+2] fp32) is given, fills and returns that packed (O, m, l) tensor instead.
    """
    B, S, Hq, Hkv, D = _decode_shapes(q, k, v, kv_layout)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        nbytes = decode_workspace_bytes(B, S, Hq, Hkv, D, num_workers)
        if workspace is None:
            workspace = _workspace(q.device, nbytes)
            kv_layout |= _lib.WS_COUNTERS_ZERO
        if partial_out is not None:
            if partial_out.dtype != torch.float32 or tuple(partial_out.shape) != (B, Hq, D + 2) \
                    or not partial_out.is_contiguous() or not partial_out.is_cuda:
                raise ValueError("partial_out must be a contiguous CUDA fp32 tensor of shape [B,Hq,D+2]")
            o_ptr, p_ptr, result = None, partial_out.data_ptr(), partial_out
        else:
            if out is None:
                out = torch.empty_like(q)
            if out.dtype != torch.bfloat16 or out.shape != q.shape or not out.is_contiguous():
                raise ValueError("Output tensor must be contiguous bf16 of q's shape")
            o_ptr, p_ptr, result = out.data_ptr(), None, out
        rc = lib.cllo_gqa_decode_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), float(scale), o_ptr,
                                      workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                                      B, S, Hq, Hkv, D, kv_layout, num_workers, p_ptr, _stream_ptr())
    _lib.check(rc, "cllo_gqa_decode_bf16")
    return result


def gqa_decode_sharded(q, k_local, v_local, peer_gather, peer_flags, rank, world, epoch=0, scale=None,
                       kv_layout=KV_BHSD, out=None, num_workers=0, workspace=None):
    """One step of a KV-position-sharded decode in one kernel (``cllo_gqa_decode_sharded_bf16``).

    ``k_local`` / ``v_local`` hold this rank's positions; ``peer_gather`` / ``peer_flags`` are ctypes arrays of
    ``world`` device pointers (every rank's exchange buffers as mapped here).  Returns the full out [B,Hq,D] bf16,
    identical on every rank.  Every rank must call once per step.
    """
    B, S, Hq, Hkv, D = _decode_shapes(q, k_local, v_local, kv_layout)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty_like(q)
    if out.dtype != torch.bfloat16 or out.shape != q.shape or not out.is_contiguous():
        raise ValueError("Output tensor must be contiguous bf16 of q's shape")
    with torch.cuda.device(q.device):
        nbytes = decode_workspace_bytes(B, S, Hq, Hkv, D, num_workers)
        if workspace is None:
            workspace = _workspace(q.device, nbytes)
            kv_layout |= _lib.WS_COUNTERS_ZERO
        rc = _lib.load().cllo_gqa_decode_sharded_bf16(
            q.data_ptr(), k_local.data_ptr(), v_local.data_ptr(), float(scale), out.data_ptr(),
            workspace.data_ptr(), workspace.numel() * workspace.element_size(), B, S, Hq, Hkv, D, kv_layout,
            num_workers, peer_gather, peer_flags, rank, world, epoch, _stream_ptr())
    _lib.check(rc, "cllo_gqa_decode_sharded_bf16")
    return out


def gqa_decode_rope_append(q, k_new, v_new, k_cache, v_cache, seq_len, positions=None, rope_base=10000.0, scale=None,
                           kv_layout=KV_BHSD, out=None, num_workers=0, workspace=None):
    """One decode step with rotary embedding and cache append inside the attention kernel
    (``cllo_gqa_decode_rope_append_bf16``).

    q [B,Hq,D], k_new / v_new [B,Hkv,D]: the new token, un-rotated.  k_cache / v_cache: [B,S_cap,Hkv,D] (KV_BSHD) or
    [B,Hkv,S_cap,D] (KV_BHSD) holding ``seq_len - 1`` earlier tokens; the call writes the rotated new key and the new
    value at position ``seq_len - 1`` (in place) and returns the attention output over ``seq_len`` positions.
    ``positions`` (int32 [B], optional) gives the rotary position per sequence; default ``seq_len - 1``.
    """
    B, S_cap, Hq, Hkv, D = _decode_shapes(q, k_cache, v_cache, kv_layout)
    for name, t in (("k_new", k_new), ("v_new", v_new)):
        _require_cuda_bf16(name, t)
        if tuple(t.shape) != (B, Hkv, D) or not t.is_contiguous():
            raise ValueError("%s must be contiguous [B,Hkv,D]" % name)
    if not 1 <= seq_len <= S_cap:
        raise ValueError("seq_len must lie in [1, cache capacity]")
    if positions is not None:
        if positions.dtype != torch.int32 or tuple(positions.shape) != (B,) or not positions.is_cuda \
                or not positions.is_contiguous():
            raise ValueError("positions must be a contiguous CUDA int32 tensor [B]")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty_like(q)
    if out.dtype != torch.bfloat16 or out.shape != q.shape or not out.is_contiguous():
        raise ValueError("Output tensor must be contiguous bf16 of q's shape")
    with torch.cuda.device(q.device):
        nbytes = decode_workspace_bytes(B, seq_len, Hq, Hkv, D, num_workers)
        if workspace is None:
            workspace = _workspace(q.device, nbytes)
            kv_layout |= _lib.WS_COUNTERS_ZERO
        rc = _lib.load().cllo_gqa_decode_rope_append_bf16(
            q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            positions.data_ptr() if positions is not None else None, float(rope_base), float(scale), out.data_ptr(),
            workspace.data_ptr(), workspace.numel() * workspace.element_size(), B, seq_len, S_cap, Hq, Hkv, D,
            kv_layout, num_workers, _stream_ptr())
    _lib.check(rc, "cllo_gqa_decode_rope_append_bf16")
    return out


def set_exchange_wait_limit(sm_cycles):
    """Upper bound, in SM clock cycles, of one wait for a peer in the sharded decode (<= 0: the default, ~1 s)."""
    _lib.check(_lib.load().cllo_set_exchange_wait_limit(int(sm_cycles)), "cllo_set_exchange_wait_limit")


def gqa_combine(partials, out=None):
    """LSE merge through ``cllo_gqa_combine_bf16``: partials [nsplit,B,Hq,D+2] fp32 -> out [B,Hq,D] bf16."""
    if not partials.is_cuda or partials.dtype != torch.float32 or partials.dim() != 4 \
            or partials.shape[-1] != PARTIAL_WIDTH or not partials.is_contiguous():
        raise ValueError("partials must be a contiguous CUDA fp32 tensor [nsplit,B,Hq,%d]" % PARTIAL_WIDTH)
    nsplit, B, Hq, _ = partials.shape
    if out is None:
        out = torch.empty((B, Hq, HEAD_DIM), dtype=torch.bfloat16, device=partials.device)
    with torch.cuda.device(partials.device):
        rc = _lib.load().cllo_gqa_combine_bf16(partials.data_ptr(), nsplit, out.data_ptr(), B * Hq, HEAD_DIM,
                                               _stream_ptr())
    _lib.check(rc, "cllo_gqa_combine_bf16")
    return out


def LaunchFlashGqaBf16Kernel(q, k, v, scale, o, oIntermediate, batchSize, seqLength, numQueryHeads, numKvHeads,
                             headDim):
    """Mirror of upstream's C++ launcher (decode_flash_gqa_kernel.cuh:28-38), tensors instead of pointers.

    Like upstream it returns None and does nothing on shapes it rejects
    (decode_flash_gqa_kernel.cu:416-437) -- but it rejects far fewer: any group size and any S >= 1 work;
    only headDim != 128 or non-divisible head counts are refused.  ``oIntermediate`` ([B,Hq,D] fp32) is used
    as scratch when it is big enough, exactly as upstream uses it.
    """
    if batchSize <= 0 or seqLength <= 0 or numQueryHeads <= 0 or numKvHeads <= 0 or headDim <= 0:
        return
    if numQueryHeads % numKvHeads != 0 or headDim != HEAD_DIM:
        return
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o)):
        _require_cuda_bf16(name, t)
    with torch.cuda.device(q.device):
        ws = None
        need = decode_workspace_bytes(batchSize, seqLength, numQueryHeads, numKvHeads, headDim)
        if oIntermediate is not None and oIntermediate.is_cuda and \
                oIntermediate.numel() * oIntermediate.element_size() >= need and oIntermediate.data_ptr() % 256 == 0:
            ws = oIntermediate.view(torch.uint8).view(-1) if oIntermediate.is_contiguous() else None
        if ws is None:
            ws = _workspace(q.device, need)
        rc = _lib.load().cllo_gqa_decode_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), float(scale), o.data_ptr(),
                                              ws.data_ptr(), ws.numel(), batchSize, seqLength, numQueryHeads,
                                              numKvHeads, headDim, KV_BSHD, 0, None, _stream_ptr())
    _lib.check(rc, "cllo_gqa_decode_bf16")


def launch_decode_flash_gqa_bf16_kernel(q, k, v, out=None):
    """Mirror of upstream's Triton decode launcher (decode_flash_gqa_kernel.py:137-196).

    q [B,Hq,Sq,D], k, v [B,Hkv,S,D] -> out [B,Hq,Sq,D]; scale is fixed at 1/sqrt(D) (:180).  As upstream,
    only query row 0 of each head is read and written (:76,111).
    """
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("Flash GQA decoding expects bf16 inputs")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise ValueError("Flash GQA decoding kernel expects contiguous Q/K/V tensors")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("Q, K, and V must be 4-D")
    batch, q_heads, seqlen_q, head_dim = q.shape
    k_batch, num_kv_heads, seqlen_kv, k_head_dim = k.shape
    v_batch, v_heads, v_seqlen, v_head_dim = v.shape
    if batch != k_batch or batch != v_batch:
        raise ValueError("Q, K, and V must share batch dimension")
    if seqlen_kv != v_seqlen:
        raise ValueError("K and V must share sequence length")
    if k_head_dim != v_head_dim or head_dim != k_head_dim:
        raise ValueError("Q, K, and V must share head_dim")
    if v_heads != num_kv_heads:
        raise ValueError("K and V must share number of KV heads")
    if q_heads % num_kv_heads != 0:
        raise ValueError("Query heads must be divisible by KV heads")
    if head_dim != HEAD_DIM:
        raise ValueError("this build supports head_dim == 128 only")
    if out is None:
        out = torch.empty_like(q)
    if not out.is_contiguous():
        raise ValueError("Output tensor must be contiguous")
    if seqlen_q == 1:
        gqa_decode(q.view(batch, q_heads, head_dim), k, v, kv_layout=KV_BHSD, out=out.view(batch, q_heads, head_dim))
    else:
        row0 = gqa_decode(q[:, :, 0, :].contiguous(), k, v, kv_layout=KV_BHSD)
        out[:, :, 0, :] = row0
    return out


def launch_flash_gqa_forward_bf16_kernel(q, k, v, scale=None, out=None, lse=None, causal=True, **_tuning):
    """Mirror of upstream's Triton prefill launcher (flash_gqa_kernel.py:185-338).

    Accepts [Hq,Sq,D] / [Hkv,Skv,D] or the batched 4-D forms, ``causal=True`` by default (:192), returns
    ``(out, lse)`` with lse = rowmax + log(rowsum) in fp32 (:132).  Upstream's Triton tuning keywords
    (block_kv_sub, num_warps, num_stages) are accepted and ignored.
    """
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("Flash GQA forward expects bf16 inputs")
    if q.dim() not in (3, 4):
        raise ValueError("Q must be 3D or 4D")
    if k.dim() != q.dim() or v.dim() != q.dim():
        raise ValueError("Q, K, and V must have matching ranks")
    for name, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(name, t)
    squeeze = q.dim() == 3
    qb, kb, vb = (t.contiguous().unsqueeze(0) if squeeze else t.contiguous() for t in (q, k, v))
    batch, q_heads, seqlen_q, head_dim_qk = qb.shape
    _, num_kv_heads, seqlen_kv, k_head_dim = kb.shape
    _, v_heads, v_seqlen, head_dim_v = vb.shape
    if seqlen_kv != v_seqlen:
        raise ValueError("K and V must share sequence length")
    if k_head_dim != head_dim_qk:
        raise ValueError("Q and K must share head_dim_qk")
    if v_heads != num_kv_heads:
        raise ValueError("K and V must share number of KV heads")
    if q_heads % num_kv_heads != 0:
        raise ValueError("Query heads must be divisible by KV heads")
    if head_dim_qk != HEAD_DIM or head_dim_v != HEAD_DIM:
        raise ValueError("this build supports head_dim == 128 only")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim_qk)
    if out is None:
        out_b = torch.empty((batch, q_heads, seqlen_q, head_dim_v), device=qb.device, dtype=qb.dtype)
    else:
        if out.dim() != q.dim():
            raise ValueError("Output must be 3D when Q is 3D" if squeeze else "Output must be 4D when Q is 4D")
        if not out.is_contiguous():
            raise ValueError("Output tensor must be contiguous")
        out_b = out.unsqueeze(0) if squeeze else out
    if tuple(out_b.shape) != (batch, q_heads, seqlen_q, head_dim_v):
        raise ValueError("Output must have shape [batch, q_heads, seqlen_q, head_dim_v]")
    if lse is None:
        lse_b = torch.empty((batch, q_heads, seqlen_q), device=qb.device, dtype=torch.float32)
    else:
        if lse.dim() != q.dim() - 1:
            raise ValueError("LSE must be 2D when Q is 3D" if squeeze else "LSE must be 3D when Q is 4D")
        if not lse.is_contiguous() or lse.dtype != torch.float32:
            raise ValueError("LSE must be contiguous fp32")
        lse_b = lse.unsqueeze(0) if squeeze else lse
    with torch.cuda.device(qb.device):
        lib = _lib.load()
        # a few query rows against a long cache: the library asks for scratch to share the kv range out among blocks
        ws_bytes = 0 if causal else int(lib.cllo_gqa_prefill_workspace_bytes(batch, seqlen_q, seqlen_kv, q_heads,
                                                                             num_kv_heads, 0))
        if ws_bytes:
            ws = _workspace(qb.device, ws_bytes, kind="prefill")
            rc = lib.cllo_gqa_prefill_fwd_ws_bf16(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), float(scale), 0,
                                                  out_b.data_ptr(), lse_b.data_ptr(), ws.data_ptr(), ws.numel(),
                                                  batch, seqlen_q, seqlen_kv, q_heads, num_kv_heads, head_dim_qk,
                                                  _stream_ptr())
        else:
            rc = lib.cllo_gqa_prefill_fwd_bf16(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), float(scale),
                                               1 if causal else 0, out_b.data_ptr(), lse_b.data_ptr(),
                                               batch, seqlen_q, seqlen_kv, q_heads, num_kv_heads, head_dim_qk,
                                               _stream_ptr())
    _lib.check(rc, "cllo_gqa_prefill_fwd_bf16")
    if squeeze:
        return out_b.squeeze(0), lse_b.squeeze(0)
    return out_b, lse_b


def launch_flash_swa_forward_bf16_kernel(q, k, v, scale=None, out=None, lse=None, window_size=None, sink_value=None,
                                         **_tuning):
    """Mirror of upstream's sliding-window launcher (src/python/Triton/SWA/flash_swa_kernel.py:186-330).

    A query at position i attends to kv positions [i - (window_size - 1), i]; ``sink_value`` (fp32 [q_heads]) enters
    the softmax denominator as ``sink * exp(-rowmax)``.  Same ranks, layouts, checks and return value ``(out, lse)``
    as upstream; its Triton tuning keywords are accepted and ignored.
    """
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("Flash SWA forward expects bf16 inputs")
    if q.dim() not in (3, 4):
        raise ValueError("Q must be 3D or 4D")
    if k.dim() != q.dim() or v.dim() != q.dim():
        raise ValueError("Q, K, and V must have matching ranks")
    squeeze = q.dim() == 3
    qb, kb, vb = (t.contiguous().unsqueeze(0) if squeeze else t.contiguous() for t in (q, k, v))
    batch, q_heads, seqlen_q, head_dim_qk = qb.shape
    _, num_kv_heads, seqlen_kv, k_head_dim = kb.shape
    _, v_heads, v_seqlen, head_dim_v = vb.shape
    if seqlen_kv != v_seqlen:
        raise ValueError("K and V must share sequence length")
    if k_head_dim != head_dim_qk:
        raise ValueError("Q and K must share head_dim_qk")
    if v_heads != num_kv_heads:
        raise ValueError("K and V must share number of KV heads")
    if q_heads % num_kv_heads != 0:
        raise ValueError("Query heads must be divisible by KV heads")
    if window_size is None:
        raise ValueError("window_size must be provided")
    if sink_value is None:
        raise ValueError("sink_value must be provided")
    if not isinstance(sink_value, torch.Tensor):
        raise ValueError("sink_value must be a torch.Tensor")
    if sink_value.dim() != 1:
        raise ValueError("sink_value must be a 1D tensor with shape [q_heads]")
    if sink_value.numel() != q_heads:
        raise ValueError(f"sink_value must have {q_heads} elements")
    if sink_value.device != qb.device:
        raise ValueError("sink_value must be on the same device as Q")
    for name, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(name, t)
    if head_dim_qk != HEAD_DIM or head_dim_v != HEAD_DIM:
        raise ValueError("this build supports head_dim == 128 only")
    if int(window_size) <= 0:
        raise ValueError("window_size must be positive")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim_qk)
    if out is None:
        out_b = torch.empty((batch, q_heads, seqlen_q, head_dim_v), device=qb.device, dtype=qb.dtype)
    else:
        if out.dim() != q.dim():
            raise ValueError("Output must be 3D when Q is 3D" if squeeze else "Output must be 4D when Q is 4D")
        out_b = out.unsqueeze(0) if squeeze else out
    if tuple(out_b.shape) != (batch, q_heads, seqlen_q, head_dim_v) or not out_b.is_contiguous():
        raise ValueError("Output must have shape [batch, q_heads, seqlen_q, head_dim_v]")
    if lse is None:
        lse_b = torch.empty((batch, q_heads, seqlen_q), device=qb.device, dtype=torch.float32)
    else:
        if lse.dim() != q.dim() - 1:
            raise ValueError("LSE must be 2D when Q is 3D" if squeeze else "LSE must be 3D when Q is 4D")
        lse_b = lse.unsqueeze(0) if squeeze else lse
    if tuple(lse_b.shape) != (batch, q_heads, seqlen_q) or not lse_b.is_contiguous() or lse_b.dtype != torch.float32:
        raise ValueError("LSE must have shape [batch, q_heads, seqlen_q]")
    sink = sink_value.to(torch.float32).contiguous()
    with torch.cuda.device(qb.device):
        rc = _lib.load().cllo_swa_prefill_fwd_bf16(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), float(scale),
                                                   int(window_size), sink.data_ptr(), out_b.data_ptr(),
                                                   lse_b.data_ptr(), batch, seqlen_q, seqlen_kv, q_heads, num_kv_heads,
                                                   head_dim_qk, _stream_ptr())
    _lib.check(rc, "cllo_swa_prefill_fwd_bf16")
    if squeeze:
        return out_b.squeeze(0), lse_b.squeeze(0)
    return out_b, lse_b


def launch_flash_mla_forward_bf16_kernel(q, k, v, scale=None, out=None, lse=None, causal=True, **_tuning):
    """Mirror of upstream's MLA forward launcher (src/python/Triton/flash_mla_kernel.py:315-508).

    The attention of ``launch_flash_gqa_forward_bf16_kernel`` with Q/K heads wider than V heads: q ``[.., seqlen_q,
    head_dim_qk]``, k ``[.., seqlen_kv, head_dim_qk]``, v ``[.., seqlen_kv, head_dim_v]``, out ``[.., seqlen_q,
    head_dim_v]``.  Same ranks, layouts, checks and return value ``(out, lse)`` as upstream; its Triton tuning keywords
    are accepted and ignored.  This build supports head_dim_qk = 192 with head_dim_v = 128.
    """
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("Flash MLA forward expects bf16 inputs")
    if q.dim() not in (3, 4):
        raise ValueError("Q must be 3D or 4D")
    if k.dim() != q.dim() or v.dim() != q.dim():
        raise ValueError("Q, K, and V must have matching ranks")
    squeeze = q.dim() == 3
    qb, kb, vb = (t.contiguous().unsqueeze(0) if squeeze else t.contiguous() for t in (q, k, v))
    batch, q_heads, seqlen_q, head_dim_qk = qb.shape
    _, num_kv_heads, seqlen_kv, k_head_dim = kb.shape
    _, v_heads, v_seqlen, head_dim_v = vb.shape
    if seqlen_kv != v_seqlen:
        raise ValueError("K and V must share sequence length")
    if k_head_dim != head_dim_qk:
        raise ValueError("Q and K must share head_dim_qk")
    if v_heads != num_kv_heads:
        raise ValueError("K and V must share number of KV heads")
    if q_heads % num_kv_heads != 0:
        raise ValueError("Query heads must be divisible by KV heads")
    for name, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(name, t)
    if head_dim_qk != 192 or head_dim_v != 128:
        raise ValueError("this build supports head_dim_qk == 192 with head_dim_v == 128 only")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim_qk)
    if out is None:
        out_b = torch.empty((batch, q_heads, seqlen_q, head_dim_v), device=qb.device, dtype=qb.dtype)
    else:
        if out.dim() != q.dim():
            raise ValueError("Output must be 3D when Q is 3D" if squeeze else "Output must be 4D when Q is 4D")
        out_b = out.unsqueeze(0) if squeeze else out
    if tuple(out_b.shape) != (batch, q_heads, seqlen_q, head_dim_v) or not out_b.is_contiguous():
        raise ValueError("Output must have shape [batch, q_heads, seqlen_q, head_dim_v]")
    if lse is None:
        lse_b = torch.empty((batch, q_heads, seqlen_q), device=qb.device, dtype=torch.float32)
    else:
        if lse.dim() != q.dim() - 1:
            raise ValueError("LSE must be 2D when Q is 3D" if squeeze else "LSE must be 3D when Q is 4D")
        lse_b = lse.unsqueeze(0) if squeeze else lse
    if tuple(lse_b.shape) != (batch, q_heads, seqlen_q) or not lse_b.is_contiguous() or lse_b.dtype != torch.float32:
        raise ValueError("LSE must have shape [batch, q_heads, seqlen_q]")
    if seqlen_q > 0:
        with torch.cuda.device(qb.device):
            rc = _lib.load().cllo_mla_prefill_fwd_bf16(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), float(scale),
                                                       1 if causal else 0, out_b.data_ptr(), lse_b.data_ptr(), batch,
                                                       seqlen_q, seqlen_kv, q_heads, num_kv_heads, head_dim_qk,
                                                       head_dim_v, _stream_ptr())
        _lib.check(rc, "cllo_mla_prefill_fwd_bf16")
    if squeeze:
        return out_b.squeeze(0), lse_b.squeeze(0)
    return out_b, lse_b


def launch_flash_sgqa_forward_bf16_kernel(q, k, v, sparse_kv_indices, num_sparse_kv, scale=None, out=None, lse=None,
                                          causal=True, block_sparse_sub=None, num_warps=None, num_stages=None):
    """Mirror of upstream's sparse-index GQA launcher (src/python/Triton/SparseGQA/flash_sgqa_kernel.py:202-396).

    ``sparse_kv_indices`` (int32 ``[batch, num_kv_heads, seqlen_q, num_sparse_kv]``) lists, per kv head and query token,
    the kv tokens that token attends to; entries outside ``[0, seqlen_kv)`` (upstream pads with -1) and, when
    ``causal``, entries above the query position are ignored.  Same ranks, layouts, checks and return value
    ``(out, lse)`` as upstream; its Triton tuning keywords are validated as upstream does and otherwise ignored.
    """
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("Flash SGQA forward expects bf16 inputs")
    if sparse_kv_indices.dtype != torch.int32:
        raise ValueError("sparse_kv_indices must be int32")
    if sparse_kv_indices.dim() != 4:
        raise ValueError("sparse_kv_indices must be 4D [batch, num_kv_heads, seqlen_q, num_sparse_kv]")
    if not isinstance(num_sparse_kv, int):
        raise ValueError("num_sparse_kv must be an int")
    if num_sparse_kv < 1:
        raise ValueError("num_sparse_kv must be >= 1")
    if block_sparse_sub is not None and (not isinstance(block_sparse_sub, int) or block_sparse_sub < 1):
        raise ValueError("block_sparse_sub must be None or an int >= 1")
    if num_warps is not None and (not isinstance(num_warps, int) or num_warps < 1):
        raise ValueError("num_warps must be None or an int >= 1")
    if num_stages is not None and (not isinstance(num_stages, int) or num_stages < 1):
        raise ValueError("num_stages must be None or an int >= 1")
    if q.dim() not in (3, 4):
        raise ValueError("Q must be 3D or 4D")
    if k.dim() != q.dim() or v.dim() != q.dim():
        raise ValueError("Q, K, and V must have matching ranks")
    squeeze = q.dim() == 3
    qb, kb, vb = (t.contiguous().unsqueeze(0) if squeeze else t.contiguous() for t in (q, k, v))
    batch, q_heads, seqlen_q, head_dim_qk = qb.shape
    _, num_kv_heads, seqlen_kv, k_head_dim = kb.shape
    _, v_heads, v_seqlen, head_dim_v = vb.shape
    if seqlen_kv != v_seqlen:
        raise ValueError("K and V must share sequence length")
    if k_head_dim != head_dim_qk:
        raise ValueError("Q and K must share head_dim_qk")
    if v_heads != num_kv_heads:
        raise ValueError("K and V must share number of KV heads")
    if q_heads % num_kv_heads != 0:
        raise ValueError("Query heads must be divisible by KV heads")
    if tuple(sparse_kv_indices.shape) != (batch, num_kv_heads, seqlen_q, num_sparse_kv):
        raise ValueError("sparse_kv_indices must have shape "
                         f"[batch, num_kv_heads, seqlen_q, {num_sparse_kv}]")
    for name, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(name, t)
    if sparse_kv_indices.device != qb.device:
        raise ValueError("sparse_kv_indices must be on the same device as Q")
    if head_dim_qk != HEAD_DIM or head_dim_v != HEAD_DIM:
        raise ValueError("this build supports head_dim == 128 only")
    if q_heads // num_kv_heads > 16:
        raise ValueError("this build supports at most 16 query heads per KV head")
    idx = sparse_kv_indices.contiguous()
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim_qk)
    if out is None:
        out_b = torch.empty((batch, q_heads, seqlen_q, head_dim_v), device=qb.device, dtype=qb.dtype)
    else:
        if out.dim() != q.dim():
            raise ValueError("Output must be 3D when Q is 3D" if squeeze else "Output must be 4D when Q is 4D")
        if not out.is_contiguous():
            raise ValueError("Output must be contiguous when provided")
        out_b = out.unsqueeze(0) if squeeze else out
    if tuple(out_b.shape) != (batch, q_heads, seqlen_q, head_dim_v):
        raise ValueError("Output must have shape [batch, q_heads, seqlen_q, head_dim_v]")
    if lse is None:
        lse_b = torch.empty((batch, q_heads, seqlen_q), device=qb.device, dtype=torch.float32)
    else:
        if lse.dim() != q.dim() - 1:
            raise ValueError("LSE must be 2D when Q is 3D" if squeeze else "LSE must be 3D when Q is 4D")
        if not lse.is_contiguous():
            raise ValueError("LSE must be contiguous when provided")
        lse_b = lse.unsqueeze(0) if squeeze else lse
    if tuple(lse_b.shape) != (batch, q_heads, seqlen_q) or lse_b.dtype != torch.float32:
        raise ValueError("LSE must have shape [batch, q_heads, seqlen_q]")
    if seqlen_q > 0:
        with torch.cuda.device(qb.device):
            rc = _lib.load().cllo_sgqa_prefill_fwd_bf16(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), idx.data_ptr(),
                                                        num_sparse_kv, float(scale), 1 if causal else 0,
                                                        out_b.data_ptr(), lse_b.data_ptr(), batch, seqlen_q, seqlen_kv,
                                                        q_heads, num_kv_heads, head_dim_qk, _stream_ptr())
        _lib.check(rc, "cllo_sgqa_prefill_fwd_bf16")
    if squeeze:
        return out_b.squeeze(0), lse_b.squeeze(0)
    return out_b, lse_b


def launch_flash_gqa_backward_bf16_kernel(q, k, v, o, lse, grad_o, scale=None, causal=True, **_tuning):
    """Mirror of upstream's backward launcher (src/python/Triton/flash_gqa_backward_kernel.py:312-478).

    3-D or 4-D tensors as the forward launcher; ``lse`` is the forward's fp32 log-sum-exp; returns
    ``(grad_q, grad_k, grad_v)`` in bf16 with the shapes of q, k, v.  Upstream's Triton tuning keywords are accepted
    and ignored.
    """
    return _attention_backward(q, k, v, o, lse, grad_o, scale, causal, 0, "Flash GQA backward")


def launch_flash_swa_backward_bf16_kernel(q, k, v, o, lse, grad_o, scale=None, window_size=None, **_tuning):
    """Mirror of upstream's sliding-window backward launcher (src/python/Triton/SWA/flash_swa_backward_kernel.py:323).

    ``lse`` is the log-sum-exp written by ``launch_flash_swa_forward_bf16_kernel`` (it already contains the sink term,
    which is all the backward needs of it).
    """
    if window_size is None:
        raise ValueError("window_size must be provided")
    if int(window_size) <= 0:
        raise ValueError("window_size must be positive")
    return _attention_backward(q, k, v, o, lse, grad_o, scale, True, int(window_size), "Flash SWA backward")


def _attention_backward(q, k, v, o, lse, grad_o, scale, causal, window, what):
    if (q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16
            or o.dtype != torch.bfloat16 or grad_o.dtype != torch.bfloat16):
        raise ValueError(what + " expects bf16 inputs and grad_o")
    if lse.dtype != torch.float32:
        raise ValueError(what + " expects lse to be float32")
    if q.dim() not in (3, 4):
        raise ValueError("Q must be 3D or 4D")
    if k.dim() != q.dim() or v.dim() != q.dim() or o.dim() != q.dim() or grad_o.dim() != q.dim():
        raise ValueError("Q, K, V, O, and grad_o must have matching ranks")
    squeeze = q.dim() == 3
    qb, kb, vb, ob, gob = (t.contiguous().unsqueeze(0) if squeeze else t.contiguous() for t in (q, k, v, o, grad_o))
    lse_b = (lse.contiguous().unsqueeze(0) if squeeze else lse.contiguous())
    batch, q_heads, seqlen_q, head_dim_qk = qb.shape
    _, num_kv_heads, seqlen_kv, k_head_dim = kb.shape
    _, v_heads, v_seqlen, head_dim_v = vb.shape
    if seqlen_kv != v_seqlen:
        raise ValueError("K and V must share sequence length")
    if tuple(ob.shape) != (batch, q_heads, seqlen_q, head_dim_v) or ob.shape != gob.shape:
        raise ValueError("O and grad_o must have shape [batch, q_heads, seqlen_q, head_dim_v]")
    if k_head_dim != head_dim_qk:
        raise ValueError("Q and K must share head_dim_qk")
    if v_heads != num_kv_heads:
        raise ValueError("K and V must share number of KV heads")
    if q_heads % num_kv_heads != 0:
        raise ValueError("Query heads must be divisible by KV heads")
    if tuple(lse_b.shape) != (batch, q_heads, seqlen_q):
        raise ValueError("LSE must have shape [batch, q_heads, seqlen_q]")
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o), ("grad_o", grad_o)):
        _require_cuda_bf16(name, t)
    if head_dim_qk != HEAD_DIM or head_dim_v != HEAD_DIM:
        raise ValueError("this build supports head_dim == 128 only")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim_qk)
    grad_q, grad_k, grad_v = torch.empty_like(qb), torch.empty_like(kb), torch.empty_like(vb)
    lib = _lib.load()
    with torch.cuda.device(qb.device):
        nbytes = int(lib.cllo_gqa_bwd_workspace_bytes(batch, seqlen_q, seqlen_kv, q_heads, num_kv_heads))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=qb.device)
        fn = lib.cllo_swa_bwd_bf16 if window > 0 else lib.cllo_gqa_bwd_bf16
        rc = fn(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), ob.data_ptr(), lse_b.data_ptr(), gob.data_ptr(),
                float(scale), window if window > 0 else (1 if causal else 0), grad_q.data_ptr(), grad_k.data_ptr(),
                grad_v.data_ptr(), ws.data_ptr(), nbytes, batch, seqlen_q, seqlen_kv, q_heads, num_kv_heads, head_dim_qk,
                _stream_ptr())
    _lib.check(rc, "cllo_swa_bwd_bf16" if window > 0 else "cllo_gqa_bwd_bf16")
    if squeeze:
        return grad_q.squeeze(0), grad_k.squeeze(0), grad_v.squeeze(0)
    return grad_q, grad_k, grad_v


def LaunchRopeBf16Kernel(input, output, batchSize, seqLen, hiddenDim, base=10000.0):
    """Mirror of upstream's C++ RoPE launcher (include/cplusplus/RoPE/rope_kernel.cuh:22), tensors instead of pointers.

    input/output [batchSize, seqLen, hiddenDim] bf16 (the same tensor is allowed).  Like upstream it returns None and
    does nothing on sizes it refuses (rope_kernel.cu:124-136): non-positive sizes, hiddenDim not a multiple of 8.
    """
    if batchSize <= 0 or seqLen <= 0 or hiddenDim <= 0 or hiddenDim % 8 != 0:
        return
    _require_cuda_bf16("input", input)
    _require_cuda_bf16("output", output)
    with torch.cuda.device(input.device):
        rc = _lib.load().cllo_rope_bf16(input.data_ptr(), output.data_ptr(), batchSize, seqLen, hiddenDim, float(base),
                                        _stream_ptr())
    _lib.check(rc, "cllo_rope_bf16")


def device_status():
    """Synchronise and return (status, detail) from ``cllo_device_status``."""
    import ctypes
    detail = (ctypes.c_int * 4)()
    rc = _lib.load().cllo_device_status(detail)
    if rc != 0:
        # a kernel gave up half-way: the cached workspaces may hold counts of pieces that never got merged
        with _workspaces_lock:
            for ws in _workspaces.values():
                ws.zero_()
    return rc, list(detail)
