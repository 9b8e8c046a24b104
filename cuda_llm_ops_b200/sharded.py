"""Multi-GPU use of the GQA path: one process per GPU, ``torch.distributed`` for the plumbing.

Upstream has no multi-GPU code at all; these are the two shardings the path admits.

* Independent sequences (decode or prefill over a batch): give every rank a contiguous slice of the
  batch (``shard_batch``) and run the single-GPU entry point on it.  No collective.
* One long sequence (decode): split the KV cache by position (``shard_kv_positions``).  Every rank runs the
  split-KV decode over its own positions and produces one packed fp32 partial ``(O, m, l)`` per query
  head; ONE all-gather brings all ranks' partials into local memory and the log-sum-exp combine kernel
  merges them, so every rank ends with the full output.  The partials are tiny (Hq * (D+2) floats per
  rank), so the exchange is latency-bound; kernels only ever read local memory.
"""
import ctypes

import torch
import torch.distributed as dist

from . import _lib, flash_gqa


def shard_batch(batch, world_size, rank):
    """Contiguous [begin, end) slice of ``batch`` sequences for ``rank``; sizes differ by at most one."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank/world_size")
    base, extra = divmod(batch, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_kv_positions(seq_len, world_size, rank, align=64):
    """Contiguous [begin, end) range of KV positions for ``rank``.

    Boundaries are multiples of ``align`` (the decode kernel's tile) except the last one; trailing ranks may
    get an empty range when the sequence is short, which the combine step ignores (l == 0).
    """
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank/world_size")
    tiles = (seq_len + align - 1) // align
    base, extra = divmod(tiles, world_size)
    t0 = rank * base + min(rank, extra)
    t1 = t0 + base + (1 if rank < extra else 0)
    return min(t0 * align, seq_len), min(t1 * align, seq_len)


class _PeerBuffers:
    """Gather slots and flag words in memory that every rank of the node can address (torch symmetric memory).

    Layout per rank: [2 parities][world][rows][D+2] fp32 gather slots, then `world` uint32 flag words and
    one launch counter.
    """

    def __init__(self, group, rows, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.world = dist.get_world_size(group)
        self.rows = rows
        n_gather = 2 * self.world * rows * flash_gqa.PARTIAL_WIDTH
        self.storage = symm_mem.empty(n_gather + 64, dtype=torch.float32, device=device)
        self.storage.zero_()
        handle = symm_mem.rendezvous(self.storage, group if group is not None else dist.group.WORLD)
        ptrs = [int(x) for x in handle.buffer_ptrs]
        self.handle = handle
        arr = ctypes.c_void_p * self.world
        self.gather_ptrs = arr(*ptrs)
        self.flag_ptrs = arr(*[x + n_gather * 4 for x in ptrs])
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flag words are zero before anybody publishes an epoch


class KVShardedDecoder:
    """Decode of sequences whose KV cache is sharded by position across the ranks of ``group``.

    ``exchange`` selects how the per-rank partials meet:
      * ``"peer"``: one kernel (``cllo_gqa_exchange_combine_bf16``) stores the local partial into every
        peer's memory, waits for the peers' flags and merges -- no library collective;
      * ``"nccl"``: ``all_gather_into_tensor`` followed by the combine kernel (also the path CPU ranks take);
      * ``"auto"``: ``"peer"`` when the ranks can map each other's memory, else ``"nccl"``.

    ``decode_fn(q, k, v, scale, kv_layout, partial_out)`` and ``combine_fn(partials) -> out`` default to the
    CUDA entry points; tests on CPU ranks (gloo) inject checker implementations to exercise the exchange.
    """

    def __init__(self, group=None, decode_fn=None, combine_fn=None, exchange="nccl"):
        if exchange not in ("nccl", "peer", "auto"):
            raise ValueError("exchange must be 'nccl', 'peer' or 'auto'")
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._decode = decode_fn or self._cuda_decode
        self._combine = combine_fn or flash_gqa.gqa_combine
        self._gathered = None
        self._exchange_request = exchange
        self.exchange = "nccl"  # what is actually in use; settled at the first decode on a device
        self._peer = None
        self._local = None

    @staticmethod
    def _cuda_decode(q, k, v, scale, kv_layout, partial_out):
        return flash_gqa.gqa_decode(q, k, v, scale=scale, kv_layout=kv_layout, partial_out=partial_out)

    def _buffers(self, B, Hq, device):
        shape = (self.world_size, B, Hq, flash_gqa.PARTIAL_WIDTH)
        if self._gathered is None or tuple(self._gathered.shape) != shape or self._gathered.device != device:
            self._gathered = torch.zeros(shape, dtype=torch.float32, device=device)
        return self._gathered

    def _setup_peer(self, rows, device):
        """Try to set up peer-addressable buffers; every rank must agree on the outcome."""
        ok = 1
        try:
            peer = _PeerBuffers(self.group, rows, device)
        except Exception as exc:  # symmetric memory unavailable (no P2P, old driver, ...)
            if self._exchange_request == "peer":
                raise
            peer, ok = None, 0
            self._peer_error = repr(exc)
        flag = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 1:
            self._peer, self.exchange = peer, "peer"
        else:
            self._peer, self.exchange = None, "nccl"

    def local_partial(self, q, k_local, v_local, scale=None, kv_layout=flash_gqa.KV_BHSD, out=None):
        """This rank's packed (O, m, l): into ``out`` if given, else straight into its slot of the gather buffer."""
        B, Hq, _ = q.shape
        mine = out if out is not None else self._buffers(B, Hq, q.device)[self.rank]
        s_axis = 1 if kv_layout == flash_gqa.KV_BSHD else 2
        if k_local.shape[s_axis] == 0:
            mine.zero_()
            mine[..., flash_gqa.HEAD_DIM] = float("-inf")
        else:
            self._decode(q, k_local, v_local, scale, kv_layout, mine)
        return mine

    def decode(self, q, k_local, v_local, scale=None, kv_layout=flash_gqa.KV_BHSD, out=None):
        """q [B,Hq,D] replicated; k_local/v_local hold this rank's positions.  Returns the full O on every rank."""
        B, Hq, D = q.shape
        if self._exchange_request != "nccl" and q.is_cuda and self.world_size > 1:
            if self._peer is None and self.exchange == "nccl" and not getattr(self, "_peer_tried", False):
                self._peer_tried = True
                self._setup_peer(B * Hq, q.device)
            if self._peer is not None and self._peer.rows == B * Hq:
                return self._decode_peer(q, k_local, v_local, scale, kv_layout, out)
        mine = self.local_partial(q, k_local, v_local, scale, kv_layout)
        gathered = self._gathered
        if self.world_size > 1:
            # NCCL gathers in place (this rank's slot already holds its partial); CPU backends get a copy
            src = mine.reshape(-1) if mine.is_cuda else mine.reshape(-1).clone()
            dist.all_gather_into_tensor(gathered.view(-1), src, group=self.group)
        merged = self._combine(gathered)
        if out is not None:
            out.copy_(merged)
            return out
        return merged

    def _decode_peer(self, q, k_local, v_local, scale, kv_layout, out):
        B, Hq, D = q.shape
        if self._local is None or tuple(self._local.shape) != (B, Hq, flash_gqa.PARTIAL_WIDTH):
            self._local = torch.zeros((B, Hq, flash_gqa.PARTIAL_WIDTH), dtype=torch.float32, device=q.device)
        self.local_partial(q, k_local, v_local, scale, kv_layout, out=self._local)
        if out is None:
            out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=q.device)
        peer = self._peer
        with torch.cuda.device(q.device):
            # epoch 0: the kernel counts its launches on the device, so this call can sit in a CUDA graph
            rc = _lib.load().cllo_gqa_exchange_combine_bf16(
                self._local.data_ptr(), peer.gather_ptrs, peer.flag_ptrs, self.rank, self.world_size, 0,
                out.data_ptr(), B * Hq, D, torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "cllo_gqa_exchange_combine_bf16")
        return out
