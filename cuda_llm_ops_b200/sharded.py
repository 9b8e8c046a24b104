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

    Layout per rank as ``include/cllo_flash_gqa.h`` describes it: [2 parities][world][rows][D+2] fp32 gather
    slots, then [world][CLLO_SHARD_MAX_UNITS] uint32 flag words and one completion counter, all zero at first.
    """

    def __init__(self, group, B, Hq, device):
        import torch.distributed._symmetric_memory as symm_mem
        lib = _lib.load()
        self.world = dist.get_world_size(group)
        self.shape = (B, Hq)
        gather_bytes = int(lib.cllo_gqa_shard_gather_bytes(self.world, B, Hq, flash_gqa.HEAD_DIM))
        flag_bytes = int(lib.cllo_gqa_shard_flag_bytes(self.world))
        if gather_bytes == 0 or flag_bytes == 0:
            raise ValueError("unsupported world size or shape for the peer exchange")
        self.storage = symm_mem.empty((gather_bytes + flag_bytes + 255) // 4, dtype=torch.float32, device=device)
        self.storage.zero_()
        handle = symm_mem.rendezvous(self.storage, group if group is not None else dist.group.WORLD)
        ptrs = [int(x) for x in handle.buffer_ptrs]
        self.handle = handle
        arr = ctypes.c_void_p * self.world
        self.gather_ptrs = arr(*ptrs)
        self.flag_ptrs = arr(*[x + gather_bytes for x in ptrs])
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flag words are zero before anybody publishes a step


class KVShardedDecoder:
    """Decode of sequences whose KV cache is sharded by position across the ranks of ``group``.

    ``exchange`` selects how the per-rank partials meet:
      * ``"fused"``: ONE kernel per step (``cllo_gqa_decode_sharded_bf16``): the split-KV decode publishes each
        head group's merged partial to every peer as soon as it is complete, waits for the peers' and writes the
        final output -- no library collective, no second launch;
      * ``"peer"``: decode into a local partial, then ``cllo_gqa_exchange_combine_bf16`` (same exchange protocol,
        driven from memory);
      * ``"nccl"``: ``all_gather_into_tensor`` followed by the combine kernel (also the path CPU ranks take);
      * ``"auto"``: ``"fused"`` when the ranks can map each other's memory, else ``"nccl"``.

    The peer forms wait for each other on the device with a bound (about a second; ``set_exchange_wait_limit``):
    a rank that is later than that makes the others give up, their output rows become NaN and the device status
    reports a time-out.  ``decode(..., check=True)`` reads that status (it synchronises the device) and raises.
    The NCCL form simply waits.

    ``decode_fn(q, k, v, scale, kv_layout, partial_out)`` and ``combine_fn(partials) -> out`` default to the
    CUDA entry points; tests on CPU ranks (gloo) inject checker implementations to exercise the exchange.
    """

    def __init__(self, group=None, decode_fn=None, combine_fn=None, exchange="nccl"):
        if exchange not in ("nccl", "peer", "fused", "auto"):
            raise ValueError("exchange must be 'nccl', 'peer', 'fused' or 'auto'")
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._decode = decode_fn or self._cuda_decode
        self._combine = combine_fn or flash_gqa.gqa_combine
        self._gathered = None
        self._exchange_request = exchange
        self.exchange = "nccl"  # what is actually in use; settled at the first decode on a device
        self._peer = None
        self._peer_tried = False
        self._local = None

    @staticmethod
    def _cuda_decode(q, k, v, scale, kv_layout, partial_out):
        return flash_gqa.gqa_decode(q, k, v, scale=scale, kv_layout=kv_layout, partial_out=partial_out)

    def _buffers(self, B, Hq, device):
        shape = (self.world_size, B, Hq, flash_gqa.PARTIAL_WIDTH)
        if self._gathered is None or tuple(self._gathered.shape) != shape or self._gathered.device != device:
            self._gathered = torch.zeros(shape, dtype=torch.float32, device=device)
        return self._gathered

    def _setup_peer(self, B, Hq, device):
        """Try to set up peer-addressable buffers; every rank must agree on the outcome."""
        ok = 1
        try:
            peer = _PeerBuffers(self.group, B, Hq, device)
        except Exception as exc:  # symmetric memory unavailable (no P2P, old driver, ...) or shape not supported
            if self._exchange_request in ("peer", "fused"):
                raise
            peer, ok = None, 0
            self._peer_error = repr(exc)
        flag = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 1:
            self._peer = peer
            self.exchange = "peer" if self._exchange_request == "peer" else "fused"
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

    def decode(self, q, k_local, v_local, scale=None, kv_layout=flash_gqa.KV_BHSD, out=None, check=False):
        """q [B,Hq,D] replicated; k_local/v_local hold this rank's positions.  Returns the full O on every rank."""
        B, Hq, D = q.shape
        if self._exchange_request != "nccl" and q.is_cuda and self.world_size > 1:
            if not self._peer_tried:
                self._peer_tried = True
                self._setup_peer(B, Hq, q.device)
            if self._peer is not None and self._peer.shape == (B, Hq):
                res = self._decode_peer(q, k_local, v_local, scale, kv_layout, out)
                if check:
                    rc, detail = flash_gqa.device_status()
                    if rc != 0:
                        raise RuntimeError("sharded decode: a peer did not deliver its partial in time "
                                           "(device status %d, detail %s); the output holds NaN" % (rc, detail))
                return res
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
        if out is None:
            out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=q.device)
        peer = self._peer
        s_axis = 1 if kv_layout == flash_gqa.KV_BSHD else 2
        if self.exchange == "fused" and k_local.shape[s_axis] > 0:
            # epoch 0: the kernels count their launches on the device, so a step can sit in a CUDA graph
            flash_gqa.gqa_decode_sharded(q, k_local, v_local, peer.gather_ptrs, peer.flag_ptrs, self.rank,
                                         self.world_size, epoch=0, scale=scale, kv_layout=kv_layout, out=out)
            return out
        # two launches: this rank's partial (an empty share gives l = 0 rows), then the exchange from memory
        if self._local is None or tuple(self._local.shape) != (B, Hq, flash_gqa.PARTIAL_WIDTH):
            self._local = torch.zeros((B, Hq, flash_gqa.PARTIAL_WIDTH), dtype=torch.float32, device=q.device)
        self.local_partial(q, k_local, v_local, scale, kv_layout, out=self._local)
        Hkv = k_local.shape[2] if kv_layout == flash_gqa.KV_BSHD else k_local.shape[1]
        with torch.cuda.device(q.device):
            rc = _lib.load().cllo_gqa_exchange_combine_bf16(
                self._local.data_ptr(), peer.gather_ptrs, peer.flag_ptrs, self.rank, self.world_size, 0,
                out.data_ptr(), B, Hq, Hkv, D, torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "cllo_gqa_exchange_combine_bf16")
        return out
