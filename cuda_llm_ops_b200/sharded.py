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
import torch
import torch.distributed as dist

from . import flash_gqa


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


class KVShardedDecoder:
    """Decode of sequences whose KV cache is sharded by position across the ranks of ``group``.

    ``decode_fn(q, k, v, scale, kv_layout, partial_out)`` and ``combine_fn(partials) -> out`` default to the
    CUDA entry points; tests on CPU ranks (gloo) inject checker implementations to exercise the exchange.
    """

    def __init__(self, group=None, decode_fn=None, combine_fn=None):
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._decode = decode_fn or self._cuda_decode
        self._combine = combine_fn or flash_gqa.gqa_combine
        self._gathered = None

    @staticmethod
    def _cuda_decode(q, k, v, scale, kv_layout, partial_out):
        return flash_gqa.gqa_decode(q, k, v, scale=scale, kv_layout=kv_layout, partial_out=partial_out)

    def _buffers(self, B, Hq, device):
        shape = (self.world_size, B, Hq, flash_gqa.PARTIAL_WIDTH)
        if self._gathered is None or tuple(self._gathered.shape) != shape or self._gathered.device != device:
            self._gathered = torch.zeros(shape, dtype=torch.float32, device=device)
        return self._gathered

    def local_partial(self, q, k_local, v_local, scale=None, kv_layout=flash_gqa.KV_BHSD):
        """This rank's packed (O, m, l), written straight into its slot of the gather buffer."""
        B, Hq, _ = q.shape
        gathered = self._buffers(B, Hq, q.device)
        mine = gathered[self.rank]
        s_axis = 1 if kv_layout == flash_gqa.KV_BSHD else 2
        if k_local.shape[s_axis] == 0:
            mine.zero_()
            mine[..., flash_gqa.HEAD_DIM] = float("-inf")
        else:
            self._decode(q, k_local, v_local, scale, kv_layout, mine)
        return mine

    def decode(self, q, k_local, v_local, scale=None, kv_layout=flash_gqa.KV_BHSD):
        """q [B,Hq,D] replicated; k_local/v_local hold this rank's positions.  Returns the full O on every rank."""
        mine = self.local_partial(q, k_local, v_local, scale, kv_layout)
        gathered = self._gathered
        if self.world_size > 1:
            # NCCL gathers in place (this rank's slot already holds its partial); CPU backends get a copy
            src = mine.reshape(-1) if mine.is_cuda else mine.reshape(-1).clone()
            dist.all_gather_into_tensor(gathered.view(-1), src, group=self.group)
        return self._combine(gathered)
