"""World-size-2 run of the KV-position-sharded decode on CPU ranks (gloo).

The product's exchange code (partition, in-place gather layout, combine call) is what runs; the two device
kernels are replaced by the CPU oracle, injected through KVShardedDecoder's decode_fn / combine_fn hooks.
"""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

SCALE = float(1.0 / np.sqrt(128.0))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _worker(rank, world, port, S, result_dir):
    import oracle_lib as ol
    import cuda_llm_ops_b200 as ops
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hq, Hkv = 2, 8, 2
        q = ol.randn_bf16((B, Hq, 128), 7)
        k = ol.randn_bf16((B, Hkv, S, 128), 8, std=0.5)
        v = ol.randn_bf16((B, Hkv, S, 128), 9, std=0.5)
        s0, s1 = ops.shard_kv_positions(S, world, rank)

        def decode_fn(qt, kt, vt, scale, kv_layout, partial_out):
            _, ou, m, l = ol.decode(_bits(qt), _bits(kt), _bits(vt), SCALE if scale is None else scale, kv_layout,
                                    want_partial=True)
            partial_out.copy_(torch.from_numpy(ol.pack_partial(ou, m, l)))
            return partial_out

        def combine_fn(gathered):
            o, _ = ol.combine(gathered.numpy())
            return torch.from_numpy(o.view(np.int16)).view(torch.bfloat16)

        to_t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)  # noqa: E731
        dec = ops.KVShardedDecoder(decode_fn=decode_fn, combine_fn=combine_fn)
        assert dec.world_size == world and dec.rank == rank
        out = dec.decode(to_t(q), to_t(k[:, :, s0:s1]), to_t(v[:, :, s0:s1]), kv_layout=ops.KV_BHSD)
        want = ol.decode(q, k, v, SCALE, 1)
        mx, mean, rel = ol.errors(_bits(out), want)
        # every rank holds every rank's partial after the gather
        g = dec._gathered.numpy()
        others_filled = all(np.isfinite(g[r, ..., 128]).all() or ops.shard_kv_positions(S, world, r)[0] == S
                            for r in range(world))
        np.save(os.path.join(result_dir, "r%d.npy" % rank), np.array([mx, mean, rel, float(others_filled)]))
    finally:
        dist.destroy_process_group()


def _run(world, S, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, S, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        mx, mean, rel, filled = np.load(os.path.join(str(tmp_path), "r%d.npy" % r))
        assert filled == 1.0
        assert mx <= 4e-3 and rel <= 5e-3, (r, mx, mean, rel)


def test_two_ranks_position_sharded_decode_equals_unsharded(tmp_path):
    _run(2, 700, tmp_path)


def test_a_rank_with_an_empty_shard_is_ignored(tmp_path):
    # 40 tokens = one 64-token tile: rank 1 owns nothing and contributes (O=0, m=-inf, l=0)
    _run(2, 40, tmp_path)
