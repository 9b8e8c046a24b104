"""Two-GPU run of the KV-position-sharded decode over NCCL (skipped on a single-GPU machine)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

pytestmark = pytest.mark.gpu
SCALE = float(1.0 / np.sqrt(128.0))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    import oracle_lib as ol
    import cuda_llm_ops_b200 as ops
    from gpu_util import to_bits, to_dev
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        B, S, Hq, Hkv = 1, 5000, 64, 8
        q = ol.randn_bf16((B, Hq, 128), 301)
        k = ol.randn_bf16((B, S, Hkv, 128), 302, std=0.5)
        v = ol.randn_bf16((B, S, Hkv, 128), 303, std=0.5)
        s0, s1 = ops.shard_kv_positions(S, world, rank)
        qd, kd, vd = to_dev(q), to_dev(np.ascontiguousarray(k[:, s0:s1])), to_dev(np.ascontiguousarray(v[:, s0:s1]))
        dec = ops.KVShardedDecoder(exchange="nccl")
        out = dec.decode(qd, kd, vd, kv_layout=ops.KV_BSHD)
        torch.cuda.synchronize()
        # the exchange over peer memory -- fused into the decode kernel, and from a stored partial -- must give
        # the same answer, call after call (gather slots alternate by call parity, flag words carry a growing
        # step number); the last calls check the device status as a caller would
        peer_err, used_peer = 0.0, 1.0
        for kind in ("auto", "peer"):
            dec_p = ops.KVShardedDecoder(exchange=kind)
            for i in range(5):
                out_p = dec_p.decode(qd, kd, vd, kv_layout=ops.KV_BSHD, check=(i == 4))
                torch.cuda.synchronize()
                peer_err = max(peer_err, ol.errors(to_bits(out_p), to_bits(out))[0])
            if dec_p.exchange != ("fused" if kind == "auto" else "peer"):
                used_peer = 0.0
        single = ops.gqa_decode(to_dev(q), to_dev(k), to_dev(v), kv_layout=ops.KV_BSHD)
        torch.cuda.synchronize()
        want = ol.decode(q, k, v, SCALE, 0)
        res = list(ol.errors(to_bits(out), want)) + list(ol.errors(to_bits(out), to_bits(single)))
        rc, _ = ops.device_status()
        np.save(os.path.join(out_dir, "r%d.npy" % rank), np.array(res + [float(rc), peer_err, used_peer]))
    finally:
        dist.destroy_process_group()


def test_two_gpu_position_sharded_decode_matches_oracle_and_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        mx, mean, rel, mx1, mean1, rel1, rc, peer_err, used_peer = np.load(os.path.join(str(tmp_path), "r%d.npy" % r))
        assert rc == 0
        assert peer_err <= 4e-3, peer_err  # same partials merged in another grouping: a bf16 ulp at most
        assert used_peer == 1.0, "rank %d fell back to NCCL although the GPUs can map each other's memory" % r
        assert mx <= 2e-2 and mean <= 2e-3 and rel <= 2e-2, (r, mx, mean, rel)          # vs CPU oracle
        assert mx1 <= 4e-3 and rel1 <= 5e-3, (r, mx1, mean1, rel1)                       # vs the 1-GPU result
