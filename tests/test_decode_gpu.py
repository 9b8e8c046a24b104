"""Parity of the CUDA split-KV decode (through the C ABI) with the CPU oracle and upstream's golden vectors."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import assert_clean_status, to_bits, to_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def _run(q, k, v, layout, scale=SCALE, num_workers=0):
    import cuda_llm_ops_b200 as ops
    out = ops.gqa_decode(to_dev(q), to_dev(k), to_dev(v), scale=scale, kv_layout=layout, num_workers=num_workers)
    torch.cuda.synchronize()
    return to_bits(out)


@pytest.mark.parametrize("name", ["decode_g4", "decode_g16_rag", "decode_g8_tiny", "decode_g1"])
def test_golden_vectors_from_upstream_torch_oracle(golden, name):
    q = golden[name + "/q"][:, :, 0, :]
    got = _run(q, golden[name + "/k"], golden[name + "/v"], layout=1)
    ol.assert_parity(got, golden[name + "/o"][:, :, 0, :], name)
    assert_clean_status()


# (B, S, Hq, Hkv): the CPU-runnable baseline config first, then group sizes / ragged lengths / tiny inputs
CASES = [
    (4, 1024, 32, 8),     # baseline config 1 (group 4)
    (2, 512, 32, 2),      # group 16, the only group upstream's CUDA kernel accepts
    (1, 4096, 16, 2),     # group 8, long enough that every worker gets partial units
    (3, 333, 12, 4),      # group 3, ragged last tile
    (1, 1, 8, 8),         # a single token, group 1
    (2, 63, 40, 2),       # group 20 -> two 16-row blocks per kv head
    (1, 65, 16, 1),       # one token into the second tile
    (5, 200, 8, 1),
    (2, 3000, 64, 2),     # group 32: two 16-row blocks per kv head, every block's share cut between workers
]


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("B,S,Hq,Hkv", CASES)
def test_parity_with_cpu_oracle(B, S, Hq, Hkv, layout):
    q = ol.randn_bf16((B, Hq, 128), 11)
    kshape = (B, S, Hkv, 128) if layout == 0 else (B, Hkv, S, 128)
    k = ol.randn_bf16(kshape, 12)
    v = ol.randn_bf16(kshape, 13)
    want = ol.decode(q, k, v, SCALE, layout)
    got = _run(q, k, v, layout)
    ol.assert_parity(got, want, "B%d S%d Hq%d Hkv%d layout%d" % (B, S, Hq, Hkv, layout))
    assert_clean_status()


@pytest.mark.parametrize("workers", [1, 2, 3, 7, 31, 148, 296, 1000])
def test_result_does_not_depend_on_the_number_of_workers(workers):
    B, S, Hq, Hkv = 2, 3000, 16, 2  # 188 tiles: the largest counts launch more blocks than the GPU has SMs
    q = ol.randn_bf16((B, Hq, 128), 21)
    k = ol.randn_bf16((B, S, Hkv, 128), 22)
    v = ol.randn_bf16((B, S, Hkv, 128), 23)
    want = ol.decode(q, k, v, SCALE, 0)
    got = _run(q, k, v, 0, num_workers=workers)
    ol.assert_parity(got, want, "workers=%d" % workers)
    assert_clean_status()


def test_large_scores_and_other_scale():
    # std 3 inputs make the softmax very peaked; a non-default scale checks the log2 folding
    B, S, Hq, Hkv = 1, 700, 8, 2
    q = ol.randn_bf16((B, Hq, 128), 31, std=3.0)
    k = ol.randn_bf16((B, Hkv, S, 128), 32, std=3.0)
    v = ol.randn_bf16((B, Hkv, S, 128), 33)
    want = ol.decode(q, k, v, 0.05, 1)
    got = _run(q, k, v, 1, scale=0.05)
    ol.assert_parity(got, want, "peaked")


def test_deterministic_across_runs():
    B, S, Hq, Hkv = 3, 2048, 32, 4
    q = ol.randn_bf16((B, Hq, 128), 41)
    k = ol.randn_bf16((B, S, Hkv, 128), 42)
    v = ol.randn_bf16((B, S, Hkv, 128), 43)
    first = _run(q, k, v, 0)
    for _ in range(5):
        assert np.array_equal(_run(q, k, v, 0), first)


def test_partials_of_position_shards_combine_to_the_full_result():
    """The multi-GPU exchange emulated on one device: shard KV by position, gather, LSE-combine."""
    import cuda_llm_ops_b200 as ops
    B, S, Hq, Hkv, shards = 1, 3000, 16, 2, 4
    q = ol.randn_bf16((B, Hq, 128), 51)
    k = ol.randn_bf16((B, Hkv, S, 128), 52, std=0.5)
    v = ol.randn_bf16((B, Hkv, S, 128), 53, std=0.5)
    want = ol.decode(q, k, v, SCALE, 1)
    qd = to_dev(q)
    gathered = torch.zeros((shards, B, Hq, 130), dtype=torch.float32, device="cuda")
    for r in range(shards):
        s0, s1 = ops.shard_kv_positions(S, shards, r)
        ks = to_dev(np.ascontiguousarray(k[:, :, s0:s1]))
        vs = to_dev(np.ascontiguousarray(v[:, :, s0:s1]))
        ops.gqa_decode(qd, ks, vs, scale=SCALE, kv_layout=1, partial_out=gathered[r])
        # each shard's partial agrees with the oracle's partial of the same range
        _, ou, m, l = ol.decode(q, k, v, SCALE, 1, s_begin=s0, s_end=s1, want_partial=True)
        got = gathered[r].cpu().numpy()
        w_got = np.exp(got[..., 128] - m)  # the two maxima may differ by rounding; compare rescaled
        assert np.allclose(got[..., 129] * w_got, l, rtol=2e-2)
        assert np.allclose(got[..., :128] * w_got[..., None], ou, rtol=5e-2, atol=5e-2)
    out = ops.gqa_combine(gathered)
    torch.cuda.synchronize()
    ol.assert_parity(to_bits(out), want, "sharded")
    # and against the oracle's own combine of the GPU partials
    o2, _ = ol.combine(gathered.cpu().numpy())
    ol.assert_parity(to_bits(out), o2, "combine kernel")
    assert_clean_status()


def test_upstream_launcher_mirrors(golden):
    import cuda_llm_ops_b200 as ops
    # Triton-style launcher: [B,H,S,D] tensors, 4-D q
    name = "decode_g4"
    out = ops.launch_decode_flash_gqa_bf16_kernel(to_dev(golden[name + "/q"]), to_dev(golden[name + "/k"]),
                                                  to_dev(golden[name + "/v"]))
    torch.cuda.synchronize()
    ol.assert_parity(to_bits(out), golden[name + "/o"], "triton mirror")
    # C++-style launcher: [B,S,Hkv,D], caller-provided oIntermediate
    B, S, Hq, Hkv = 2, 256, 32, 2
    q = ol.randn_bf16((B, Hq, 128), 61)
    k = ol.randn_bf16((B, S, Hkv, 128), 62)
    v = ol.randn_bf16((B, S, Hkv, 128), 63)
    o = torch.zeros((B, Hq, 128), dtype=torch.bfloat16, device="cuda")
    inter = torch.zeros((B, Hq, 128), dtype=torch.float32, device="cuda")
    ops.LaunchFlashGqaBf16Kernel(to_dev(q), to_dev(k), to_dev(v), SCALE, o, inter, B, S, Hq, Hkv, 128)
    torch.cuda.synchronize()
    ol.assert_parity(to_bits(o), ol.decode(q, k, v, SCALE, 0), "c++ mirror")


def test_cabi_compat_entry_point():
    import ctypes
    from cuda_llm_ops_b200 import _lib
    lib = _lib.load()
    B, S, Hq, Hkv = 2, 300, 16, 1
    q = ol.randn_bf16((B, Hq, 128), 71)
    k = ol.randn_bf16((B, S, Hkv, 128), 72)
    v = ol.randn_bf16((B, S, Hkv, 128), 73)
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    o = torch.zeros((B, Hq, 128), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    rc = lib.cllo_gqa_decode_bf16_compat(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), SCALE, o.data_ptr(), None,
                                         B, S, Hq, Hkv, 128)
    assert rc == 0
    torch.cuda.synchronize()
    ol.assert_parity(to_bits(o), ol.decode(q, k, v, SCALE, 0), "compat")
    assert lib.cllo_shutdown() == 0
    # error codes: too-small workspace, bad head_dim
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    rc = lib.cllo_gqa_decode_bf16(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), SCALE, o.data_ptr(), ws.data_ptr(), 256,
                                  B, S, Hq, Hkv, 128, 0, 0, None, None)
    assert rc == _lib.E_WORKSPACE
    rc = lib.cllo_gqa_decode_bf16(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), SCALE, o.data_ptr(), ws.data_ptr(), 256,
                                  B, S, Hq, Hkv, 64, 0, 0, None, None)
    assert rc == _lib.E_UNSUPPORTED


def test_headline_shape_sampled_units_and_split_invariance():
    """Baseline config 2 (B=60, S=4096, Hq=128, Hkv=8) at full size: the oracle checks sampled (batch, kv head)
    units exactly; a second run with a different worker count must agree everywhere (size-independent property)."""
    import cuda_llm_ops_b200 as ops
    B, S, Hq, Hkv = 60, 4096, 128, 8
    g = torch.Generator(device="cuda").manual_seed(1234)
    q = torch.randn((B, Hq, 128), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((B, S, Hkv, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((B, S, Hkv, 128), generator=g, device="cuda").to(torch.bfloat16)
    out = ops.gqa_decode(q, k, v, kv_layout=0)
    out2 = ops.gqa_decode(q, k, v, kv_layout=0, num_workers=111)
    torch.cuda.synchronize()
    a, b2 = to_bits(out), to_bits(out2)
    mx, mean, rel = ol.errors(a, b2)
    assert mx <= 4e-3 and rel <= 5e-3, (mx, mean, rel)
    for b, h in [(0, 0), (17, 3), (59, 7), (33, 5)]:
        qs = to_bits(q[b:b + 1, h * 16:(h + 1) * 16])
        ks = to_bits(k[b:b + 1, :, h:h + 1])
        vs = to_bits(v[b:b + 1, :, h:h + 1])
        want = ol.decode(qs, ks, vs, SCALE, 0)
        ol.assert_parity(a[b:b + 1, h * 16:(h + 1) * 16], want, "unit (%d,%d)" % (b, h))
    assert_clean_status()


def test_long_context_shape_at_full_size():
    """Baseline config 4 (one sequence, S=1,048,576, Hq=64, Hkv=8, inputs 0.5*N(0,1)) at full size: K and V hold
    2^30 elements each.  The whole output is compared with the oracle, and the partials of two unequal position
    ranges must combine to the same result."""
    import cuda_llm_ops_b200 as ops
    S, Hq, Hkv = 1 << 20, 64, 8
    g = torch.Generator(device="cuda").manual_seed(77)
    q = (0.5 * torch.randn((1, Hq, 128), generator=g, device="cuda")).to(torch.bfloat16)
    k = torch.empty((1, Hkv, S, 128), dtype=torch.bfloat16, device="cuda")
    v = torch.empty((1, Hkv, S, 128), dtype=torch.bfloat16, device="cuda")
    for h in range(Hkv):
        k[0, h] = (0.5 * torch.randn((S, 128), generator=g, device="cuda")).to(torch.bfloat16)
        v[0, h] = (0.5 * torch.randn((S, 128), generator=g, device="cuda")).to(torch.bfloat16)
    out = ops.gqa_decode(q, k, v, scale=SCALE, kv_layout=1)
    cut = 700_001
    parts = torch.zeros((2, 1, Hq, 130), dtype=torch.float32, device="cuda")
    ops.gqa_decode(q, k[:, :, :cut].contiguous(), v[:, :, :cut].contiguous(), scale=SCALE, kv_layout=1,
                   partial_out=parts[0])
    ops.gqa_decode(q, k[:, :, cut:].contiguous(), v[:, :, cut:].contiguous(), scale=SCALE, kv_layout=1,
                   partial_out=parts[1])
    merged = ops.gqa_combine(parts)
    torch.cuda.synchronize()
    assert_clean_status()
    got = to_bits(out)
    want = ol.decode(to_bits(q), to_bits(k), to_bits(v), SCALE, 1)
    ol.assert_parity(got, want, "long context")
    ol.assert_parity(to_bits(merged), want, "long context, two position ranges")


def _exchange_buffers(world, B, Hq):
    """One rank's gather slots + flag words (zeroed), as (tensor, gather pointer, flag pointer)."""
    from cuda_llm_ops_b200 import _lib
    lib = _lib.load()
    gb, fb = int(lib.cllo_gqa_shard_gather_bytes(world, B, Hq, 128)), int(lib.cllo_gqa_shard_flag_bytes(world))
    assert gb > 0 and fb > 0
    buf = torch.zeros((gb + fb) // 4, dtype=torch.float32, device="cuda")
    return buf, buf.data_ptr(), buf.data_ptr() + gb


def test_exchange_kernels_with_a_world_of_one():
    """Both forms of the peer exchange with world = 1 (their own buffers as the only peer): the fused decode and
    the exchange from a stored partial must equal the plain decode, call after call (epoch 0 = the kernels count
    their launches on the device)."""
    import ctypes
    import cuda_llm_ops_b200 as ops
    from cuda_llm_ops_b200 import _lib
    B, S, Hq, Hkv = 2, 900, 16, 2
    q = ol.randn_bf16((B, Hq, 128), 81)
    k = ol.randn_bf16((B, Hkv, S, 128), 82)
    v = ol.randn_bf16((B, Hkv, S, 128), 83)
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    part = torch.zeros((B, Hq, 130), dtype=torch.float32, device="cuda")
    ops.gqa_decode(qd, kd, vd, scale=SCALE, kv_layout=1, partial_out=part)
    buf, g_ptr, f_ptr = _exchange_buffers(1, B, Hq)
    arr = ctypes.c_void_p * 1
    gather, flags = arr(g_ptr), arr(f_ptr)
    want = ol.decode(q, k, v, SCALE, 1)
    for step in range(4):
        out = torch.zeros((B, Hq, 128), dtype=torch.bfloat16, device="cuda")
        if step % 2 == 0:
            rc = _lib.load().cllo_gqa_exchange_combine_bf16(part.data_ptr(), gather, flags, 0, 1, 0, out.data_ptr(),
                                                            B, Hq, Hkv, 128, None)
            assert rc == 0
        else:
            ops.gqa_decode_sharded(qd, kd, vd, gather, flags, 0, 1, epoch=0, scale=SCALE, kv_layout=1, out=out)
        torch.cuda.synchronize()
        ol.assert_parity(to_bits(out), want, "exchange world=1, step %d" % step)
    assert_clean_status()


@pytest.mark.parametrize("B,S,Hq,Hkv,workers", [(1, 6000, 64, 8, 0), (2, 1500, 40, 2, 37)])
def test_two_rank_exchange_on_one_gpu_and_the_wait_that_runs_out(B, S, Hq, Hkv, workers):
    """The two-rank protocol with both ranks' buffers on this GPU, one rank at a time (kernels that wait for one
    another must not share a GPU).  Rank 1 goes first: it delivers its rows and then waits for a rank 0 that is
    not there -- with the wait limit set to a few milliseconds the wait runs out, the kernel returns on its own,
    the output rows are NaN and the device status names the exchange wait.  Then rank 0 runs the fused decode
    (it finds rank 1's rows waiting), and rank 1 repeats its step (it now finds rank 0's): both must give the
    unsharded result."""
    import ctypes
    import cuda_llm_ops_b200 as ops
    from cuda_llm_ops_b200 import _lib
    lib = _lib.load()
    q = ol.randn_bf16((B, Hq, 128), 91)
    k = ol.randn_bf16((B, S, Hkv, 128), 92, std=0.5)
    v = ol.randn_bf16((B, S, Hkv, 128), 93, std=0.5)
    want = ol.decode(q, k, v, SCALE, 0)
    qd = to_dev(q)
    cut = ops.shard_kv_positions(S, 2, 0)[1]
    k0, v0 = to_dev(np.ascontiguousarray(k[:, :cut])), to_dev(np.ascontiguousarray(v[:, :cut]))
    k1, v1 = to_dev(np.ascontiguousarray(k[:, cut:])), to_dev(np.ascontiguousarray(v[:, cut:]))
    part1 = torch.zeros((B, Hq, 130), dtype=torch.float32, device="cuda")
    ops.gqa_decode(qd, k1, v1, scale=SCALE, kv_layout=0, partial_out=part1)
    buf_a, ga, fa = _exchange_buffers(2, B, Hq)  # rank 0's
    buf_b, gb, fb = _exchange_buffers(2, B, Hq)  # rank 1's
    arr = ctypes.c_void_p * 2
    gather, flags = arr(ga, gb), arr(fa, fb)
    out0 = torch.zeros((B, Hq, 128), dtype=torch.bfloat16, device="cuda")
    out1 = torch.zeros((B, Hq, 128), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    assert_clean_status()
    ops.set_exchange_wait_limit(4_000_000)  # about 2 ms
    try:
        rc = lib.cllo_gqa_exchange_combine_bf16(part1.data_ptr(), gather, flags, 1, 2, 1, out1.data_ptr(),
                                                B, Hq, Hkv, 128, None)
        assert rc == 0  # the launch itself succeeds; the time-out is a device-side status
        rc, detail = ops.device_status()
        assert rc == _lib.E_DEVICE_TIMEOUT and detail[2] == 8, (rc, detail)  # site 8: the exchange flag wait
        assert torch.isnan(out1.float()).all()
        assert ops.device_status()[0] == 0  # reading the status cleared it
    finally:
        ops.set_exchange_wait_limit(0)
    ops.gqa_decode_sharded(qd, k0, v0, gather, flags, 0, 2, epoch=1, scale=SCALE, kv_layout=0, out=out0,
                           num_workers=workers)
    rc = lib.cllo_gqa_exchange_combine_bf16(part1.data_ptr(), gather, flags, 1, 2, 1, out1.data_ptr(),
                                            B, Hq, Hkv, 128, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert_clean_status()
    ol.assert_parity(to_bits(out0), want, "rank 0, fused")
    ol.assert_parity(to_bits(out1), want, "rank 1, exchange from memory")
    assert np.array_equal(to_bits(out0), to_bits(out1))  # same rows merged in the same order on both ranks
    # an ordinary decode still works after the time-out
    ol.assert_parity(_run(q, k, v, 0), want, "plain decode afterwards")
