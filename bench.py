#!/usr/bin/env python
"""Benchmark of the flash-GQA path.  Prints ONE JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads (synthetic, seeded; shapes are the baseline configurations of this path):
    all             (default) the headline decode_b60 line, and inside it -- under config.also_measured and
                    roofline.others -- short runs of the other baseline configurations: prefill_nc (with its own
                    end-to-end leg and CPU baseline), prefill_causal, decode_long, and on several GPUs decode_b60_strong
                    (ONE batch of 60 split across the ranks) plus a parity check of the position-sharded decode
                    against the single-GPU result and the CPU oracle
    decode_b60      GQA decode, B=60 per GPU, S=4096, Hq=128, Hkv=8, D=128, K/V [B,S,Hkv,D]   (headline)
    decode_b60_strong  the same shape as ONE batch of 60 sequences split 60/30/15/8,7 across the ranks (strong scaling)
    decode_step_rope   decode_b60 with the rotary embedding of the new token and the cache append inside the kernel
    decode_long     one sequence, S=1,048,576, Hq=64, Hkv=8, KV sharded by position across GPUs
                    (all-gather of per-GPU partials + LSE combine; strong scaling)
    prefill_nc      prefill forward, non-causal, B=1, S=4096, Hq=16, Hkv=1
    prefill_causal  prefill forward, causal, B=8 in total (strong scaling), S=16384, Hq=64, Hkv=8; batch-sharded
    rope            rotary position embedding, upstream's shape
    mla             MLA-shaped forward (head_dim_qk 192, head_dim_v 128), causal, upstream's shape
    sgqa            sparse-index GQA forward, upstream's shape (S=32768, 16 query heads on one kv head, lists of 512)
    backward        GQA attention backward (dQ, dK, dV), causal, upstream's shape
    swa             sliding-window forward with sink (mask variant of the prefill kernel), upstream's shape
    prefill_chunk   64 query tokens against 8192 cached keys (the one-tile kernel, heads of a group sharing a tile)

A step is one pass of the hot path over one batch.  `value` is whole-job throughput with inputs
resident in HBM; `e2e` is the same metric through the package's public launcher with HOST buffers
(pinned), host<->device copies inside the timed region.  `--impl reference` times upstream's own CPU
implementation of the decode path on this machine's host cores instead.
"""
import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from one ncu capture each
# (decode: 4 x a B=15 capture of the same kernel, traffic grows with the K/V bytes; prefill: a capture of the
# workload itself).  A capture describes the kernel as it was when it was taken: "captured_at" says which.
NCU_TRAFFIC_BYTES = {"decode_b60": 4 * 256_469_504, "prefill_nc": 19_081_728}
NCU_TRAFFIC_CAPTURED_AT = {"decode_b60": "split-KV kernel with the merge inside, 120 workers (B=15 capture x 4)",
                           "prefill_nc": "two-tile tcgen05 kernel, region-C version"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
            "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t_begin, t_end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        for ts, line in self.rows:
            if ts < t_begin - 0.02 or ts > t_end + 0.06:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
def decode_bytes(B, S, Hq, Hkv, D=128):
    """Algorithmic bytes of one decode pass: K and V read once, Q read, O written (bf16)."""
    return 2 * (B * S * Hkv * D) * 2 + 2 * (B * Hq * D) * 2


def prefill_flops(B, Hq, Sq, Skv, D=128, causal=False):
    f = 4.0 * B * Hq * Sq * Skv * D
    return f / 2 if causal else f


def measure(args, wl, rank, world, local_rank, steps, warmup, light=False):
    """Times one workload; returns its JSON line as a dict on rank 0 and None on the other ranks.

    ``light`` (the extra workloads of the default run): no clock-sampling repeats, and an end-to-end leg and a CPU
    baseline only where the line is asked to carry them (prefill_nc).
    """
    import torch
    import torch.distributed as dist
    import cuda_llm_ops_b200 as ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks = measured_peaks()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def randn_bf16(shape, std=1.0, g=None):
        # generated in slices to keep the fp32 temporary small
        g = g or gen
        out = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        flat = out.view(-1)
        step = 1 << 26
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = (torch.randn(n, generator=g, device=dev) * std).to(torch.bfloat16)
        return out

    def seeded(seed):
        return torch.Generator(device=dev).manual_seed(seed)

    extra = {}
    if wl == "decode_b60_strong":
        # baseline configuration 2 as stated: ONE batch of 60 sequences, split across the ranks (60 / 30 / 15 / 8,7)
        S, Hq, Hkv = 4096, 128, 8
        b0, b1 = ops.shard_batch(60, world, rank)
        B = b1 - b0
        layout = ops.KV_BSHD
        q, k, v = randn_bf16((B, Hq, 128)), randn_bf16((B, S, Hkv, 128)), randn_bf16((B, S, Hkv, 128))
        out = torch.empty_like(q)
        step_fn = lambda: ops.gqa_decode(q, k, v, kv_layout=layout, out=out)  # noqa: E731
        units_per_rank = decode_bytes(B, S, Hq, Hkv)
        total_units = decode_bytes(60, S, Hq, Hkv)
        metric, unit, scale_div, bound = "gqa_decode_achieved_hbm_tbps", "TB/s", 1e12, "hbm"
        launches_per_step = 1
        scaling = "strong"
        config = {"workload": "decode_b60_strong: GQA decode, ONE batch of 60 sequences split across %d GPU(s) "
                              "(this rank: %d), S=4096, Hq=128, Hkv=8, D=128, K/V [B,S,Hkv,D], N(0,1) seeded" % (world, B),
                  "global_batch": 60, "kv_seq_len": S, "sharding": "batch (no collective)",
                  "l2": "a rank's share at 8 GPUs (118-134 MB) is about the size of the 126 MB L2: the line says what "
                        "a decode step of this batch costs, not an HBM figure"}
        host_in = [q, k, v]
    elif wl == "decode_step_rope":
        # a whole decoder step at the headline shape: rotary embedding of the new token's Q and K, cache append, attention
        B, S, Hq, Hkv = (args.batch or 60), 4096, 128, 8
        layout = ops.KV_BSHD
        q, k, v = randn_bf16((B, Hq, 128)), randn_bf16((B, S, Hkv, 128)), randn_bf16((B, S, Hkv, 128))
        k_new, v_new = randn_bf16((B, Hkv, 128)), randn_bf16((B, Hkv, 128))
        out = torch.empty_like(q)
        step_fn = lambda: ops.gqa_decode_rope_append(q, k_new, v_new, k, v, S, kv_layout=layout, out=out)  # noqa: E731
        units_per_rank = decode_bytes(B, S, Hq, Hkv) + 4 * (B * Hkv * 128) * 2  # + new K/V read and appended
        total_units = units_per_rank * world
        metric, unit, scale_div, bound = "gqa_decode_achieved_hbm_tbps", "TB/s", 1e12, "hbm"
        launches_per_step = 1
        scaling = "weak"
        config = {"workload": "decode_step_rope: rotary embedding of the new token + cache append + GQA decode in one "
                              "kernel, B=%d per GPU, S=4096, Hq=128, Hkv=8, D=128, K/V [B,S,Hkv,D]" % B,
                  "global_batch": B * world, "kv_seq_len": S, "sharding": "batch (no collective)",
                  "l2": "inputs exceed the 126 MB L2; no flush needed"}
        host_in = [q, k, v]
    elif wl == "decode_b60":
        B, S, Hq, Hkv = (args.batch or 60), 4096, 128, 8
        layout = ops.KV_BSHD if args.layout == "bshd" else ops.KV_BHSD
        kshape = (B, S, Hkv, 128) if layout == ops.KV_BSHD else (B, Hkv, S, 128)
        q, k, v = randn_bf16((B, Hq, 128)), randn_bf16(kshape), randn_bf16(kshape)
        out = torch.empty_like(q)
        step_fn = lambda: ops.gqa_decode(q, k, v, kv_layout=layout, out=out)  # noqa: E731
        units_per_rank = decode_bytes(B, S, Hq, Hkv)
        total_units = units_per_rank * world
        metric, unit, scale_div, bound = "gqa_decode_achieved_hbm_tbps", "TB/s", 1e12, "hbm"
        launches_per_step = 1  # the decode kernel (the merge runs inside it; a memset node zeroes its counters)
        scaling = "weak"
        config = {"workload": "decode_b60: GQA decode B=%d per GPU, S=4096, Hq=128, Hkv=8, D=128, one query token, "
                              "K/V %s, N(0,1) seeded" % (B, "[B,S,Hkv,D]" if layout == ops.KV_BSHD else "[B,Hkv,S,D]"),
                  "global_batch": B * world, "kv_seq_len": S, "sharding": "batch (no collective)",
                  "l2": "inputs (%.2f GB per GPU) exceed the 126 MB L2; no flush needed" % (units_per_rank / 1e9)}
        host_in = [q, k, v]
    elif wl == "decode_long":
        S_total, Hq, Hkv = (args.kv_len or (1 << 20)), 64, 8
        s0, s1 = ops.shard_kv_positions(S_total, world, rank)
        # every tensor has its own seed (K and V per shard), so that rank 0 can rebuild the whole sequence for the
        # single-GPU comparison below
        q = randn_bf16((1, Hq, 128), 0.5, seeded(4000))
        k = randn_bf16((1, s1 - s0, Hkv, 128), 0.5, seeded(5000 + 2 * rank))
        v = randn_bf16((1, s1 - s0, Hkv, 128), 0.5, seeded(5001 + 2 * rank))
        dec = ops.KVShardedDecoder(exchange=args.exchange) if world > 1 else None
        if world > 1:
            out = torch.empty_like(q)
            step_fn = lambda: dec.decode(q, k, v, kv_layout=ops.KV_BSHD, out=out)  # noqa: E731
            launches_per_step = 1
        else:
            out = torch.empty_like(q)
            step_fn = lambda: ops.gqa_decode(q, k, v, kv_layout=ops.KV_BSHD, out=out)  # noqa: E731
            launches_per_step = 1
        total_units = decode_bytes(1, S_total, Hq, Hkv)
        units_per_rank = decode_bytes(1, s1 - s0, Hq, Hkv)
        metric, unit, scale_div, bound = "gqa_decode_achieved_hbm_tbps", "TB/s", 1e12, "hbm"
        scaling = "strong"
        config = {"workload": "decode_long: one sequence, S=%d, Hq=64, Hkv=8, D=128, K/V [1,S,Hkv,D] 0.5*N(0,1)" % S_total,
                  "global_batch": 1, "kv_seq_len": S_total,
                  "sharding": "KV positions; per-GPU (O,m,l) partials exchanged over peer memory (or NCCL all-gather) "
                              "+ LSE combine" if world > 1 else "none",
                  "l2": "inputs exceed L2"}
        host_in = [q, k, v]
    elif wl == "swa":
        # upstream's sliding-window benchmark shape (README: 280 us / 61 TFLOPS on an RTX 5080 Laptop)
        B, S, Hq, Hkv, window = 1, 4096, 16, 1, 512
        q, k, v = randn_bf16((B, Hq, S, 128)), randn_bf16((B, Hkv, S, 128)), randn_bf16((B, Hkv, S, 128))
        sink = torch.rand(Hq, device=dev, generator=gen) + 0.5
        out = torch.empty_like(q)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        inner = lambda: ops.launch_flash_swa_forward_bf16_kernel(q, k, v, out=out, lse=lse, window_size=window,  # noqa: E731
                                                                 sink_value=sink)
        step_fn = lambda: (flush.zero_(), inner())  # noqa: E731
        # upstream's own FLOP convention: 2 * Sq * window * (Dqk + Dv) per head (test_flash_swa_kernel.py:318-337)
        units_per_rank = 2.0 * S * window * 256 * B * Hq
        total_units = units_per_rank * world
        metric, unit, scale_div, bound = "swa_prefill_tflops", "TFLOP/s", 1e12, "tensor"
        launches_per_step = 1
        scaling = "weak"
        config = {"workload": "swa: sliding-window forward with sink, B=1, S=4096, Hq=16, Hkv=1, D=128, window=512",
                  "global_batch": B * world, "seq_len": S, "sharding": "batch (no collective)",
                  "l2": "256 MB buffer rewritten between iterations (outside the per-step event brackets)"}
        host_in = [q, k, v]
    elif wl == "rope":
        # upstream's RoPE benchmark shape (README: 510 us / 0.48 "TB/s" on an RTX 5080 Laptop)
        B, S, hidden = 1, 512 * 1024, 128
        x = randn_bf16((B, S, hidden))
        out = torch.empty_like(x)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        inner = lambda: ops.LaunchRopeBf16Kernel(x, out, B, S, hidden)  # noqa: E731
        step_fn = lambda: (flush.zero_(), inner())  # noqa: E731
        units_per_rank = 2.0 * B * S * hidden * 2  # read + write, bf16 (same terms as upstream's test_rope.cu:165)
        total_units = units_per_rank * world
        metric, unit, scale_div, bound = "rope_achieved_hbm_tbps", "TB/s", 1e12, "hbm"
        launches_per_step = 1
        scaling = "weak"
        config = {"workload": "rope: rotary embedding B=1, S=524288, hidden=128, bf16",
                  "global_batch": B * world, "seq_len": S, "sharding": "batch (no collective)",
                  "l2": "256 MB buffer rewritten between iterations (outside the per-step event brackets)"}
        host_in = [x]
    elif wl == "mla":
        # upstream's MLA forward benchmark shape (README: 1440 us / 59.65 TFLOPS on an RTX 5080 Laptop), causal
        B, S, Hq, Hkv = 1, 4096, 16, 16
        q, k, v = randn_bf16((B, Hq, S, 192)), randn_bf16((B, Hkv, S, 192)), randn_bf16((B, Hkv, S, 128))
        out = torch.empty((B, Hq, S, 128), dtype=torch.bfloat16, device=dev)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        inner = lambda: ops.launch_flash_mla_forward_bf16_kernel(q, k, v, out=out, lse=lse, causal=True)  # noqa: E731
        step_fn = lambda: (flush.zero_(), inner())  # noqa: E731
        # upstream's FLOP convention: 2 * Sq * Skv * (head_dim_qk + head_dim_v) / 2 per head (test_flash_mla_kernel.py:282-302)
        units_per_rank = float(B * Hq) * (2 * S * S * (192 + 128) // 2)
        total_units = units_per_rank * world
        metric, unit, scale_div, bound = "mla_prefill_tflops", "TFLOP/s", 1e12, "tensor"
        launches_per_step = 1
        scaling = "weak"
        config = {"workload": "mla: MLA-shaped forward, causal, B=1, S=4096, Hq=16, Hkv=16, head_dim_qk=192, head_dim_v=128",
                  "global_batch": B * world, "seq_len": S, "sharding": "batch (no collective)",
                  "l2": "256 MB buffer rewritten between iterations (outside the per-step event brackets)"}
        host_in = [q, k, v]
    elif wl == "prefill_chunk":
        # a chunk of 64 new query tokens against 8192 cached ones (chunked prefill / speculative decoding): the
        # one-tile kernel, two heads of a group sharing each 128-row tile
        B, Sq, Skv, Hq, Hkv = (args.batch or 8), 64, 8192, 32, 4
        q, k, v = randn_bf16((B, Hq, Sq, 128)), randn_bf16((B, Hkv, Skv, 128)), randn_bf16((B, Hkv, Skv, 128))
        out = torch.empty_like(q)
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        inner = lambda: ops.launch_flash_gqa_forward_bf16_kernel(q, k, v, out=out, lse=lse, causal=False)  # noqa: E731
        step_fn = lambda: (flush.zero_(), inner())  # noqa: E731
        units_per_rank = 4.0 * B * Hq * Sq * Skv * 128
        total_units = units_per_rank * world
        metric, unit, scale_div, bound = "gqa_prefill_tflops", "TFLOP/s", 1e12, "tensor"
        launches_per_step = 1
        scaling = "weak"
        config = {"workload": "prefill_chunk: GQA forward, non-causal, 64 query tokens against 8192 keys, B=8 per GPU, "
                              "Hq=32, Hkv=4, D=128",
                  "global_batch": B * world, "seq_len": Skv, "sharding": "batch (no collective)",
                  "l2": "256 MB buffer rewritten between iterations (outside the per-step event brackets)"}
        host_in = [q, k, v]
    elif wl == "sgqa":
        # upstream's sparse-index GQA benchmark shape (README: 3690 us / 37.2 TFLOPS on an RTX 5080 Laptop).  Lists as
        # in upstream's test: the 16 most recent tokens, then uniformly drawn earlier ones, padded with -1 while the
        # prefix is shorter than the list (drawn with replacement here; upstream draws without).
        B, S, Hq, Hkv, n_sparse = 1, 32768, 16, 1, 512
        q, k, v = randn_bf16((B, Hq, S, 128)), randn_bf16((B, Hkv, S, 128)), randn_bf16((B, Hkv, S, 128))
        pos = torch.arange(S, device=dev, dtype=torch.int32).view(1, 1, S, 1)
        gen = torch.Generator(device=dev).manual_seed(4321 + rank)
        idx = (torch.rand((B, Hkv, S, n_sparse), generator=gen, device=dev) * (pos - 15).clamp(min=1)).to(torch.int32)
        slot = torch.arange(n_sparse, device=dev, dtype=torch.int32).view(1, 1, 1, n_sparse)
        idx = torch.where(slot < 16, pos - slot, idx)                     # the recent window
        idx = torch.where((slot <= pos) & (idx >= 0), idx, torch.full_like(idx, -1)).contiguous()
        out = torch.empty_like(q)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        inner = lambda: ops.launch_flash_sgqa_forward_bf16_kernel(q, k, v, idx, n_sparse, out=out, lse=lse)  # noqa: E731
        step_fn = lambda: (flush.zero_(), inner())  # noqa: E731
        # upstream's FLOP convention: 4 * heads * tokens * list length * head_dim (test_flash_sgqa_kernel.py)
        units_per_rank = 4.0 * B * Hq * S * n_sparse * 128
        total_units = units_per_rank * world
        metric, unit, scale_div, bound = "sgqa_prefill_tflops", "TFLOP/s", 1e12, "tensor"
        launches_per_step = 1
        scaling = "weak"
        config = {"workload": "sgqa: sparse-index GQA forward, causal, B=1, S=32768, Hq=16, Hkv=1, D=128, "
                              "512 list entries per token (16 recent + uniform earlier ones)",
                  "global_batch": B * world, "seq_len": S, "sharding": "batch (no collective)",
                  "l2": "256 MB buffer rewritten between iterations (outside the per-step event brackets)"}
        host_in = [q, k, v, idx]
    elif wl == "backward":
        # upstream's backward benchmark shape (README: 3100 us / 55 TFLOPS on an RTX 5080 Laptop), causal
        B, S, Hq, Hkv = 1, 4096, 16, 1
        q, k, v = randn_bf16((B, Hq, S, 128)), randn_bf16((B, Hkv, S, 128)), randn_bf16((B, Hkv, S, 128))
        grad_o = randn_bf16((B, Hq, S, 128))
        out, lse = ops.launch_flash_gqa_forward_bf16_kernel(q, k, v, causal=True)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        inner = lambda: ops.launch_flash_gqa_backward_bf16_kernel(q, k, v, out, lse, grad_o, causal=True)  # noqa: E731
        step_fn = lambda: (flush.zero_(), inner())  # noqa: E731
        # upstream's own FLOP convention: 5 products, halved for causality (test_flash_gqa_kernel.py:362)
        units_per_rank = float(B * Hq) * (2 * S * S * (3 * 128 + 2 * 128) // 2)
        total_units = units_per_rank * world
        metric, unit, scale_div, bound = "gqa_backward_tflops", "TFLOP/s", 1e12, "tensor"
        launches_per_step = 3
        scaling = "weak"
        config = {"workload": "backward: GQA attention backward, causal, B=1, S=4096, Hq=16, Hkv=1, D=128",
                  "global_batch": B * world, "seq_len": S, "sharding": "batch (no collective)",
                  "l2": "256 MB buffer rewritten between iterations (outside the per-step event brackets)"}
        host_in = [q, k, v]
    elif wl in ("prefill_nc", "prefill_causal"):
        causal = wl == "prefill_causal"
        if causal:
            B, S, Hq, Hkv = max(1, 8 // world), 16384, 64, 8
            scaling = "strong"
        else:
            B, S, Hq, Hkv = 1, 4096, 16, 1
            scaling = "weak"
        q, k, v = randn_bf16((B, Hq, S, 128)), randn_bf16((B, Hkv, S, 128)), randn_bf16((B, Hkv, S, 128))
        out = torch.empty_like(q)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=dev)
        step_fn = lambda: ops.launch_flash_gqa_forward_bf16_kernel(q, k, v, out=out, lse=lse, causal=causal)  # noqa: E731
        units_per_rank = prefill_flops(B, Hq, S, S, causal=causal)
        total_units = units_per_rank * world
        metric, unit, scale_div, bound = "gqa_prefill_tflops", "TFLOP/s", 1e12, "tensor"
        launches_per_step = 1
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if not causal else None
        if flush is not None:
            inner = step_fn
            step_fn = lambda: (flush.zero_(), inner())  # noqa: E731
        config = {"workload": "%s: GQA prefill forward %s, B=%d per GPU, S=%d, Hq=%d, Hkv=%d, D=128, [B,H,S,D], N(0,1) seeded"
                              % (wl, "causal" if causal else "non-causal", B, S, Hq, Hkv),
                  "global_batch": B * world, "seq_len": S, "sharding": "batch (no collective)",
                  "l2": "256 MB buffer rewritten between iterations (its time is subtracted; see kernel_ms)"
                        if flush is not None else "inputs exceed L2"}
        host_in = [q, k, v]
    else:
        raise SystemExit("unknown workload " + wl)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        step_fn()
    barrier()
    if wl == "decode_long" and world > 1 and dec.exchange == "peer" and not args.no_graph:
        # the two kernels of a step (decode, exchange) replayed from a CUDA graph: at ~100 us per step on 8 GPUs,
        # host launch jitter between the ranks otherwise shows up as waiting in the exchange.  (The fused form is
        # one kernel per step and is launched directly: measured 2 us faster than replaying a one-node graph.)
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                step_fn()
        torch.cuda.current_stream().wait_stream(side)
        step_fn = graph.replay
        config["launch"] = "CUDA graph replay"
        for _ in range(3):
            step_fn()
        barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    # device time on the launching stream (torch's current stream is the one the C ABI receives)
    barrier()
    t_begin = time.time()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    if wl in ("prefill_nc", "swa", "backward", "rope", "sgqa", "mla", "prefill_chunk"):
        # the L2 flush sits between iterations, so each step gets its own pair of events
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            flush.zero_()
            starts[i].record()
            inner()
            ends[i].record()
        barrier()
        per_step = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        total_ms = sum(per_step)
    else:
        t0.record()
        for i in range(steps):
            step_fn()
        t1.record()
        barrier()
        total_ms = t0.elapsed_time(t1)
        per_step = [total_ms / steps]
    t_end = time.time()
    tt = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    total_ms = float(tt.item())
    # keep the GPUs busy with the same step a little longer so that the clock samples see load.  Every rank
    # runs the same number of repeats (the step may contain a collective), derived from the reduced time.
    if total_ms < 600.0 and not args.profile and not light:
        reps = int(min(20000, 600.0 / max(total_ms / steps, 1e-3)))
        for _ in range(reps):
            step_fn()
        barrier()
        t_end = time.time()
        extra["clock_sampling"] = "timed region + %d untimed repeats of the same step" % reps
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    if wl == "prefill_nc" and not args.profile:
        # The same kernel with cold inputs but without a flush: eight input sets (272 MB, more than the L2) used in
        # rotation, steps back to back under one pair of events.  Reported beside the flushed figure, not instead.
        sets = [(randn_bf16((B, Hq, S, 128)), randn_bf16((B, Hkv, S, 128)), randn_bf16((B, Hkv, S, 128)),
                 torch.empty_like(q)) for _ in range(8)]
        rot = lambda i: ops.launch_flash_gqa_forward_bf16_kernel(sets[i % 8][0], sets[i % 8][1], sets[i % 8][2],  # noqa: E731
                                                                 out=sets[i % 8][3], lse=lse, causal=False)
        for i in range(8):
            rot(i)
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for i in range(32):
            rot(i)
        r1.record()
        barrier()
        rot_ms = r0.elapsed_time(r1) / 32
        extra["rotating_inputs"] = {"ms_per_step": rot_ms, "value_per_gpu": units_per_rank / (rot_ms * 1e-3) / scale_div,
                                    "unit": unit, "note": "eight input sets (272 MB > 126 MB L2) in rotation, 32 steps "
                                                          "back to back, no flush; the line's value is the flushed one"}
        del sets

    ms_per_step = total_ms / steps
    value = total_units / (ms_per_step * 1e-3) / scale_div

    # ---- end to end: pinned host buffers -> device -> kernel -> host ----
    e2e = None
    if (wl == "prefill_nc" or (wl == "decode_b60" and not light)) and not args.profile:
        host = [t.cpu().pin_memory() for t in host_in]
        dev_in = [torch.empty_like(t) for t in host_in]
        out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        if wl == "decode_b60":
            def e2e_step():
                for d, h in zip(dev_in, host):
                    d.copy_(h, non_blocking=True)
                ops.gqa_decode(dev_in[0], dev_in[1], dev_in[2], kv_layout=layout, out=out)
                out_host.copy_(out, non_blocking=True)
                torch.cuda.current_stream().synchronize()
        else:
            def e2e_step():
                for d, h in zip(dev_in, host):
                    d.copy_(h, non_blocking=True)
                ops.launch_flash_gqa_forward_bf16_kernel(dev_in[0], dev_in[1], dev_in[2], out=out, lse=lse, causal=False)
                out_host.copy_(out, non_blocking=True)
                torch.cuda.current_stream().synchronize()
        n_e2e = max(3, min(steps, 10))
        e2e_step()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        et = torch.tensor([e0.elapsed_time(e1) / n_e2e], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(et, op=dist.ReduceOp.MAX)
        e2e_ms = float(et.item())
        e2e = {"value": total_units / (e2e_ms * 1e-3) / scale_div, "unit": unit, "ms_per_step": e2e_ms,
               "steps": n_e2e,
               "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in host)),
               "d2h_bytes_per_step": int(out_host.numel() * out_host.element_size())}

    rc, detail = ops.device_status()
    if rc != 0:
        raise SystemExit("device status %d %s" % (rc, detail))
    sharded_check = None
    if wl == "decode_long" and world > 1:
        config["exchange"] = dec.exchange
        # kernels of this library per step -- fused: one | peer: decode + exchange | nccl: decode + combine
        launches_per_step = 1 if dec.exchange == "fused" else 2
        if not args.profile:
            sharded_check = check_sharded_decode(ops, torch, dist, dev, rank, world, q, k, v, out, S_total, Hq, Hkv,
                                                 randn_bf16, seeded, barrier)

    if rank != 0:
        return None
    kernel_ms = statistics.mean(per_step)
    achieved = units_per_rank / (kernel_ms * 1e-3) / (1e9 if bound == "hbm" else 1e12)
    peak = peaks["hbm_gbs"] if bound == "hbm" else peaks["bf16_tflops"]
    traffic = NCU_TRAFFIC_BYTES.get(wl)
    roofline = {"bound": bound, "achieved": achieved, "peak": peak, "unit": "GB/s" if bound == "hbm" else "TFLOP/s",
                "frac": achieved / peak, "traffic": traffic, "peak_source": peaks["source"],
                "kernel": "rope_bf16_kernel" if wl == "rope" else "decode_splitkv_kernel; the divisor is the average time of a whole call over the timed region, "
                          "which also holds the counters' memset and launch gaps" if bound == "hbm"
                          else ("bwd_delta_kernel + bwd_grads_kernel (dK/dV and dQ blocks in one grid) + bwd_reduce_kernel (one call)" if wl == "backward"
                                else ("sgqa_fwd_kernel (bound by gathering 512 B per list entry out of L2, mma.sync "
                                      "products; the tensor peak is quoted for scale only)" if wl == "sgqa"
                                      else ("mla_fwd_kernel" if wl == "mla" else
                                            ("mla_fwd_kernel<128> (the one-tile kernel)" if wl == "prefill_chunk"
                                             else "prefill_fwd_kernel")))),
                "kernel_ms": kernel_ms, "kernel_ms_min": min(per_step)}
    if traffic is not None:
        roofline["traffic_captured_at"] = NCU_TRAFFIC_CAPTURED_AT.get(wl)
    if bound == "hbm":
        roofline["frac_of_nominal_8TBps"] = achieved / 8000.0
    else:
        roofline["frac_of_nominal_2250TF"] = achieved / 2250.0
        roofline["frac_of_sustained"] = achieved / peaks["bf16_tflops_sustained"]

    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps,
            "warmup": max(warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config, "roofline": roofline,
            "e2e": e2e, "gpu_launches": launches_per_step * steps, "clocks": clocks, "impl": "ours"}
    line["us_per_step"] = ms_per_step * 1e3
    if e2e is not None:
        # the end-to-end leg is bound by the host link: say what that link delivered on this rank
        e2e["h2d_gbs_per_rank"] = e2e["h2d_bytes_per_step"] / (e2e["ms_per_step"] * 1e-3) / 1e9
    if sharded_check is not None:
        line["sharded_check"] = sharded_check
    if world == 1 and not args.no_cpu_baseline and not args.profile:
        if wl == "decode_b60" and not light:
            line["cpu_baseline"] = cpu_baseline_decode()
        elif wl == "prefill_nc":
            line["cpu_baseline"] = cpu_baseline_prefill_nc()
        elif wl == "prefill_causal" and not light:
            line["cpu_baseline"] = cpu_baseline_prefill_causal()
    if extra:
        line["extra"] = extra
    return line


def check_sharded_decode(ops, torch, dist, dev, rank, world, q, k, v, out_sharded, S_total, Hq, Hkv, randn_bf16,
                         seeded, barrier):
    """The position-sharded result against the single-GPU result and the CPU oracle, and the single-GPU time of the
    same sequence (the N=1 point of the strong-scaling curve, taken in the same run).  Rank 0 rebuilds the whole
    sequence from the shards' seeds; the other ranks wait.  Returns a dict on rank 0, None elsewhere."""
    import numpy as np
    result = None
    if rank == 0:
        from gpu_util import to_bits
        import oracle_lib as ol
        kf = torch.empty((1, S_total, Hkv, 128), dtype=torch.bfloat16, device=dev)
        vf = torch.empty_like(kf)
        for r in range(world):
            s0, s1 = ops.shard_kv_positions(S_total, world, r)
            kf[:, s0:s1] = randn_bf16((1, s1 - s0, Hkv, 128), 0.5, seeded(5000 + 2 * r))
            vf[:, s0:s1] = randn_bf16((1, s1 - s0, Hkv, 128), 0.5, seeded(5001 + 2 * r))
        single = torch.empty_like(q)
        for _ in range(3):
            ops.gqa_decode(q, kf, vf, kv_layout=ops.KV_BSHD, out=single)
        torch.cuda.synchronize()
        n1 = 20
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n1):
            ops.gqa_decode(q, kf, vf, kv_layout=ops.KV_BSHD, out=single)
        t1.record()
        torch.cuda.synchronize()
        single_us = t0.elapsed_time(t1) / n1 * 1e3
        mx, mean, rel = ol.errors(to_bits(out_sharded), to_bits(single))
        # the CPU oracle on one kv head (its 8 query heads), the whole sequence
        h = Hkv - 1
        g = Hq // Hkv
        qs = to_bits(q[:, h * g:(h + 1) * g])
        ks, vs = to_bits(kf[:, :, h:h + 1]), to_bits(vf[:, :, h:h + 1])
        want = ol.decode(qs, ks, vs, 1.0 / np.sqrt(128.0), 0)
        omx, omean, orel = ol.errors(to_bits(out_sharded[:, h * g:(h + 1) * g]), want)
        result = {"single_gpu_us_same_run": single_us,
                  "vs_single_gpu": {"max_abs": mx, "mean_abs": mean, "rel_l2": rel},
                  "vs_cpu_oracle_kv_head_%d" % h: {"max_abs": omx, "mean_abs": omean, "rel_l2": orel},
                  "ok": bool(mx <= 4e-3 and rel <= 5e-3 and omx <= 2e-2 and omean <= 2e-3 and orel <= 2e-2)}
        del kf, vf
    barrier()
    return result


# ------------------------------------------------------------------------------------------------
# CPU arms (upstream's own CPU implementation of the decode path)
# ------------------------------------------------------------------------------------------------
def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _run_ref_binary():
    """One run of the unmodified upstream benchmark program (stubbed runtime): its CPU loop at the headline shape."""
    import oracle_lib as ol
    env = dict(os.environ, OMP_NUM_THREADS=str(host_threads()))  # torchrun exports OMP_NUM_THREADS=1
    out = subprocess.run([ol.REF_BIN], capture_output=True, text=True, timeout=1200, env=env)
    m = re.search(r"CPU time = ([0-9.eE+-]+)s", out.stdout)
    if out.returncode != 0 or not m:
        raise RuntimeError("reference binary failed: " + out.stdout[-400:] + out.stderr[-400:])
    err = re.search(r"O error = (\S+)", out.stdout)
    return float(m.group(1)), (float(err.group(1)) if err else None)


def _port_sample_seconds(B):
    import numpy as np
    import oracle_lib as ol
    S, Hq, Hkv = 4096, 128, 8
    q = ol.randn_bf16((B, Hq, 128), 1)
    k = ol.randn_bf16((B, S, Hkv, 128), 2)
    v = ol.randn_bf16((B, S, Hkv, 128), 3)
    t = time.perf_counter()
    ol.decode(q, k, v, 1.0 / np.sqrt(128.0), 0, par_heads=False)
    return time.perf_counter() - t


def cpu_baseline_decode():
    import oracle_lib as ol
    cores = host_threads() if os.path.exists(ol.REF_BIN) else ol.lib().cllo_oracle_num_threads()
    full = decode_bytes(60, 4096, 128, 8)
    if os.path.exists(ol.REF_BIN):
        secs, err = _run_ref_binary()
        return {"value": full / secs / 1e12, "unit": "TB/s", "cores": cores, "kind": "reference", "seconds": secs,
                "sample": "the whole headline workload (B=60, S=4096, Hq=128, Hkv=8), one run of upstream's "
                          "unmodified test_decode_flash_gqa.cu CPU loop (OpenMP over batch); restatement vs "
                          "upstream relative error printed by that program: %s" % err}
    B = 16
    secs = _port_sample_seconds(B)
    return {"value": decode_bytes(B, 4096, 128, 8) / secs / 1e12, "unit": "TB/s", "cores": cores, "kind": "port",
            "seconds": secs, "sample": "B=%d of the 60 sequences of the headline workload, C restatement" % B}


def cpu_baseline_prefill_nc():
    """The C restatement of upstream's torch forward reference (examples/python/Triton/test_flash_gqa_kernel.py:27-94,
    mask made optional) on the whole non-causal baseline shape, all host threads."""
    import numpy as np
    import oracle_lib as ol
    B, S, Hq, Hkv = 1, 4096, 16, 1
    q, k, v = ol.randn_bf16((B, Hq, S, 128), 1), ol.randn_bf16((B, Hkv, S, 128), 2), ol.randn_bf16((B, Hkv, S, 128), 3)
    t = time.perf_counter()
    ol.prefill(q, k, v, 1.0 / np.sqrt(128.0), False)
    secs = time.perf_counter() - t
    return {"value": prefill_flops(B, Hq, S, S) / secs / 1e12, "unit": "TFLOP/s", "cores": ol.lib().cllo_oracle_num_threads(),
            "kind": "port", "seconds": secs,
            "sample": "the whole prefill_nc workload (B=1, S=4096, Hq=16, Hkv=1, non-causal), one run of the C "
                      "restatement of upstream's forward reference"}


def cpu_baseline_prefill_causal():
    """The same restatement on a bounded sample of the causal baseline shape: the last 2048 query rows of one head."""
    import numpy as np
    import oracle_lib as ol
    S, rows = 16384, 2048
    q, k, v = ol.randn_bf16((1, 1, S, 128), 1), ol.randn_bf16((1, 1, S, 128), 2), ol.randn_bf16((1, 1, S, 128), 3)
    t = time.perf_counter()
    ol.prefill(q, k, v, 1.0 / np.sqrt(128.0), True, row_begin=S - rows, row_end=S)
    secs = time.perf_counter() - t
    flops = 4.0 * 128 * sum(range(S - rows + 1, S + 1))  # visible keys of those rows
    return {"value": flops / secs / 1e12, "unit": "TFLOP/s", "cores": ol.lib().cllo_oracle_num_threads(), "kind": "port",
            "seconds": secs, "sample": "query rows [%d, %d) of one (batch, head) of the causal shape (S=16384), C "
                                       "restatement of upstream's forward reference" % (S - rows, S)}


def run_ours(args, rank, world, local_rank):
    """The default run: the headline line, carrying short runs of the other baseline configurations."""
    import torch

    def run(wl, steps, warmup, light):
        res = measure(args, wl, rank, world, local_rank, steps, warmup, light)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        return res

    if args.workload != "all":
        line = run(args.workload, args.steps, args.warmup, False)
        if rank == 0:
            print(json.dumps(line), flush=True)
        return
    line = run("decode_b60", args.steps, args.warmup, False)
    plan = [("prefill_nc", 30), ("prefill_causal", 5), ("decode_long", 50)]
    if world > 1:
        plan.append(("decode_b60_strong", 100))
    also, roof = {}, {}
    for wl, steps in plan:
        res = run(wl, steps, 5, True)
        if rank != 0:
            continue
        r = res["roofline"]
        entry = {"workload": res["config"]["workload"], "metric": res["metric"], "value": res["value"],
                 "unit": res["unit"], "us_per_step": res["us_per_step"], "steps": res["steps"], "scaling": res["scaling"],
                 "sharding": res["config"].get("sharding")}
        for key in ("exchange", "launch"):
            if key in res["config"]:
                entry[key] = res["config"][key]
        for key in ("e2e", "cpu_baseline", "sharded_check"):
            if res.get(key) is not None:
                entry[key] = res[key]
        if (res.get("extra") or {}).get("rotating_inputs"):
            entry["rotating_inputs"] = res["extra"]["rotating_inputs"]
        if wl == "decode_long" and res.get("sharded_check"):
            entry["speedup_over_1_gpu_same_run"] = res["sharded_check"]["single_gpu_us_same_run"] / res["us_per_step"]
        also[wl] = entry
        roof[wl] = {"bound": r["bound"], "achieved_per_gpu": r["achieved"], "peak": r["peak"], "unit": r["unit"],
                    "frac": r["frac"], "kernel_ms": r["kernel_ms"],
                    "frac_of_nominal": r.get("frac_of_nominal_8TBps", r.get("frac_of_nominal_2250TF"))}
    if rank == 0:
        line["config"]["also_measured"] = also
        line["roofline"]["others"] = roof
        print(json.dumps(line), flush=True)


def run_reference(args, rank, world):
    """Upstream's CPU implementation on the host cores; rank 0 only."""
    if rank != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(host_threads())  # before the OpenMP runtime of the port starts
    import oracle_lib as ol
    ol.build_oracle()
    cores = host_threads() if os.path.exists(ol.REF_BIN) else ol.lib().cllo_oracle_num_threads()
    full = decode_bytes(60, 4096, 128, 8)
    if os.path.exists(ol.REF_BIN):
        n = max(1, min(args.steps, 4))  # each run regenerates 1 GB of inputs (~20-30 s); keep the arm to minutes
        secs = [_run_ref_binary()[0] for _ in range(n)]
        kind, sample = "reference", ("%d run(s) of upstream's unmodified test_decode_flash_gqa.cu CPU loop on the whole "
                                     "headline workload; --steps %d requested, capped at 4" % (n, args.steps))
        per = statistics.mean(secs)
        units = full
    else:
        B = 16
        n = max(1, min(args.steps, 10))
        secs = [_port_sample_seconds(B) for _ in range(n)]
        kind, sample = "port", "B=%d of 60 sequences per step, C restatement of upstream's loop, %d step(s)" % (B, n)
        per = statistics.mean(secs)
        units = decode_bytes(B, 4096, 128, 8)
    value = units / per / 1e12
    line = {"metric": "gqa_decode_achieved_hbm_tbps", "value": value, "unit": "TB/s", "n_gpus": world, "steps": n,
            "warmup": 0, "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {"workload": "decode_b60: GQA decode B=60, S=4096, Hq=128, Hkv=8, D=128 on host cores"},
            "cpu_baseline": {"value": value, "unit": "TB/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all",
                    choices=["all", "decode_b60", "decode_b60_strong", "decode_step_rope", "decode_long", "prefill_nc", "prefill_causal", "swa", "backward", "rope", "sgqa", "mla", "prefill_chunk"])
    ap.add_argument("--layout", default="bshd", choices=["bshd", "bhsd"])
    ap.add_argument("--batch", type=int, default=0,
                    help="decode_b60 / prefill_chunk: override the per-GPU batch (small cases for profiler captures; "
                         "prefill_chunk at a batch of 1-4 runs with the kv range shared out among blocks)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "peer", "nccl"],
                    help="decode_long on several GPUs: how the per-GPU partials are exchanged")
    ap.add_argument("--kv-len", type=int, default=0,
                    help="decode_long only: override the total KV length (profiling one GPU's share of a sharded run)")
    ap.add_argument("--no-graph", action="store_true", help="decode_long on several GPUs: launch eagerly")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="for runs under a profiler: no CPU baseline, no end-to-end leg, no clock-sampling repeats")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with: python -m torch.distributed.run --nnodes=1 "
                             "--nproc-per-node %d --master-addr 127.0.0.1 bench.py --gpus %d ..." % (args.gpus, args.gpus))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
