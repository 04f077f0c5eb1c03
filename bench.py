#!/usr/bin/env python
"""Benchmark of the block-sparse attention hot path.

    python bench.py --gpus N --steps K --warmup W [--workload prefill|train|decode|varlen]
    torchrun --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # CPU restatement of the reference path

One JSON line on stdout (rank 0).  The default workload is BASELINE config 2
(Phi-3-small-shape local-stride prefill forward): a step is one forward pass
over one synthetic batch; ``value`` = attended-block TFLOP/s of the whole job
with inputs resident in HBM; ``e2e`` = the same through the module API with
pinned host inputs copied in and the output copied back every step.

Multi-GPU (one process per GPU): q heads are sharded over the ranks through
``active_head_range`` (no collective on the data path) and the batch grows with
the world size, so per-GPU work is constant ("weak").  ``--workload decode`` at
N > 1 shards the KV sequence and merges partial (O, LSE) after one NCCL
all-gather.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sparse_attn_attended_tflops"
NOMINAL_BF16_TFLOPS = 2250.0
NOMINAL_HBM_GBS = 8000.0
E2E_CHUNK = 4096   # query rows per pipelined chunk of the end-to-end prefill step

WORKLOADS = {
    # BASELINE.json configs[1..4]
    "prefill": dict(B=4, S=8192, Hq=32, Hkv=8, D=128, block=64, local=16, stride=8),
    "train": dict(B=2, S=8192, Hq=32, Hkv=32, D=128, block=64, local=32, stride=8),
    "decode": dict(B=64, S=8192, Hq=32, Hkv=8, D=128, block=64, local=16, stride=8),
    "varlen": dict(H=32, D=128, block=64, max_seq=16384, nseq=16, lo=512, hi=4096, p=0.2),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(tflops=d["bf16_tflops"], tflops_sustained=d.get("bf16_tflops_sustained"),
                    hbm=d["hbm_gbs"], source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi SM clock / throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- work accounting
def local_stride_mask_np(Hq, S, block, local, stride, Hkv):
    """Block mask of the local-stride pattern (numpy; FLOP accounting only)."""
    nb = (S + block - 1) // block
    step = max(1, int(stride / Hq))
    g = Hq // Hkv
    q = np.arange(nb)[:, None]
    k = np.arange(nb)[None, :]
    loc = ((q - k) < local) & ((k - q) < 1)
    out = np.zeros((Hq, nb, nb), dtype=bool)
    for h in range(Hq):
        vert = ((np.arange(nb) + (h // g) * step) % stride == 0)[None, :]
        out[h] = (vert | loc) & (q >= k)
    return out


def tile_flops(block, D):
    return 4.0 * block * block * D      # QK^T and PV, 2 flops per MAC


# --------------------------------------------------------------------------- GPU arm
def setup_dist(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        torch.cuda.set_device(0)
    return world, rank, local_rank


def barrier_sync(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def time_steps(fn, steps, warmup, world):
    """W warm-up steps, then exactly K steps between CUDA events on the launching
    stream, bracketed by barrier + synchronize; returns ms per step (this rank)."""
    for _ in range(warmup):
        fn()
    barrier_sync(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier_sync(world)
    return e0.elapsed_time(e1) / steps


def cpu_baseline_c1(max_seconds=20.0):
    """BASELINE config 1 on the host cores: the masked-dense torch path of the
    reference (restated in oracle/), fp32, all threads.  Returns the dict for the
    JSON line; value is attended-block TFLOP/s (620 tiles of 64x64x64)."""
    from oracle import dkernel_oracle as O
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 1024, 8, 64) for _ in range(3))
    bm = O.block_mask(8, 1024, 64, 4, 4)
    dense = O.token_mask(bm, 64, 1024, 1024)
    cores = torch.get_num_threads()
    O.masked_dense_attention(q, k, v, dense, 0.125, seq_dim=1)
    best, t_start, n = float("inf"), time.time(), 0
    while n < 5 or (time.time() - t_start < 2.0 and n < 50):
        t0 = time.perf_counter()
        O.masked_dense_attention(q, k, v, dense, 0.125, seq_dim=1)
        best = min(best, time.perf_counter() - t0)
        n += 1
        if time.time() - t_start > max_seconds:
            break
    flops = int(bm.sum()) * 4.0 * 64 * 64 * 64
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"BASELINE config 1 (B1,S1024,H8,D64,fp32, block 64, local 4, stride 4), "
                      f"masked-dense oracle, best of {n} runs = {best * 1e3:.2f} ms"}


def run_prefill(args, world, rank):
    from dkernel_b200 import LocalStrideSparseAttention, _lib
    from dkernel_b200.dist import head_shard
    cfg = WORKLOADS["prefill"]
    B, S, Hq, Hkv, D = cfg["B"] * world, cfg["S"], cfg["Hq"], cfg["Hkv"], cfg["D"]
    (h0, h1), (kv0, kv1) = head_shard(Hq, Hkv, rank, world)
    hq_l, hkv_l = h1 - h0, kv1 - kv0
    attn = LocalStrideSparseAttention(Hq, S, cfg["block"], cfg["local"], cfg["stride"], num_kv_heads=Hkv,
                                      active_head_range=(h0, h1) if world > 1 else None, seq_dim=1)
    g = torch.Generator().manual_seed(1234 + rank)
    hq_host = torch.randn((B, S, hq_l, D), generator=g).to(torch.bfloat16).pin_memory()
    hk_host = torch.randn((B, S, hkv_l, D), generator=g).to(torch.bfloat16).pin_memory()
    hv_host = torch.randn((B, S, hkv_l, D), generator=g).to(torch.bfloat16).pin_memory()
    q, k, v = hq_host.cuda(), hk_host.cuda(), hv_host.cuda()
    scale = 1.0 / math.sqrt(D)
    mask = local_stride_mask_np(Hq, S, cfg["block"], cfg["local"], cfg["stride"], Hkv)[h0:h1]
    tiles = int(mask.sum()) * B
    flops = tiles * tile_flops(cfg["block"], D)

    def step():
        with torch.no_grad():
            attn(q, k, v, sm_scale=scale, return_lse=True)

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ms = time_steps(step, args.steps, args.warmup, world)
    clocks = sampler.stop()
    assert _lib.wait_status() == 0, "a device-side wait gave up: results invalid"

    # e2e: pinned host -> device, forward through the public API, output -> pinned host
    out_host = torch.empty((B, S, hq_l, D), dtype=torch.bfloat16).pin_memory()
    lse_host = torch.empty((B, hq_l, S), dtype=torch.float32).pin_memory()

    # The step is pipelined over three streams in chunks of E2E_CHUNK query rows: causal attention
    # of rows [s0, s1) needs keys [0, s1) only, so chunk c is computed (q shorter than k, the
    # module's chunked-prefill case) while the host->device copy of chunk c+1 and the device->host
    # copy of chunk c-1 run (PCIe is full duplex); the timed stream waits for the last copy out.
    # All chunk copies are contiguous; the LSE rows go out once per batch element.
    qd, kd, vd = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    lse_dev = torch.empty((B, hq_l, S), dtype=torch.float32, device="cuda")
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    chunk = max(cfg["block"], min(args.e2e_chunk, S))
    # one module per chunk offset: the pattern rows of query rows [s0, s1) over keys [0, s1)
    # (the reference's recipe for sequence partitions: get_sparse_attn_mask with
    # q_start_position / kv_seqlen, then SparseAttention on the block mask)
    from dkernel_b200 import SparseAttention, get_sparse_attn_mask
    chunk_attn = {}
    for s0 in range(0, S, chunk):
        s1 = min(s0 + chunk, S)
        bmask = get_sparse_attn_mask(Hq, s1 - s0, cfg["block"], cfg["local"], cfg["stride"], dtype=torch.uint8,
                                     num_kv_heads=Hkv, q_start_position=s0, kv_start_position=0,
                                     kv_seqlen=s1)[1]
        chunk_attn[s0] = SparseAttention(cfg["block"], bmask[h0:h1].contiguous(), seq_dim=1, causal=True)

    def step_e2e():
        main = torch.cuda.current_stream()
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        with torch.no_grad():
            for b in range(B):
                for s0 in range(0, S, chunk):
                    s1 = min(s0 + chunk, S)
                    with torch.cuda.stream(s_in):
                        qd[b, s0:s1].copy_(hq_host[b, s0:s1], non_blocking=True)
                        kd[b, s0:s1].copy_(hk_host[b, s0:s1], non_blocking=True)
                        vd[b, s0:s1].copy_(hv_host[b, s0:s1], non_blocking=True)
                        ev_in = torch.cuda.Event()
                        ev_in.record(s_in)
                    main.wait_event(ev_in)
                    o, l = chunk_attn[s0](qd[b:b + 1, s0:s1], kd[b:b + 1, :s1], vd[b:b + 1, :s1],
                                          sm_scale=scale, return_lse=True)
                    lse_dev[b, :, s0:s1].copy_(l[0])
                    ev_c = torch.cuda.Event()
                    ev_c.record(main)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(ev_c)
                        out_host[b, s0:s1].copy_(o[0], non_blocking=True)
                        o.record_stream(s_out)
                        if s1 == S:
                            lse_host[b].copy_(lse_dev[b], non_blocking=True)
        main.wait_stream(s_out)

    # the chunked step must reproduce the one-call result
    with torch.no_grad():
        o_full, l_full = attn(q, k, v, sm_scale=scale, return_lse=True)
    step_e2e()
    torch.cuda.synchronize()
    assert (out_host.float() - o_full.cpu().float()).abs().max().item() <= 2e-2, "chunked e2e output differs"
    assert (lse_host - l_full.cpu()).abs().max().item() <= 1e-3, "chunked e2e LSE differs"
    del o_full, l_full

    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e = time_steps(step_e2e, e2e_steps, 3, world)

    ms_max = max_over_ranks(ms, world)
    ms_e2e_max = max_over_ranks(ms_e2e, world)
    flops_all = sum_over_ranks(flops, world)
    peaks = measured_peaks()
    kernel_tflops = flops / (ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": flops_all / (ms_max * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_max,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "prefill_fwd: BASELINE config 2 (Phi-3-small shape), B=%d (4 per GPU), S=8192, "
                               "Hq=32, Hkv=8, D=128, block 64, local 16, stride 8, causal, return_lse" % B,
                   "parallelism": f"heads sharded over {world} GPU(s) via active_head_range, no collective",
                   "attended_tiles_per_step": int(round(flops_all / tile_flops(cfg["block"], D))),
                   "flops_convention": "4*64*64*128 per attended block, diagonal blocks counted full",
                   "l2": "inputs (q 256 MiB + k,v 64 MiB each per GPU) exceed the 126 MB L2"},
        "e2e": {"value": flops_all / (ms_e2e_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": ms_e2e_max,
                "pipeline": f"chunked prefill, {chunk} query rows per module call, copies overlapped",
                "h2d_bytes_per_step": (hq_host.numel() + hk_host.numel() + hv_host.numel()) * 2,
                "d2h_bytes_per_step": out_host.numel() * 2 + lse_host.numel() * 4},
        "gpu_launches": args.steps,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": peaks["tflops"],
                     "unit": "TFLOP/s", "frac": kernel_tflops / peaks["tflops"],
                     "traffic": TRAFFIC.get("prefill"), "peak_source": peaks["source"] + " (burst)",
                     "frac_of_sustained": kernel_tflops / peaks["tflops_sustained"] if peaks["tflops_sustained"] else None,
                     "frac_of_nominal_2250": kernel_tflops / NOMINAL_BF16_TFLOPS,
                     "kernel": "fwd_persist_kernel<bf16>", "kernel_ms": ms},
    }
    return line


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel from
# the committed ncu captures (profiles/*.md), one GPU, the full workload; None = not captured.
# train: dK/dV 796.7 MB + dQ 664.6 MB (the roofline line covers both backward kernels).
TRAFFIC = {"prefill": 684.5e6, "train": 796.7e6 + 664.6e6, "decode": 406.3e6, "varlen": None}


def run_train(args, world, rank):
    from dkernel_b200 import LocalStrideSparseAttention, _lib
    from dkernel_b200.dist import head_shard
    cfg = WORKLOADS["train"]
    B, S, Hq, D = cfg["B"] * world, cfg["S"], cfg["Hq"], cfg["D"]
    (h0, h1), _ = head_shard(Hq, Hq, rank, world)
    hl = h1 - h0
    attn = LocalStrideSparseAttention(Hq, S, cfg["block"], cfg["local"], cfg["stride"],
                                      active_head_range=(h0, h1) if world > 1 else None, seq_dim=1)
    g = torch.Generator().manual_seed(99 + rank)
    q, k, v, do = (torch.randn((B, S, hl, D), generator=g).to(torch.bfloat16).cuda() for _ in range(4))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    mask = local_stride_mask_np(Hq, S, cfg["block"], cfg["local"], cfg["stride"], Hq)[h0:h1]
    tiles = int(mask.sum()) * B
    fwd_flops = tiles * tile_flops(cfg["block"], D)

    def step():
        q.grad = k.grad = v.grad = None
        out = attn(q, k, v)
        out.backward(do)

    def step_fwd():
        with torch.no_grad():
            attn(q, k, v, return_lse=True)

    ms_fwd = max_over_ranks(time_steps(step_fwd, args.steps, args.warmup, world), world)
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ms = max_over_ranks(time_steps(step, args.steps, args.warmup, world), world)
    clocks = sampler.stop()
    assert _lib.wait_status() == 0
    total = sum_over_ranks(fwd_flops * 3.5, world)
    peaks = measured_peaks()
    bwd_ms = ms - ms_fwd
    bwd_tflops = sum_over_ranks(fwd_flops * 2.5, world) / world / (bwd_ms * 1e-3) / 1e12
    return {
        "metric": METRIC, "value": total / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "train fwd+bwd: BASELINE config 3, B=%d (2 per GPU), S=8192, H=32, D=128, "
                               "block 64, local 32, stride 8; FLOPs = 3.5 x forward (5 backward GEMMs, "
                               "recomputation not counted)" % B,
                   "fwd_ms": ms_fwd, "bwd_ms": bwd_ms},
        "gpu_launches": args.steps * 4, "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": bwd_tflops, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": bwd_tflops / peaks["tflops"], "traffic": TRAFFIC.get("train"),
                     "peak_source": peaks["source"] + " (burst)",
                     "frac_of_sustained": bwd_tflops / peaks["tflops_sustained"] if peaks["tflops_sustained"] else None,
                     "kernel": "bwd_dkdv_sm100_kernel + bwd_dq_sm100_kernel (+ delta pre-pass)"},
    }


def decode_inputs(cfg, rank_seed=0):
    B, S, Hq, Hkv, D = cfg["B"], cfg["S"], cfg["Hq"], cfg["Hkv"], cfg["D"]
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(1024, 8193, (B,), generator=g)
    return lens


def attended_kv_tokens(lens, mask_kv, block):
    """sum over sequences and kv heads of the real tokens in attended blocks."""
    total = 0
    for L in lens.tolist():
        row = (L - 1) // block
        for h in range(mask_kv.shape[0]):
            cols = np.nonzero(mask_kv[h, row])[0]
            total += int(np.minimum((cols + 1) * block, L).sum() - (cols * block).sum())
    return total


def run_decode(args, world, rank):
    from dkernel_b200 import LocalStrideSparseAttention, _lib
    from dkernel_b200.dist import kv_shard_ranges, sharded_decode
    cfg = WORKLOADS["decode"]
    B, S, Hq, Hkv, D, bs = cfg["B"], cfg["S"], cfg["Hq"], cfg["Hkv"], cfg["D"], cfg["block"]
    lens = decode_inputs(cfg)
    attn = LocalStrideSparseAttention(Hq, S, bs, cfg["local"], cfg["stride"], num_kv_heads=Hkv, seq_dim=1)
    g = torch.Generator().manual_seed(7)
    q = torch.randn((B, 1, Hq, D), generator=g).to(torch.bfloat16).cuda()
    mask_kv = local_stride_mask_np(Hq, S, bs, cfg["local"], cfg["stride"], Hkv)[::Hq // Hkv]
    tokens = attended_kv_tokens(lens, mask_kv, bs)
    bytes_alg = tokens * D * 2 * 2 + 2 * B * Hq * D * 2
    scale = 1.0 / math.sqrt(D)
    nbuf = 4 if world == 1 else 2            # rotate K/V buffers so the L2 never holds the next step's data
    if world == 1:
        left = (S - lens).to(torch.int32).cuda()
        bufs = []
        for i in range(nbuf):
            k = torch.randn((B, S, Hkv, D), generator=g).to(torch.bfloat16).cuda()
            v = torch.randn((B, S, Hkv, D), generator=g).to(torch.bfloat16).cuda()
            bufs.append((k, v))
        it = [0]

        def eager_step():
            k, v = bufs[it[0] % nbuf]
            it[0] += 1
            with torch.no_grad():
                attn(q, k, v, sm_scale=scale, left_paddings=left, return_lse=True)
        launches = 2
    else:
        lo, hi = kv_shard_ranges(lens, rank, world, bs)
        n = (hi - lo).clamp_min(0)
        cap = int(((S // world + bs - 1) // bs + 1) * bs)
        bufs = []
        for i in range(nbuf):
            ks = torch.randn((B, cap, Hkv, D), generator=g).to(torch.bfloat16).cuda()
            vs = torch.randn((B, cap, Hkv, D), generator=g).to(torch.bfloat16).cuda()
            bufs.append((ks, vs))
        n_d, lo_d, len_d = (t.to(torch.int32).cuda() for t in (n, lo, lens))
        it = [0]

        def eager_step():
            ks, vs = bufs[it[0] % nbuf]
            it[0] += 1
            with torch.no_grad():
                sharded_decode(attn, q, ks, vs, n_d, lo_d, len_d, scale)
        launches = 4   # decode, split merge, NCCL all-gather, partition merge
    step, launch_mode = eager_step, "eager calls"
    if not args.no_graph and args.steps % nbuf == 0:
        # A decode step is a few short kernels (and, sharded, one small all-gather): the call is
        # captured once per K/V buffer set and replayed, as a serving loop would, so that the step
        # is not bound by the Python launch path.
        try:
            graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
            with torch.cuda.stream(side):
                for _ in range(nbuf):
                    eager_step()
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(nbuf):
                        eager_step()
            torch.cuda.synchronize()

            def step():
                if it[0] % nbuf == 0:
                    graph.replay()
                it[0] += 1
            it[0] = 0
            launch_mode = f"CUDA graph of {nbuf} calls (one per K/V buffer set), replayed"
        except Exception as e:   # capture unsupported in this setup: time the eager calls
            launch_mode = f"eager calls (graph capture failed: {type(e).__name__})"
            step = eager_step
        if world > 1:
            # every rank must make the same choice, or the collectives would not match up
            flag = torch.tensor([1.0 if step is not eager_step else 0.0], device="cuda")
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
            if flag.item() == 0.0 and step is not eager_step:
                step, launch_mode = eager_step, "eager calls (graph capture failed on another rank)"
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ms = max_over_ranks(time_steps(step, args.steps, args.warmup, world), world)
    clocks = sampler.stop()
    assert _lib.wait_status() == 0
    peaks = measured_peaks()
    gbs = bytes_alg / world / (ms * 1e-3) / 1e9
    return {
        "metric": "sparse_attn_decode_us_per_step", "value": ms * 1e3, "unit": "us", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "decode: BASELINE config 4, B=64, one query token, Hq=32, Hkv=8, D=128, KV lengths "
                               "U[1024,8192] left-padded to 8192, block 64, local 16, stride 8",
                   "parallelism": "single GPU" if world == 1 else
                   f"KV sequence sharded over {world} GPUs, one NCCL all-gather of (O,LSE) + fused merge",
                   "algorithmic_bytes_per_step": bytes_alg,
                   "launch": launch_mode,
                   "l2": f"{nbuf} K/V buffer sets rotated ({nbuf}x{2 * B * S * Hkv * D * 2 / world / 2**20:.0f} MiB)"},
        "gpu_launches": args.steps * launches, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm"], "traffic": TRAFFIC.get("decode"),
                     "peak_source": peaks["source"], "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS,
                     "kernel": "decode_kernel<bf16,128> (+ merge_kernel)", "per_gpu": True},
    }


def run_varlen(args, world, rank):
    from dkernel_b200 import SparseAttention, _lib
    from dkernel_b200.dist import head_shard
    import warnings
    cfg = WORKLOADS["varlen"]
    H, D, bs = cfg["H"], cfg["D"], cfg["block"]
    nb = cfg["max_seq"] // bs
    g = torch.Generator().manual_seed(0)
    pat = torch.rand((H, nb, nb), generator=g) < cfg["p"]
    pat |= torch.eye(nb, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
    lens = torch.randint(cfg["lo"], cfg["hi"] + 1, (cfg["nseq"],), generator=g)
    (h0, h1), _ = head_shard(H, H, rank, world)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        attn = SparseAttention(bs, pat[h0:h1].cuda())
    T = int(lens.sum())
    q, k, v = (torch.randn((T, h1 - h0, D), generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    cu = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)]).to(torch.int32).cuda()
    tiles = 0
    pn = pat[h0:h1].numpy()
    for L in lens.tolist():
        n = (L + bs - 1) // bs
        tiles += int(pn[:, :n, :n].sum())
    flops = tiles * tile_flops(bs, D)

    def step():
        with torch.no_grad():
            attn(q, k, v, cu_seqlen_k=cu)

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ms = time_steps(step, args.steps, args.warmup, world)
    clocks = sampler.stop()
    assert _lib.wait_status() == 0
    ms_max = max_over_ranks(ms, world)
    total = sum_over_ranks(flops, world)
    peaks = measured_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    return {
        "metric": METRIC, "value": total / (ms_max * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_max, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "varlen prefill, user pattern: BASELINE config 5, H=32, D=128, block 64, "
                               "Bernoulli(0.2) lower-triangular 256x256 pattern, 16 packed sequences "
                               f"U[512,4096] (sum {T} tokens)",
                   "parallelism": f"heads sharded over {world} GPU(s)", "attended_tiles": int(total / tile_flops(bs, D))},
        "gpu_launches": args.steps, "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": tf / peaks["tflops"], "traffic": TRAFFIC.get("varlen"),
                     "peak_source": peaks["source"] + " (burst)", "kernel": "fwd_persist_kernel<bf16>"},
    }


# --------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The reference's CPU path for this metric: masked-dense attention (its test
    oracle, restated in oracle/) on the host cores, all threads.  Each step is a
    bounded sample of the GPU arm's workload: ONE (batch, head) pair of config 2
    at full sequence length (the pattern differs per kv group; head 0 is used)."""
    from oracle import dkernel_oracle as O
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    cfg = WORKLOADS["prefill"]
    S, D, bs = cfg["S"], cfg["D"], cfg["block"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    q = torch.randn((1, S, 1, D), generator=g).to(torch.bfloat16)
    k = torch.randn((1, S, 1, D), generator=g).to(torch.bfloat16)
    v = torch.randn((1, S, 1, D), generator=g).to(torch.bfloat16)
    bm = O.block_mask(cfg["Hq"], S, bs, cfg["local"], cfg["stride"], num_kv_heads=cfg["Hkv"])[:1]
    flops = int(bm.sum()) * tile_flops(bs, D)
    dense = O.token_mask(bm, bs, S, S)

    def step():
        O.masked_dense_attention(q.float(), k.float(), v.float(), dense, 1 / math.sqrt(D), seq_dim=1)

    for _ in range(min(args.warmup, 2)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = flops / dt / 1e12
    sample = ("1 of the %d (batch, head) pairs of BASELINE config 2 per step (B=1, Hq=1 slice, S=8192, D=128), "
              "masked-dense fp32 on CPU" % (cfg["B"] * cfg["Hq"]))
    return {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "prefill_fwd: BASELINE config 2 (Phi-3-small shape) -- " + sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill", choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-chunk", type=int, default=E2E_CHUNK,
                    help="prefill: query rows per pipelined chunk of the end-to-end step")
    ap.add_argument("--no-graph", action="store_true", help="decode: time eager module calls, not a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = min(args.steps, 5)
        line = run_reference(args)
        if line is not None:
            print(json.dumps(line), flush=True)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path); "
                         "use --impl reference for the CPU restatement")
    args.warmup = max(args.warmup, 3)
    world, rank, _ = setup_dist(args)
    if args.gpus != world and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)
    line = {"prefill": run_prefill, "train": run_train, "decode": run_decode,
            "varlen": run_varlen}[args.workload](args, world, rank)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_c1()
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
