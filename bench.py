#!/usr/bin/env python
"""Benchmark of the block-sparse attention hot path.

    python bench.py --gpus N --steps K --warmup W [--workload prefill|train|decode|varlen]
    torchrun --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # CPU restatement of the reference path

One JSON line on stdout (rank 0).  The headline is BASELINE config 2
(Phi-3-small-shape local-stride prefill forward): a step is one forward pass
over one synthetic batch; ``value`` = attended-block TFLOP/s of the whole job
with inputs resident in HBM; ``e2e`` = the same through the module API with
pinned host inputs copied in and the output copied back every step.  Every
timed region is exactly K steps between CUDA events; it is repeated (5 times by
default) and the median is reported with the spread.

The default run (``--workload all``) also times the rest of the metric and puts
compact numeric sub-records under ``config.sub`` (and their roofline fractions
under ``roofline.sub``): at one GPU the training step of config 3 (forward,
backward), the decode step of config 4 (CUDA-graph replay and eager calls), the
packed varlen prefill of config 5 and a head-dim-64 prefill; at N > 1 the
KV-sharded decode step (peer-store exchange kernel and NCCL all-gather route,
both checked against the one-GPU decode of the same cache before timing), and
configs 2 and 5 at fixed total size with heads sharded ("strong").

Multi-GPU (one process per GPU): q heads are sharded over the ranks through
``active_head_range`` (no collective on the data path) and the batch grows with
the world size, so per-GPU work of the headline is constant ("weak").
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
    """SM clock and throttle reasons sampled while a timed region runs: NVML polled from a thread
    every few milliseconds (a timed region lasts tens of milliseconds), nvidia-smi as fallback."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_index: int, period_s: float = 0.004):
        self.gpu, self.period = gpu_index, period_s
        self.proc = self.thread = self.handle = None
        self.lines, self.sm, self.bits, self.power = [], [], 0, []
        self.stop_flag = threading.Event()
        self.max_mhz = None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                return int(vis.split(",")[self.gpu])
            except (ValueError, IndexError):
                return self.gpu
        return self.gpu

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:      # the CUDA ordinal and the NVML index need not agree: look the device up by UUID
                uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
                uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.handle = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self._physical_index())], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
            except Exception:
                pass
            time.sleep(self.period)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.handle is not None:
            self.stop_flag.set()
            self.thread.join(timeout=1)
            reasons = sorted(name for bit, name in self.REASONS.items() if self.bits & bit)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None,
                    "sm_min_mhz": float(min(self.sm)) if self.sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": reasons, "samples": len(self.sm),
                    "power_w_max": float(max(self.power)) if self.power else None, "source": "nvml"}
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
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


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
def bind_to_gpu_cpus(local_rank: int):
    """Pin this process to the host cores NVML reports as local to its GPU, before any pinned host
    memory is allocated (first touch then places the staging buffers on that NUMA node).  Returns
    the number of cores bound to, or None when NVML or the affinity call is unavailable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
        uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def setup_dist(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # also at one GPU: on a two-socket host the pinned staging buffers of the end-to-end step should
    # sit on the GPU's own NUMA node
    args.bound_cpus = bind_to_gpu_cpus(local_rank)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                timeout=datetime.timedelta(seconds=300))
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


REPEATS = 5


def time_steps(fn, steps, warmup, world, repeats=None):
    """W warm-up steps, then `repeats` timed regions of exactly K steps each, every region
    between CUDA events on the launching stream and bracketed by barrier + synchronize.
    Returns (median ms per step of this rank, [ms per step of every region])."""
    repeats = repeats or REPEATS
    for _ in range(warmup):
        fn()
    regions = []
    for _ in range(repeats):
        barrier_sync(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier_sync(world)
        regions.append(e0.elapsed_time(e1) / steps)
    return float(np.median(regions)), regions


def timed(fn, steps, warmup, world, repeats=None):
    """time_steps with the clocks sampled over all regions and the max over ranks taken.
    Returns (ms median max-over-ranks, spread dict, clocks dict, ms of this rank)."""
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ms, regions = time_steps(fn, steps, warmup, world, repeats)
    clocks = sampler.stop()
    ms_max = max_over_ranks(ms, world)
    spread = {"ms_min": min(regions), "ms_max": max(regions), "repeats": len(regions)}
    return ms_max, spread, clocks, ms


def cpu_baseline_c1(max_seconds=12.0):
    """BASELINE config 1 on the host cores: the masked-dense torch path of the
    reference (restated in oracle/), fp32, with all threads and with one.  Returns the dict for
    the JSON line; value is attended-block TFLOP/s (620 tiles of 64x64x64)."""
    from oracle import dkernel_oracle as O
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 1024, 8, 64) for _ in range(3))
    bm = O.block_mask(8, 1024, 64, 4, 4)
    dense = O.token_mask(bm, 64, 1024, 1024)
    cores = torch.get_num_threads()
    flops = int(bm.sum()) * 4.0 * 64 * 64 * 64

    def best_of(budget):
        O.masked_dense_attention(q, k, v, dense, 0.125, seq_dim=1)
        best, t_start, n = float("inf"), time.time(), 0
        while n < 5 or (time.time() - t_start < 2.0 and n < 50):
            t0 = time.perf_counter()
            O.masked_dense_attention(q, k, v, dense, 0.125, seq_dim=1)
            best = min(best, time.perf_counter() - t0)
            n += 1
            if time.time() - t_start > budget:
                break
        return best, n

    best, n = best_of(max_seconds * 0.6)
    torch.set_num_threads(1)
    best1, n1 = best_of(max_seconds * 0.4)
    torch.set_num_threads(cores)
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "value_1thread": flops / best1 / 1e12,
            "sample": f"BASELINE config 1 (B1,S1024,H8,D64,fp32, block 64, local 4, stride 4), "
                      f"masked-dense oracle, best of {n} runs = {best * 1e3:.2f} ms on {cores} threads, "
                      f"best of {n1} = {best1 * 1e3:.2f} ms on 1 thread"}


def _free():
    import gc
    gc.collect()
    torch.cuda.empty_cache()


def tensor_roofline(tflops, kernel, traffic=None, source=None):
    peaks = measured_peaks()
    r = {"bound": "tensor", "achieved": tflops, "peak": peaks["tflops"], "unit": "TFLOP/s",
         "frac": tflops / peaks["tflops"], "traffic": traffic,
         "peak_source": peaks["source"] + " (burst)",
         "frac_of_sustained": tflops / peaks["tflops_sustained"] if peaks["tflops_sustained"] else None,
         "frac_of_nominal_2250": tflops / NOMINAL_BF16_TFLOPS, "kernel": kernel}
    if traffic is not None:
        r["traffic_source"] = source or "ncu capture of the same workload, not measured in this run"
    return r


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, taken
# from ncu captures of the same full-size workloads on one GPU; None = not captured.
# train: dK/dV 3035.4 MB + dQ 2477.2 MB with the dS hand-over, 2 x 2.19 GB of which is the dS scratch
# written and read back (the roofline line covers both backward kernels); the recompute route moves
# 796.7 + 664.6 MB.
TRAFFIC = {"prefill": 670.8e6, "train": 3035.4e6 + 2477.2e6, "decode": 406.3e6, "varlen": 1249.4e6}


def run_prefill(args, world, rank, strong=False, with_e2e=True):
    """BASELINE config 2.  strong=False: 4 sequences per GPU, heads sharded (weak scaling, the
    headline); strong=True: the one-GPU problem (B=4) with its heads split over the ranks."""
    from dkernel_b200 import LocalStrideSparseAttention, _lib
    from dkernel_b200.dist import head_shard
    cfg = WORKLOADS["prefill"]
    B, S, Hq, Hkv, D = cfg["B"] * (1 if strong else world), cfg["S"], cfg["Hq"], cfg["Hkv"], cfg["D"]
    (h0, h1), (kv0, kv1) = head_shard(Hq, Hkv, rank, world)
    hq_l, hkv_l = h1 - h0, kv1 - kv0
    attn = LocalStrideSparseAttention(Hq, S, cfg["block"], cfg["local"], cfg["stride"], num_kv_heads=Hkv,
                                      active_head_range=(h0, h1) if world > 1 else None, seq_dim=1)
    g = torch.Generator().manual_seed(1234 + rank)
    hq_host = torch.randn((B, S, hq_l, D), generator=g).to(torch.bfloat16)
    hk_host = torch.randn((B, S, hkv_l, D), generator=g).to(torch.bfloat16)
    hv_host = torch.randn((B, S, hkv_l, D), generator=g).to(torch.bfloat16)
    if with_e2e:
        hq_host, hk_host, hv_host = hq_host.pin_memory(), hk_host.pin_memory(), hv_host.pin_memory()
    q, k, v = hq_host.cuda(), hk_host.cuda(), hv_host.cuda()
    scale = 1.0 / math.sqrt(D)
    mask = local_stride_mask_np(Hq, S, cfg["block"], cfg["local"], cfg["stride"], Hkv)[h0:h1]
    tiles = int(mask.sum()) * B
    flops = tiles * tile_flops(cfg["block"], D)

    def step():
        with torch.no_grad():
            attn(q, k, v, sm_scale=scale, return_lse=True)

    ms_max, spread, clocks, ms = timed(step, args.steps, args.warmup, world)
    assert _lib.wait_status() == 0, "a device-side wait gave up: results invalid"
    flops_all = sum_over_ranks(flops, world)
    kernel_tflops = flops / (ms * 1e-3) / 1e12
    if strong:
        return {"ms": ms_max, "tflops": flops_all / (ms_max * 1e-3) / 1e12, "B": B, "scaling": "strong",
                "tiles": int(round(flops_all / tile_flops(cfg["block"], D))), **spread,
                "sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}

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
                   "l2": "inputs (q 256 MiB + k,v 64 MiB each per GPU) exceed the 126 MB L2",
                   "timing": f"median of {spread['repeats']} regions of {args.steps} steps",
                   **spread},
        "gpu_launches": args.steps,
        "clocks": clocks,
        "roofline": {**tensor_roofline(kernel_tflops, "fwd_persist_kernel<bf16,128>", TRAFFIC.get("prefill")),
                     "kernel_ms": ms},
    }
    if not with_e2e:
        return line

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
    ms_e2e, _ = time_steps(step_e2e, e2e_steps, 3, world, repeats=3)
    ms_e2e_max = max_over_ranks(ms_e2e, world)
    line["e2e"] = {"value": flops_all / (ms_e2e_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                   "ms_per_step": ms_e2e_max, "steps_per_region": e2e_steps,
                   "pipeline": f"chunked prefill, {chunk} query rows per module call, copies overlapped",
                   "host_cores_bound": getattr(args, "bound_cpus", None),
                   "h2d_bytes_per_step": (hq_host.numel() + hk_host.numel() + hv_host.numel()) * 2,
                   "d2h_bytes_per_step": out_host.numel() * 2 + lse_host.numel() * 4}
    return line


def run_train(args, world, rank):
    from dkernel_b200 import LocalStrideSparseAttention, _lib
    from dkernel_b200.dist import head_shard
    cfg = WORKLOADS["train"]
    B, S, Hq, D = cfg["B"] * world, cfg["S"], cfg["Hq"], cfg["D"]
    (h0, h1), _ = head_shard(Hq, Hq, rank, world)
    hl = h1 - h0
    attn = LocalStrideSparseAttention(Hq, S, cfg["block"], cfg["local"], cfg["stride"],
                                      active_head_range=(h0, h1) if world > 1 else None, seq_dim=1)
    g = torch.Generator(device="cuda").manual_seed(99 + rank)
    q, k, v, do = (torch.randn((B, S, hl, D), generator=g, device="cuda").to(torch.bfloat16) for _ in range(4))
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

    ms_fwd, _, _, _ = timed(step_fwd, args.steps, args.warmup, world)
    ms, spread, clocks, _ = timed(step, args.steps, args.warmup, world)
    assert _lib.wait_status() == 0
    total = sum_over_ranks(fwd_flops * 3.5, world)
    bwd_ms = ms - ms_fwd
    # which backward route ran: with an affordable scratch the dK/dV kernel hands dS to the dQ kernel
    # (5 products per attended block), otherwise dQ recomputes S and dP (7)
    import dkernel_b200.ops as _ops
    ds_bytes = B * hl * attn._plan().max_head_nnz() * 8192
    handover = 0 < ds_bytes <= _ops._DS_WS_MAX_BYTES
    bwd_tflops = sum_over_ranks(fwd_flops * 2.5, world) / world / (bwd_ms * 1e-3) / 1e12
    return {
        "metric": METRIC, "value": total / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "train fwd+bwd: BASELINE config 3, B=%d (2 per GPU), S=8192, H=32, D=128, "
                               "block 64, local 32, stride 8; FLOPs = 3.5 x forward (5 backward GEMMs, "
                               "recomputation not counted)" % B,
                   "fwd_ms": ms_fwd, "bwd_ms": bwd_ms, **spread,
                   "fwd_tflops": sum_over_ranks(fwd_flops, world) / world / (ms_fwd * 1e-3) / 1e12,
                   "executed_products_per_block": 5 if handover else 7, "algorithmic_products_per_block": 5,
                   "ds_handover_scratch_bytes": ds_bytes if handover else 0},
        "gpu_launches": args.steps * 4, "clocks": clocks,
        "roofline": tensor_roofline(bwd_tflops, "bwd_dkdv_sm100_kernel + %s (+ delta pre-pass)" %
                                    ("bwd_dq_from_ds_kernel" if handover else "bwd_dq_sm100_kernel"),
                                    TRAFFIC.get("train") if handover else 796.7e6 + 664.6e6),
    }


def decode_lens(cfg):
    g = torch.Generator().manual_seed(0)
    return torch.randint(1024, 8193, (cfg["B"],), generator=g)


def attended_kv_tokens(lens, mask_kv, block):
    """sum over sequences and kv heads of the real tokens in attended blocks."""
    total = 0
    for L in lens.tolist():
        row = (L - 1) // block
        for h in range(mask_kv.shape[0]):
            cols = np.nonzero(mask_kv[h, row])[0]
            total += int(np.minimum((cols + 1) * block, L).sum() - (cols * block).sum())
    return total


def _graph_of(calls, n):
    """Capture `n` consecutive calls of `calls()` in one CUDA graph (after running them once)."""
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(n):
            calls()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(n):
                calls()
    torch.cuda.synchronize()
    return graph


def run_decode(args, world, rank):
    """BASELINE config 4.  One GPU: the module call (decode kernel + split merge), timed as a
    replayed CUDA graph and as eager calls.  N > 1: every sequence's KV sharded over the ranks;
    the merged result of both exchange routes is checked against the one-GPU decode of the same
    cache on every rank before anything is timed."""
    from dkernel_b200 import LocalStrideSparseAttention, _lib
    from dkernel_b200.dist import (ShardedDecoder, kv_shard_ranges, pack_kv_shard, pack_kv_shard_cyclic,
                                   sharded_decode)
    cfg = dict(WORKLOADS["decode"])
    if getattr(args, "decode_batch", 0):
        cfg["B"] = args.decode_batch        # a smaller batch of the same shapes (profiler captures)
    B, S, Hq, Hkv, D, bs = cfg["B"], cfg["S"], cfg["Hq"], cfg["Hkv"], cfg["D"], cfg["block"]
    lens = decode_lens(cfg)
    attn = LocalStrideSparseAttention(Hq, S, bs, cfg["local"], cfg["stride"], num_kv_heads=Hkv, seq_dim=1)
    g = torch.Generator(device="cuda").manual_seed(7)      # the same stream of numbers on every rank
    q = torch.randn((B, 1, Hq, D), generator=g, device="cuda").to(torch.bfloat16)
    mask_kv = local_stride_mask_np(Hq, S, bs, cfg["local"], cfg["stride"], Hkv)[::Hq // Hkv]
    tokens = attended_kv_tokens(lens, mask_kv, bs)
    bytes_alg = tokens * D * 2 * 2 + 2 * B * Hq * D * 2
    scale = 1.0 / math.sqrt(D)
    left = (S - lens).to(torch.int32).cuda()
    steps = max(4, args.steps // 4 * 4)
    rec = {"algorithmic_bytes_per_step": bytes_alg, "steps": steps}
    peaks = measured_peaks()

    def make_kv():
        return (torch.randn((B, S, Hkv, D), generator=g, device="cuda").to(torch.bfloat16),
                torch.randn((B, S, Hkv, D), generator=g, device="cuda").to(torch.bfloat16))

    if world == 1:
        nbuf = 4                               # rotate K/V buffers so the L2 never holds the next step's data
        bufs = [make_kv() for _ in range(nbuf)]
        it = [0]

        def eager_step():
            k, v = bufs[it[0] % nbuf]
            it[0] += 1
            with torch.no_grad():
                attn(q, k, v, sm_scale=scale, left_paddings=left, return_lse=True)

        ms_eager, _, _, _ = timed(eager_step, steps, args.warmup, world)
        it[0] = 0
        graph = _graph_of(eager_step, nbuf)

        def graph_step():
            if it[0] % nbuf == 0:
                graph.replay()
            it[0] += 1
        it[0] = 0
        ms, spread, clocks, _ = timed(graph_step, steps, args.warmup, world)
        # the same step against an e4m3 K/V cache (per-tensor scales): half the K/V bytes
        us_fp8 = gbs_fp8 = None
        if hasattr(torch, "float8_e4m3fn") and not getattr(args, "no_fp8", False):
            ksc = vsc = 6.0 / 448.0              # N(0,1) data: |x| < 6
            bufs8 = [((k.float() / ksc).to(torch.float8_e4m3fn), (v.float() / vsc).to(torch.float8_e4m3fn))
                     for k, v in bufs]

            def fp8_step():
                k, v = bufs8[it[0] % nbuf]
                it[0] += 1
                with torch.no_grad():
                    attn(q, k, v, sm_scale=scale, left_paddings=left, return_lse=True, kv_scales=(ksc, vsc))
            it[0] = 0
            graph8 = _graph_of(fp8_step, nbuf)

            def graph8_step():
                if it[0] % nbuf == 0:
                    graph8.replay()
                it[0] += 1
            it[0] = 0
            ms8, _, _, _ = timed(graph8_step, steps, args.warmup, world)
            us_fp8 = ms8 * 1e3
            gbs_fp8 = (tokens * D * 2 + 2 * B * Hq * D * 2) / (ms8 * 1e-3) / 1e9
            del bufs8
        assert _lib.wait_status() == 0
        gbs = bytes_alg / (ms * 1e-3) / 1e9
        rec.update({"us_graph": ms * 1e3, "us_eager": ms_eager * 1e3, "us_graph_e4m3_kv": us_fp8,
                    "gbs_e4m3_kv": gbs_fp8, "hbm_frac_e4m3_kv": gbs_fp8 / peaks["hbm"] if gbs_fp8 else None, "gbs": gbs, "hbm_frac": gbs / peaks["hbm"],
                    "hbm_frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS, **spread,
                    "launch": f"CUDA graph of {nbuf} module calls (one per K/V buffer set) replayed; "
                              "us_eager = the same calls made from Python",
                    "l2": f"{nbuf} K/V buffer sets rotated ({nbuf}x{2 * B * S * Hkv * D * 2 / 2**20:.0f} MiB)",
                    "sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons"), "launches_per_step": 2})
        return rec, ms, clocks, gbs

    # ---- N > 1: shards of ONE seeded cache (identical on every rank), checked, then timed
    k_full, v_full = make_kv()
    with torch.no_grad():
        ref_o, ref_lse = attn(q, k_full, v_full, sm_scale=scale, left_paddings=left, return_lse=True)
    # Two shard layouts of the same cache: block-cyclic (block j of a sequence on rank j % N: the
    # 16-block local window spreads evenly) and contiguous position ranges (it stays on the last rank).
    cap = int(((S // world + bs - 1) // bs + 1) * bs)
    lens_d = lens.cuda()
    ks, vs, n = pack_kv_shard_cyclic(k_full, v_full, left, lens_d, rank, world, bs, capacity=cap)
    lo, hi = kv_shard_ranges(lens, rank, world, bs)
    ks2, vs2, n2 = pack_kv_shard(k_full, v_full, left.cpu(), lo, hi, capacity=cap)
    del k_full, v_full
    n_d, len_d = n.to(torch.int32).cuda(), lens.to(torch.int32).cuda()
    n2_d, lo_d = n2.to(torch.int32).cuda(), lo.to(torch.int32).cuda()
    dec, dec_err = None, ""
    try:
        dec = ShardedDecoder(attn, B, Hq, D, torch.bfloat16, torch.device("cuda", torch.cuda.current_device()))
    except Exception as e:      # no symmetric memory in this setup: only the all-gather route is timed
        dec_err = f"{type(e).__name__}: {e}"[:200]
    flag = torch.tensor([1.0 if dec is not None else 0.0], device="cuda")
    torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
    if flag.item() == 0.0:
        dec = None
        rec["xchg_unavailable"] = dec_err or "failed on another rank"
    routes = []
    with torch.no_grad():
        if dec is not None:
            routes.append(("xchg",) + tuple(dec.step(q, ks, vs, n_d, None, len_d, scale, cyclic=True)))
            routes.append(("xchg_contig",) + tuple(dec.step(q, ks2, vs2, n2_d, lo_d, len_d, scale)))
        routes.append(("nccl",) + tuple(sharded_decode(attn, q, ks, vs, n_d, None, len_d, scale, cyclic=True)))
    torch.cuda.synchronize()
    assert _lib.wait_status() == 0, "a bounded wait gave up"
    errs = {}
    for name, o, l in routes:
        e_o = (o.float() - ref_o.float()).abs().max().item()
        e_l = (l - ref_lse.reshape(B, Hq)).abs().max().item()
        assert e_o <= 2e-2 and e_l <= 1e-3, f"KV-sharded decode ({name}) differs from the one-GPU decode: {e_o} {e_l}"
        errs[name] = (e_o, e_l)
    rec.update({"check_max_abs_out": max(e[0] for e in errs.values()),
                "check_max_abs_lse": max(e[1] for e in errs.values()), "check": "vs one-GPU decode of the same cache"})
    # the second buffer set holds other random shards of the same geometry
    bufs = [(ks, vs), (torch.randn(ks.shape, generator=g, device="cuda").to(torch.bfloat16),
                       torch.randn(vs.shape, generator=g, device="cuda").to(torch.bfloat16))]
    bufs2 = [(ks2, vs2), bufs[1]]
    nbuf = len(bufs)
    it = [0]

    def step_xchg():
        a, b_ = bufs[it[0] % nbuf]
        it[0] += 1
        with torch.no_grad():
            dec.step(q, a, b_, n_d, None, len_d, scale, cyclic=True)

    def step_contig():
        a, b_ = bufs2[it[0] % nbuf]
        it[0] += 1
        with torch.no_grad():
            dec.step(q, a, b_, n2_d, lo_d, len_d, scale)

    def step_nccl():
        a, b_ = bufs[it[0] % nbuf]
        it[0] += 1
        with torch.no_grad():
            sharded_decode(attn, q, a, b_, n_d, None, len_d, scale, cyclic=True)

    results = {}
    for name, fn in ((("xchg", step_xchg), ("xchg_contig", step_contig)) if dec is not None else ()) + \
            (("nccl", step_nccl),):
        it[0] = 0
        mode = "graph"
        try:
            graph = _graph_of(fn, nbuf)

            def gstep(graph=graph):
                if it[0] % nbuf == 0:
                    graph.replay()
                it[0] += 1
            run = gstep
        except Exception as e:     # capture unsupported in this setup: time the eager calls
            mode, run = f"eager ({type(e).__name__}: {str(e)[:80]})", fn
        flag = torch.tensor([1.0 if mode == "graph" else 0.0], device="cuda")
        torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
        if flag.item() == 0.0 and mode == "graph":
            mode, run = "eager (capture failed on another rank)", fn
        it[0] = 0
        ms, spread, clocks, _ = timed(run, steps, args.warmup, world)
        results[name] = (ms, spread, clocks, mode)
    assert _lib.wait_status() == 0
    ms, spread, clocks, mode = results["xchg" if dec is not None else "nccl"]
    gbs = bytes_alg / world / (ms * 1e-3) / 1e9
    rec.update({"us_xchg": ms * 1e3 if dec is not None else None, "us_nccl": results["nccl"][0] * 1e3,
                "us_xchg_contiguous_shards": results["xchg_contig"][0] * 1e3 if dec is not None else None,
                "mode_xchg": mode if dec is not None else None,
                "mode_nccl": results["nccl"][3], "gbs_per_gpu": gbs, **spread,
                "exchange": "xchg = peer-store exchange + merge kernel (bsa_xchg_merge); "
                            "nccl = one all-gather + merge kernel; KV shards block-cyclic unless named",
                "sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons"), "launches_per_step": 3})
    return rec, ms, clocks, gbs


def decode_line(args, world, rank):
    rec, ms, clocks, gbs = run_decode(args, world, rank)
    peaks = measured_peaks()
    return {
        "metric": "sparse_attn_decode_us_per_step", "value": ms * 1e3, "unit": "us", "n_gpus": world,
        "steps": rec["steps"], "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "decode: BASELINE config 4, B=64, one query token, Hq=32, Hkv=8, D=128, KV lengths "
                               "U[1024,8192] left-padded to 8192, block 64, local 16, stride 8",
                   "parallelism": "single GPU" if world == 1 else
                   f"KV sequence sharded over {world} GPUs, peer-store exchange + merge kernel", **rec},
        "gpu_launches": rec["steps"] * rec["launches_per_step"], "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm"], "traffic": TRAFFIC.get("decode"),
                     "traffic_source": "ncu capture of the same workload, not measured in this run",
                     "peak_source": peaks["source"], "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS,
                     "kernel": "decode_kernel<bf16,128> (+ merge_kernel)", "per_gpu": True},
    }


def varlen_problem(cfg):
    H, bs = cfg["H"], cfg["block"]
    nb = cfg["max_seq"] // bs
    g = torch.Generator().manual_seed(0)
    pat = torch.rand((H, nb, nb), generator=g) < cfg["p"]
    pat |= torch.eye(nb, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
    lens = torch.randint(cfg["lo"], cfg["hi"] + 1, (cfg["nseq"],), generator=g)
    return pat, lens


def run_varlen(args, world, rank):
    """BASELINE config 5 (fixed problem; at N > 1 its 32 heads are split over the ranks)."""
    from dkernel_b200 import SparseAttention, _lib
    from dkernel_b200.dist import head_shard
    import warnings
    cfg = WORKLOADS["varlen"]
    H, D, bs = cfg["H"], cfg["D"], cfg["block"]
    pat, lens = varlen_problem(cfg)
    (h0, h1), _ = head_shard(H, H, rank, world)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        attn = SparseAttention(bs, pat[h0:h1].cuda())
    T = int(lens.sum())
    g = torch.Generator(device="cuda").manual_seed(3 + rank)
    q, k, v = (torch.randn((T, h1 - h0, D), generator=g, device="cuda").to(torch.bfloat16) for _ in range(3))
    cu = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)]).to(torch.int32).cuda()
    tiles = executed = 0
    pn = pat[h0:h1].numpy()
    for L in lens.tolist():
        n = (L + bs - 1) // bs
        sub = pn[:, :n, :n]
        tiles += int(sub.sum())
        # a 128-row tile = two adjacent row blocks walking the union of their lists
        even, odd = sub[:, 0::2], sub[:, 1::2]
        if odd.shape[1] < even.shape[1]:
            odd = np.concatenate([odd, np.zeros_like(even[:, :1])], 1)
        executed += 2 * int((even | odd).sum())
    flops = tiles * tile_flops(bs, D)

    def step():
        with torch.no_grad():
            attn(q, k, v, cu_seqlen_k=cu)

    ms_max, spread, clocks, ms = timed(step, args.steps, args.warmup, world)
    assert _lib.wait_status() == 0
    total = sum_over_ranks(flops, world)
    tf = flops / (ms * 1e-3) / 1e12
    ratio = sum_over_ranks(executed, world) / max(sum_over_ranks(tiles, world), 1)
    return {
        "metric": METRIC, "value": total / (ms_max * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_max, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "varlen prefill, user pattern: BASELINE config 5, H=32, D=128, block 64, "
                               "Bernoulli(0.2) lower-triangular 256x256 pattern, 16 packed sequences "
                               f"U[512,4096] (sum {T} tokens)",
                   "parallelism": f"heads sharded over {world} GPU(s)", "attended_tiles": int(total / tile_flops(bs, D)),
                   "executed_over_attended": ratio, **spread},
        "gpu_launches": args.steps, "clocks": clocks,
        "roofline": tensor_roofline(tf, "fwd_persist_kernel<bf16,128>", TRAFFIC.get("varlen")),
    }


def run_fwd_d64(args, world, rank):
    """Head dim 64 on the tensor-core forward: config 2's pattern and sizes with D = 64."""
    from dkernel_b200 import LocalStrideSparseAttention, _lib
    cfg = WORKLOADS["prefill"]
    B, S, Hq, Hkv, D = cfg["B"], cfg["S"], cfg["Hq"], cfg["Hkv"], 64
    attn = LocalStrideSparseAttention(Hq, S, cfg["block"], cfg["local"], cfg["stride"], num_kv_heads=Hkv, seq_dim=1)
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn((B, S, Hq, D), generator=g, device="cuda").to(torch.bfloat16)
    k, v = (torch.randn((B, S, Hkv, D), generator=g, device="cuda").to(torch.bfloat16) for _ in range(2))
    tiles = int(local_stride_mask_np(Hq, S, cfg["block"], cfg["local"], cfg["stride"], Hkv).sum()) * B
    flops = tiles * tile_flops(cfg["block"], D)

    def step():
        with torch.no_grad():
            attn(q, k, v, return_lse=True)

    ms_max, spread, clocks, ms = timed(step, args.steps, args.warmup, 1)
    assert _lib.wait_status() == 0
    tf = flops / (ms * 1e-3) / 1e12
    return {"ms": ms, "tflops": tf, "frac": tf / measured_peaks()["tflops"], **spread,
            "shape": "B4 S8192 Hq32 Hkv8 D64 bf16, config 2's pattern", "sm_mhz": clocks.get("sm_mhz")}


def run_ring(args, world, rank):
    """Context-parallel training step (N > 1): BASELINE config 3's problem (B=2, S=8192, H=32, D=128) with
    the SEQUENCE split over the ranks (ring attention, zig-zag split: K/V chunks round the ring over NCCL
    send/recv, LSE merge, dK/dV contributions sent to the chunk owner); fixed total size ("strong")."""
    from dkernel_b200 import _lib
    from dkernel_b200.dist import ContextParallelSparseAttention
    cfg = WORKLOADS["train"]
    B, S, H, D = cfg["B"], cfg["S"], cfg["Hq"], cfg["D"]
    # zig-zag split: rank r holds pieces r and 2 * world - 1 - r of the sequence, so that every rank
    # has the same share of the causal mask
    cp = ContextParallelSparseAttention(H, S, cfg["block"], cfg["local"], cfg["stride"], seq_dim=1, zigzag=True)
    g = torch.Generator(device="cuda").manual_seed(99 + rank)
    q, k, v, do = (torch.randn((B, S // world, H, D), generator=g, device="cuda").to(torch.bfloat16)
                   for _ in range(4))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()

    def step():
        q.grad = k.grad = v.grad = None
        cp(q, k, v).backward(do)

    def step_fwd():
        with torch.no_grad():
            cp(q, k, v)

    steps = max(2, args.steps // 4)
    # the full step first: its warm-up also sets up the point-to-point connections and the allocator's pools
    ms, spread, clocks, _ = timed(step, steps, 5, world, repeats=3)
    ms_fwd, _, _, _ = timed(step_fwd, steps, 5, world, repeats=3)
    assert _lib.wait_status() == 0
    tiles = int(local_stride_mask_np(H, S, cfg["block"], cfg["local"], cfg["stride"], H).sum()) * B
    flops = tiles * tile_flops(cfg["block"], D) * 3.5
    return {"ms": ms, "fwd_ms": ms_fwd, "tflops": flops / (ms * 1e-3) / 1e12, "steps": steps, **spread,
            "sm_mhz": clocks.get("sm_mhz")}


def compact(line, keys=()):
    """A sub-record of the combined line: numbers only, no prose."""
    c = line["config"]
    rec = {"ms": line["ms_per_step"], "value": line["value"], "unit": line["unit"],
           "frac": line["roofline"]["frac"], "achieved": line["roofline"]["achieved"],
           "sm_mhz": line["clocks"].get("sm_mhz"), "reasons": line["clocks"].get("reasons"),
           "clock_samples": line["clocks"].get("samples")}
    for k in ("fwd_ms", "bwd_ms", "fwd_tflops", "ms_min", "ms_max", "repeats", "executed_over_attended",
              "attended_tiles", "executed_products_per_block", "algorithmic_products_per_block",
              "ds_handover_scratch_bytes") + tuple(keys):
        if k in c:
            rec[k] = c[k]
    return rec


def run_all(args, world, rank):
    """The headline (config 2 prefill) plus the rest of the metric as sub-records.  A sub-workload
    that fails is reported as {"error": ...} in its place; the headline still prints."""
    line = run_prefill(args, world, rank)
    sub, rsub = {}, {}

    def guarded(name, fn):
        _free()
        try:
            fn()
        except Exception as e:      # keep the line; the failure is visible in the record
            sub[name] = {"error": f"{type(e).__name__}: {e}"[:300]}

    def train():
        t = run_train(args, world, rank)
        sub["train_c3"] = compact(t)
        rsub["train_bwd"] = {"achieved": t["roofline"]["achieved"], "frac": t["roofline"]["frac"],
                             "frac_of_sustained": t["roofline"]["frac_of_sustained"], "unit": "TFLOP/s"}

    def decode():
        rec, ms, clocks, gbs = run_decode(args, world, rank)
        name = "decode_c4" if world == 1 else "decode_c4_kv_sharded"
        sub[name] = {k: v for k, v in rec.items() if not isinstance(v, str) or k.startswith("mode_")
                     or k == "xchg_unavailable"}
        if world == 1:
            rsub["decode"] = {"achieved": gbs, "frac": rec["hbm_frac"], "unit": "GB/s", "bound": "hbm"}

    def varlen():
        vl = run_varlen(args, world, rank)
        sub["varlen_c5" if world == 1 else "varlen_c5_strong"] = compact(vl)
        if world == 1:
            rsub["varlen"] = {"achieved": vl["roofline"]["achieved"], "frac": vl["roofline"]["frac"],
                              "unit": "TFLOP/s"}

    def d64():
        r = run_fwd_d64(args, world, rank)
        sub["prefill_d64"] = {k: v for k, v in r.items() if not isinstance(v, str)}
        rsub["prefill_d64"] = {"achieved": r["tflops"], "frac": r["frac"], "unit": "TFLOP/s"}

    def prefill_strong():
        r = run_prefill(args, world, rank, strong=True, with_e2e=False)
        sub["prefill_c2_strong"] = {k: v for k, v in r.items() if not isinstance(v, (str, list))}

    def reference_triton():
        # optional comparator in a child process (Triton JIT; bounded): the reference's own kernels, same GPU
        if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "dkernel")):
            sub["reference_triton_c2"] = {"unavailable": "baseline/_ref not installed"}
            return
        try:
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu", "--steps",
                                str(args.steps), "--warmup", str(args.warmup)], capture_output=True, text=True,
                               timeout=300, cwd=ROOT)
            ref = json.loads(r.stdout.strip().splitlines()[-1])
        except Exception as e:
            ref = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        if "value" in ref:
            sub["reference_triton_c2"] = {"tflops": ref["value"], "ms": ref["ms_per_step"],
                                          "max_abs_diff_vs_this_repo": ref.get("max_abs_diff_vs_this_repo"),
                                          "speedup_of_this_repo": line["value"] / ref["value"]}
        else:
            sub["reference_triton_c2"] = {"unavailable": str(ref.get("unavailable"))[:200]}

    if world == 1:
        for name, fn in (("train_c3", train), ("decode_c4", decode), ("varlen_c5", varlen), ("prefill_d64", d64),
                         ("reference_triton_c2", reference_triton)):
            guarded(name, fn)

    def ring():
        sub["train_c3_ring"] = run_ring(args, world, rank)

    if world > 1:
        for name, fn in (("decode_c4_kv_sharded", decode), ("varlen_c5_strong", varlen),
                         ("prefill_c2_strong", prefill_strong), ("train_c3_ring", ring)):
            guarded(name, fn)
    _free()
    line["config"]["sub"] = sub
    line["roofline"]["sub"] = rsub
    return line


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
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "prefill_fwd: BASELINE config 2 (Phi-3-small shape) -- " + sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if getattr(args, "steps_requested", args.steps) != args.steps:
        line["config"]["steps_clamped_from"] = args.steps_requested
    return line


def run_reference_gpu(args):
    """Optional comparator, bench side only: the UNMODIFIED reference (installed under baseline/_ref)
    running its own Triton kernels on this GPU, BASELINE config 2 forward.  Its training-path kernel
    indexes K/V with the q-head id (dkernel/ops/sparse_attn_fwd.py:217-218), so K/V are repeated to
    32 heads as its callers must.  Prints one JSON line; any failure is reported in the line."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    line = {"impl": "reference-gpu", "metric": METRIC, "unit": "TFLOP/s", "n_gpus": 1, "dtype": "bf16",
            "data": "synthetic", "higher_is_better": True, "steps": args.steps, "warmup": args.warmup}
    try:
        if not os.path.isdir(os.path.join(ref_dir, "dkernel")):
            raise RuntimeError("baseline/_ref is missing (pip install --no-deps --target baseline/_ref of the reference)")
        sys.path.insert(0, ref_dir)
        import dkernel as ref
        cfg = WORKLOADS["prefill"]
        B, S, Hq, Hkv, D = cfg["B"], cfg["S"], cfg["Hq"], cfg["Hkv"], cfg["D"]
        torch.cuda.set_device(0)
        attn = ref.LocalStrideSparseAttention(Hq, S, cfg["block"], cfg["local"], cfg["stride"], num_kv_heads=Hkv,
                                              seq_dim=1)
        attn = attn.cuda() if hasattr(attn, "cuda") else attn
        g = torch.Generator(device="cuda").manual_seed(1234)
        q = torch.randn((B, S, Hq, D), generator=g, device="cuda").to(torch.bfloat16)
        k, v = (torch.randn((B, S, Hkv, D), generator=g, device="cuda").to(torch.bfloat16) for _ in range(2))
        kr, vr = k.repeat_interleave(Hq // Hkv, dim=2), v.repeat_interleave(Hq // Hkv, dim=2)
        scale = 1.0 / math.sqrt(D)

        def step():
            with torch.no_grad():
                return attn(q, kr, vr, sm_scale=scale)

        out = step()
        torch.cuda.synchronize()
        # same inputs through this repository's kernels: the comparator must compute the same thing
        from dkernel_b200 import LocalStrideSparseAttention
        mine = LocalStrideSparseAttention(Hq, S, cfg["block"], cfg["local"], cfg["stride"], num_kv_heads=Hkv, seq_dim=1)
        with torch.no_grad():
            want = mine(q, k, v, sm_scale=scale)
        line["max_abs_diff_vs_this_repo"] = (out.float() - want.float()).abs().max().item()
        ms, regions = time_steps(step, args.steps, max(args.warmup, 3), 1)
        tiles = int(local_stride_mask_np(Hq, S, cfg["block"], cfg["local"], cfg["stride"], Hkv).sum()) * B
        line.update({"value": tiles * tile_flops(cfg["block"], D) / (ms * 1e-3) / 1e12, "ms_per_step": ms,
                     "ms_min": min(regions), "ms_max": max(regions),
                     "config": {"workload": "prefill_fwd: BASELINE config 2, the reference's Triton kernels on this GPU "
                                            "(K/V repeated to 32 heads, as that kernel requires)"}})
        import triton
        line["triton"] = triton.__version__
    except Exception as e:
        line["unavailable"] = f"{type(e).__name__}: {e}"[:300]
    return line


def main():
    global REPEATS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--workload", default="all", choices=["all"] + list(WORKLOADS))
    ap.add_argument("--repeats", type=int, default=REPEATS, help="timed regions of K steps each (median reported)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--decode-batch", type=int, default=0,
                    help="decode: sequences per step instead of config 4's 64 (small case for profiler captures)")
    ap.add_argument("--no-fp8", action="store_true", help="decode: skip the e4m3 K/V measurement")
    ap.add_argument("--e2e-chunk", type=int, default=E2E_CHUNK,
                    help="prefill: query rows per pipelined chunk of the end-to-end step")
    ap.add_argument("--bwd-route", choices=["auto", "recompute"], default="auto",
                    help="train: 'recompute' gives the backward no dS scratch, so that dQ recomputes S and dP")
    args = ap.parse_args()
    if args.bwd_route == "recompute":
        import dkernel_b200.ops as _ops
        _ops._DS_WS_MAX_BYTES = 0
    if args.impl == "reference":
        # a step takes ~0.2 s of host time: bound the run to a few minutes, and say so in the line
        args.steps_requested = args.steps
        args.steps = min(args.steps, 200)
        line = run_reference(args)
        if line is not None:
            print(json.dumps(line), flush=True)
        return
    if args.impl == "reference-gpu":
        if not torch.cuda.is_available():
            print(json.dumps({"impl": "reference-gpu", "unavailable": "no CUDA device"}), flush=True)
            return
        REPEATS = max(1, args.repeats)
        print(json.dumps(run_reference_gpu(args)), flush=True)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path); "
                         "use --impl reference for the CPU restatement")
    REPEATS = max(1, args.repeats)
    args.warmup = max(args.warmup, 3)
    world, rank, _ = setup_dist(args)
    if args.gpus != world and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)
    line = {"all": run_all, "prefill": run_prefill, "train": run_train, "decode": decode_line,
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
