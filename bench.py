#!/usr/bin/env python
"""Benchmark of the two-stage block-sparse attention forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload``): the headline configuration -- B=8, H=32, S=4096, D=128,
bf16, boolean mask [B,1,S,S] built from 32x32 blocks dropped with probability p (diagonal
blocks kept, 10 % of kept blocks internally Bernoulli(0.5)), swept over
p in {0, 0.1, 0.3, 0.5, 0.7, 0.9}, lists at (BLOCK_Q, BLOCK_K) = (128, 32).  One step is
one pass of the hot path over the whole sweep: for every p, classify the mask
(stage 1) and run the attention forward (stage 2).  With N > 1 GPUs every rank owns its
own (batch, head) shard of that size (weak scaling, no collective on the data path).

Metric: effective TFLOP/s = FLOPs over the non-skipped tiles (4*D*BQ*BK per listed tile)
divided by the time of both stages.  ``value`` is measured with all inputs resident in
HBM; ``e2e`` goes through the public Python entry points with host (pinned) inputs, the
host->device and device->host copies inside the timed region.

``--impl reference`` times the reference's CPU path for the same metric on the host
cores: the C restatement of its classifier plus torch SDPA with the bool mask (its own
ground truth, test_attn.py:40) on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "effective_tflops_attn_plus_mask_preprocess"
UNIT = "TFLOP/s"
BQ, BK = 128, 32
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs
    (NVML through pynvml every 20 ms; nvidia-smi as a fallback).  Read-only."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.sm_max = None
        self._stop = threading.Event()
        self.thread = None
        self.source = None

    def _nvml_loop(self, pynvml, handle):
        while not self._stop.is_set():
            try:
                self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def _smi_loop(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [x.strip() for x in out.strip().split(",")]
                self.samples.append(float(parts[0]))
                self.sm_max = float(parts[1])
                for n, val in zip(names, parts[2:6]):
                    if val.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if visible:
                try:
                    idx = int(visible.split(",")[self.index])
                except ValueError:
                    pass
            handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.source = "nvml"
            self.thread = threading.Thread(target=self._nvml_loop, args=(pynvml, handle), daemon=True)
        except Exception:
            self.source = "nvidia-smi"
            self.thread = threading.Thread(target=self._smi_loop, daemon=True)
        self.thread.start()

    def stop(self):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=10)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.sm_max,
                "samples": len(self.samples), "reasons": sorted(self.reasons), "source": self.source}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------- CPU arm

def cpu_sample(sample_heads: int, steps: int, warmup: int):
    """The reference's CPU path on a bounded sample: one batch element, ``sample_heads`` heads of
    the headline shape, every p of the sweep.  Returns (TFLOP/s, seconds per step, description, cores)."""
    import numpy as np
    import torch.nn.functional as F

    from oracle import cclassify
    import workloads

    cfg = workloads.CONFIGS["headline"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    S, D = cfg.S, cfg.D
    q, k, v = workloads.make_qkv(1, sample_heads, S, D, torch.bfloat16, seed=100)
    masks = [workloads.random_block_mask(1, S, p, cfg.partial_frac, seed=200 + i) for i, p in enumerate(cfg.drop_ps)]
    masks_np = [np.ascontiguousarray(m.numpy()) for m in masks]

    def one_step():
        flops = 0.0
        for m, mn in zip(masks, masks_np):
            md = cclassify.classify(mn, BQ, BK)                               # stage 1 on the host
            F.scaled_dot_product_attention(q, k, v, attn_mask=m)             # test_attn.py:40
            flops += 4.0 * D * BQ * BK * sample_heads * float(md.unmasked_lens.sum() + md.masked_lens.sum())
        return flops

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    flops = 0.0
    for _ in range(steps):
        flops += one_step()
    dt = time.perf_counter() - t0
    desc = (f"B=1, H={sample_heads} of the headline shape (S={S}, D={D}, bf16), all {len(masks)} p values; "
            f"C classifier ({cclassify.threads()} threads) + torch CPU SDPA with the bool mask")
    return flops / dt / 1e12, dt / steps, desc, cores


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    warm = max(1, min(args.warmup, 1))
    val, sec, desc, cores = cpu_sample(args.cpu_heads, steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(), "sample": desc},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name():
    return ("headline: B=8 H=32 S=4096 D=128 bf16, 32x32-block mask [B,1,S,S], drop p in "
            "{0,0.1,0.3,0.5,0.7,0.9}, 10% of kept blocks Bernoulli(0.5), BLOCK_Q=128 BLOCK_K=32, per GPU")


# ------------------------------------------------------------------------------- GPU arm

def run_ours(args):
    import sparseattention_b200 as sa
    import workloads
    from sparseattention_b200 import _native

    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    _native.load_library()        # fail loudly if the CUDA library is missing

    cfg = workloads.CONFIGS[args.workload]
    B, H, S, D = (args.batch or cfg.B), cfg.H, cfg.S, cfg.D
    ps = [float(x) for x in args.ps.split(",")] if args.ps else list(cfg.drop_ps)
    dtype = torch.bfloat16
    warmup = args.warmup if args.profile else max(args.warmup, 3)
    q, k, v = workloads.make_qkv(B, H, S, D, dtype, seed=1000 + rank, device=dev)
    planes = 1 if cfg.mask_batch == 1 else B                    # distinct mask planes (the composed mask is shared)
    masks = [workloads.make_mask(cfg, p, seed=2000 + 17 * rank + i, device=dev, batch=planes)
             for i, p in enumerate(ps)]
    masks_e = [m.expand(B, H, S, S) for m in masks]

    def stage1(i):
        return sa.compute_mask_kernel(masks_e[i], BQ, BK)

    def stage2(i, md):
        return sa.sparse_attention(q, k, v, masks[i], BQ, BK, mask_metadata=md, impl="tcgen05")

    # one untimed pass: FLOP / byte accounting and a device-status check
    flops_p, bytes_p, mix = [], [], []
    for i in range(len(ps)):
        md = stage1(i)
        o = sa.sparse_attention(q, k, v, masks[i], BQ, BK, mask_metadata=md, impl="tcgen05", check_status=True)
        flops_p.append(workloads.computed_tile_flops(md.unmasked_lens, md.masked_lens, BQ, BK, D))
        lens_sum = int(md.unmasked_lens[:, 0].sum()) + int(md.masked_lens[:, 0].sum())
        bytes_p.append(workloads.classifier_bytes(planes, S, S, BQ, lens_sum))
        tiles = B * H * (S // BQ) * (S // BK)
        mix.append((float(md.unmasked_lens.sum()) / tiles, float(md.masked_lens.sum()) / tiles))
        del o, md
    flops_step = sum(flops_p)

    n_p = len(ps)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2 * n_p + 1)] for _ in range(args.steps)]

    def step(events=None):
        if events is not None:
            events[0].record()
        for i in range(n_p):
            md = stage1(i)
            if events is not None:
                events[2 * i + 1].record()
            o = stage2(i, md)
            if events is not None:
                events[2 * i + 2].record()
        return o

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record()
    for s in range(args.steps):
        step(ev[s])
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = t_start.elapsed_time(t_end)

    cls_ms = [statistics.mean(ev[s][2 * i].elapsed_time(ev[s][2 * i + 1]) for s in range(args.steps)) for i in range(n_p)]
    att_ms = [statistics.mean(ev[s][2 * i + 1].elapsed_time(ev[s][2 * i + 2]) for s in range(args.steps)) for i in range(n_p)]

    # ---- end to end through the public entry points with host buffers
    if args.profile or args.workload != "headline":
        if world > 1:
            torch.distributed.destroy_process_group()
        if rank == 0:
            print(json.dumps({"profile_run": bool(args.profile), "workload": args.workload, "B": B, "ps": ps,
                              "classify_ms": cls_ms, "attn_ms": att_ms,
                              "attn_tflops": [f / (a * 1e-3) / 1e12 for f, a in zip(flops_p, att_ms)],
                              "classify_gbs": [by / (c * 1e-3) / 1e9 for by, c in zip(bytes_p, cls_ms)],
                              "tile_mix_full_partial": mix,
                              "effective_tflops_both_stages": flops_step / (elapsed_ms / args.steps * 1e-3) / 1e12}))
        return
    host_q, host_k, host_v = (t.cpu().pin_memory() for t in (q, k, v))
    host_masks = [m.cpu().pin_memory() for m in masks]
    host_o = torch.empty((B, H, S, D), dtype=dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (host_q, host_k, host_v)) + sum(m.numel() for m in host_masks)
    d2h = n_p * host_o.numel() * host_o.element_size()

    # Three streams: host->device copies, compute (the caller's current stream), device->host
    # copies; the copies of one mask overlap the kernels of the previous one (PCIe is full duplex).
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def e2e_step():
        # steps are pipelined too: the inputs of a step travel while the results of the previous one
        # are still going back (fresh device buffers per step; the caching allocator tracks the streams)
        with torch.cuda.stream(s_in):
            dq, dk, dv = (t.to(dev, non_blocking=True) for t in (host_q, host_k, host_v))
            dms, ready = [], []
            for i in range(n_p):
                dms.append(host_masks[i].to(dev, non_blocking=True))
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
                ready.append(ev_in)
        for t in (dq, dk, dv, *dms):
            t.record_stream(main)
        for i in range(n_p):
            main.wait_event(ready[i])
            o = sa.sparse_attention(dq, dk, dv, dms[i], BQ, BK)  # the reference's call, stage 1 inside
            done = torch.cuda.Event()
            done.record(main)
            o.record_stream(s_out)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                host_o.copy_(o, non_blocking=True)

    def e2e_drain():
        main.wait_stream(s_in)
        main.wait_stream(s_out)                                  # the last result is on the host

    e2e_steps = max(1, min(args.steps, 5))
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    e2e_step()
    e2e_drain()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    for _ in range(e2e_steps):
        e2e_step()
    e2e_drain()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([elapsed_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms = float(t[0]), float(t[1])
        f = torch.tensor([flops_step], device=dev, dtype=torch.float64)
        dist.all_reduce(f, op=dist.ReduceOp.SUM)
        flops_all = float(f[0])
    else:
        flops_all = flops_step

    if rank == 0:
        peaks, peak_kind = load_peaks()
        ms_per_step = elapsed_ms / args.steps
        value = flops_all / (ms_per_step * 1e-3) / 1e12
        att_total_ms = sum(att_ms)
        att_tflops = flops_step / (att_total_ms * 1e-3) / 1e12
        cls_total_ms = sum(cls_ms)
        cls_gbs = sum(bytes_p) / (cls_total_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(), "l2": "inputs larger than L2 (Q,K,V 768 MiB, each mask 128 MiB)",
                       "flop_accounting": "4*D*BQ*BK per listed (non-skipped) tile, both stages timed",
                       "shard": "each rank owns a full (batch, head) shard of the workload"},
            "roofline": {"bound": "tensor", "achieved": att_tflops, "peak": peaks["bf16_tflops_sustained"],
                         "unit": "TFLOP/s", "frac": att_tflops / peaks["bf16_tflops_sustained"],
                         "traffic": 254.3e6 * B / 2.0, "traffic_unit": "bytes per launch (ncu capture at B=2, p=0.5, scaled by batch)",
                         "kernel": "attn_fwd_tc_kernel<bf16,128>", "peak_source": peak_kind + " (sustained bf16 matmul)",
                         "note": "FLOPs of the listed tiles of all six launches / sum of their durations (CUDA events)"},
            "roofline_classifier": {"bound": "hbm", "achieved": cls_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                    "frac": cls_gbs / peaks["hbm_gbs"], "traffic": 276.7e6 * B / 16.0,
                                    "traffic_unit": "bytes per launch (ncu capture at 16 planes, scaled by planes)",
                                    "kernel": "classify_cells_kernel + compact_lists_kernel",
                                    "note": "algorithmic bytes / duration of the whole stage-1 call incl. its allocations"},
            "sweep": [{"p": p, "classify_ms": c, "attn_ms": a, "attn_tflops": fl / (a * 1e-3) / 1e12,
                       "classify_gbs": by / (c * 1e-3) / 1e9, "full_frac": fm, "partial_frac": pm}
                      for p, c, a, fl, by, (fm, pm) in zip(ps, cls_ms, att_ms, flops_p, bytes_p, mix)],
            "e2e": {"value": flops_all / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": args.steps * n_p * 3,
            "clocks": clocks,
        }
        if world == 1 and args.comparators:
            line["comparators"] = gpu_comparators(q, k, v, masks, ps, flops_p)
        if world == 1 and not args.no_cpu_baseline:
            val, sec, desc, cores = cpu_sample(args.cpu_heads, 1, 1)
            line["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def gpu_comparators(q, k, v, masks, ps, flops_p):
    """Same-box library comparators of the reference's harness (test_attn.py:64): torch SDPA without a
    mask (the vendor's dense kernel) and with the bool mask, timed like the reference times them (CUDA
    events, best of a few runs).  Off by default; the figures are not part of the metric."""
    import torch
    import torch.nn.functional as F

    def best_ms(fn, n=5, warm=2):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return min(ts)

    B, H, S, D = q.shape
    dense = 4.0 * B * H * S * S * D
    out = {}
    t = best_ms(lambda: F.scaled_dot_product_attention(q, k, v))
    out["sdpa_dense"] = {"ms": t, "tflops_dense": dense / (t * 1e-3) / 1e12}
    rows = []
    for p, m, fl in zip(ps, masks, flops_p):
        try:
            t = best_ms(lambda: F.scaled_dot_product_attention(q, k, v, attn_mask=m), n=3, warm=1)
            rows.append({"p": p, "ms": t, "tflops_listed_tiles": fl / (t * 1e-3) / 1e12})
        except Exception as e:                      # a backend that cannot take the mask
            rows.append({"p": p, "unavailable": repr(e)[:120]})
    out["sdpa_bool_mask"] = rows
    return out


def _quiet_stdout():
    """Libraries (NCCL's version banner) write to the process's stdout; the one JSON line must be
    the only thing there.  Returns a file object bound to the real stdout and points fd 1 at stderr."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-heads", type=int, default=4, help="heads in the bounded CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--comparators", action="store_true",
                    help="N=1: also time torch SDPA (dense, and with the bool mask) on the same inputs")
    ap.add_argument("--profile", action="store_true",
                    help="profiling run: kernels only (no end-to-end leg, no CPU baseline, no warm-up floor)")
    ap.add_argument("--workload", default="headline", choices=["headline", "document", "composed", "scaling"],
                    help="headline = the benchmark line; the others print kernel-only figures for that configuration")
    ap.add_argument("--batch", type=int, default=0, help="profiling: override the batch size of the workload")
    ap.add_argument("--ps", default="", help="profiling: comma-separated subset of the drop probabilities")
    args = ap.parse_args()
    out = _quiet_stdout()
    sys.stdout = out
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
    out.flush()


if __name__ == "__main__":
    main()
