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

Beside the metric the line carries: ``sharded`` -- the multi-GPU configuration (B=16, H=32,
S=32768, document masks) cut over the ranks by (batch, head) with every rank classifying only
its own mask planes (strong scaling; per-rank stage times, imbalance, a gather check);
``comparators`` -- torch SDPA, FlexAttention and the reference's own Triton kernels on the same
GPU and inputs (N = 1); ``attention_results`` -- the per-p records in the layout of the reference
harness's ``attention_results.json`` (test_attn.py:91-128).

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
NOMINAL = {"hbm_gbs": 8000.0, "bf16_tflops": 2250.0}


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
            handle = nvml_handle(self.index)
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


def nvml_handle(local_index: int):
    """NVML handle of the CUDA device ``local_index`` of this process (read-only use)."""
    import pynvml
    pynvml.nvmlInit()
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    idx = local_index
    if visible:
        try:
            idx = int(visible.split(",")[local_index])
        except ValueError:
            pass
    return pynvml.nvmlDeviceGetHandleByIndex(idx)


def bind_to_gpu_cpus(local_index: int):
    """Restricts this process to the host CPUs NVML names as local to its GPU (same NUMA node / PCIe root),
    intersected with what the process may use, so that the pinned buffers allocated afterwards are placed
    and touched next to the GPU.  Returns a small record for the JSON line; changes nothing on the GPU."""
    rec = {"bound": False}
    try:
        import pynvml
        handle = nvml_handle(local_index)
        allowed = os.sched_getaffinity(0)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (max(allowed | {os.cpu_count() or 1}) // 64) + 1)
        local = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        both = allowed & local
        rec.update({"gpu_local_cpus": len(local), "allowed_cpus": len(allowed), "usable_local_cpus": len(both)})
        if both and both != allowed:
            os.sched_setaffinity(0, both)
            rec["bound"] = True
        elif both == allowed:
            rec["note"] = "every allowed CPU is already local to the GPU"
        else:
            rec["note"] = "no allowed CPU is local to the GPU; affinity left as it was"
    except Exception as e:                       # no NVML, or a container that hides the topology
        rec["note"] = f"not bound: {type(e).__name__}: {e}"[:160]
    return rec


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

    import workloads
    from oracle import cclassify

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
    steps = max(1, min(args.steps, 20))          # a step of the sample takes ~70 ms: 20 + 5 stay within seconds
    warm = max(1, min(args.warmup, 5))
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


# ------------------------------------------------------------------------------- helpers

def best_ms(fn, n=5, warm=2):
    """Best of ``n`` CUDA-event timings of ``fn()`` on the current stream, after ``warm`` untimed runs."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(n):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return min(ts)


def barrier(world):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


# ------------------------------------------------------------------------------- sharded configuration

def document_costs(cfg, batch, seed_base):
    """Per batch element, the sum over its documents of len^2 / 2 -- what a causal document mask
    attends to, known from the (host-side, seeded) document lengths before any mask exists."""
    import workloads
    costs = []
    for b in range(batch):
        lens = workloads.document_lengths(cfg.S, cfg.doc_len[0], cfg.doc_len[1], workloads._cpu_gen(seed_base + b))
        costs.append(sum(0.5 * n * n for n in lens))
    return costs


def run_sharded(rank, world, dev, steps, warmup, balance=True, batch=0, seq=0):
    """The multi-GPU configuration -- B=16, H=32, S=32768, D=128, bf16, per-batch document + causal masks
    with 5 % of the kept 32x32 blocks internally Bernoulli(0.5) -- cut over the ranks by (batch, head):
    strong scaling, no collective on the data path.  Every rank builds, holds and classifies only the mask
    planes of its own batch elements and runs both stages through ``sharding.run_slabs``.  Returns the
    ``sharded`` record (rank 0) or None."""
    import sparseattention_b200 as sa
    import workloads
    from oracle import attention as oa
    from sparseattention_b200 import sharding

    cfg = workloads.CONFIGS["scaling"]
    B, H, S, D = (batch or cfg.B), cfg.H, (seq or cfg.S), cfg.D
    seed_mask, seed_qkv = 5000, 6000
    if seq:
        cfg = workloads.WorkloadConfig(cfg.name, B, H, S, D, cfg.dtype, cfg.kind, cfg.drop_ps, cfg.partial_frac,
                                       (min(cfg.doc_len[0], S // 8), min(cfg.doc_len[1], S // 2)))
    costs = document_costs(cfg, B, seed_mask)
    slabs = sharding.slabs_of(B, H, rank, world, costs if balance else None)
    store = {}
    for slab in slabs:                                        # this rank's data only
        mask = workloads.document_causal_mask(1, S, cfg.doc_len, cfg.partial_frac, seed=seed_mask + slab.b, device=dev)
        q, k, v = workloads.make_qkv(1, H, S, D, torch.bfloat16, seed=seed_qkv + slab.b, device=dev)
        sl = slice(slab.h0, slab.h1)
        store[slab] = (q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous(), mask)
        del q, k, v
    fetch = store.__getitem__

    # untimed pass: FLOPs of the listed tiles, device status, and a host check of one query block per slab
    flops = 0.0
    err_max, err_mean = 0.0, 0.0
    for slab in slabs:
        q, k, v, mask = store[slab]
        h = q.shape[1]
        md = sa.compute_mask_kernel(mask.expand(1, h, S, S), BQ, BK)
        flops += workloads.computed_tile_flops(md.unmasked_lens, md.masked_lens, BQ, BK, D)
        o = sa.sparse_attention(q, k, v, mask, BQ, BK, mask_metadata=md, impl="tcgen05", check_status=True)
        blk = min(S // BQ - 1, (S // BQ) * 2 // 3 + slab.b % 7)   # past the middle, different per batch element
        rows = slice(BQ * blk, BQ * (blk + 1))
        want = torch.from_numpy(oa.sdpa_reference(q[:, :1, rows], k[:, :1], v[:, :1], mask[:, :, rows]))
        d = (o[:, :1, rows].float().cpu() - want).abs()
        err_max, err_mean = max(err_max, d.max().item()), max(err_mean, d.mean().item())
        del o, md

    def attend(q, k, v, m, bq, bk, mask_metadata=None):
        return sa.sparse_attention(q, k, v, m, bq, bk, mask_metadata=mask_metadata, impl="tcgen05")

    for _ in range(warmup):
        sharding.run_slabs(slabs, fetch, BQ, BK, attention=attend)
    barrier(world)
    events_all = []
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        ev = []
        sharding.run_slabs(slabs, fetch, BQ, BK, attention=attend, events=ev)
        events_all.append(ev)
    t1.record()
    barrier(world)
    my_ms = t0.elapsed_time(t1) / steps
    cls_ms = statistics.mean(sum(e[0].elapsed_time(e[1]) for _, e in ev) for ev in events_all) if slabs else 0.0
    att_ms = statistics.mean(sum(e[1].elapsed_time(e[2]) for _, e in ev) for ev in events_all) if slabs else 0.0
    store.clear()
    torch.cuda.empty_cache()

    # gather check on a reduced problem: every rank runs its share of globally indexed inputs through
    # sharded_forward, the outputs are assembled with one all_gather (NCCL) and compared, bit for bit,
    # with the unsharded call on this GPU
    vB, vH, vS = 4, 8, 2048
    vq, vk, vv = workloads.make_qkv(vB, vH, vS, D, torch.bfloat16, seed=77, device=dev)
    vmask = workloads.document_causal_mask(vB, vS, (200, 900), 0.05, seed=78, device=dev)
    vcosts = [float(x) for x in range(1, vB + 1)]
    whole = sa.sparse_attention(vq, vk, vv, vmask, BQ, BK)
    local = sharding.sharded_forward(vq, vk, vv, vmask, BQ, BK, rank, world, costs=vcosts)
    if world > 1:
        full = sharding.gather_outputs(local, vB, vH, device=dev, costs=vcosts)
    else:
        full = torch.empty_like(whole)
        for slab, o in local:
            full[slab.b, slab.h0:slab.h1] = o[0]
    gather_ok = bool(torch.equal(full, whole))

    rec = {"rank": rank, "units": sum(s.h1 - s.h0 for s in slabs), "classify_ms": cls_ms, "attn_ms": att_ms,
           "ms_per_step": my_ms, "flops_per_step": flops, "err_max_vs_sdpa": err_max, "err_mean_vs_sdpa": err_mean,
           "gather_bit_exact": gather_ok}
    if world > 1:
        recs = [None] * world
        torch.distributed.all_gather_object(recs, rec)
    else:
        recs = [rec]
    if rank != 0:
        return None
    ms = [r["ms_per_step"] for r in recs]
    total_flops = sum(r["flops_per_step"] for r in recs)
    peaks, _ = load_peaks()
    return {
        "workload": f"scaling: B={B} H={H} S={S} D={D} bf16, per-batch document+causal masks (lengths U[{cfg.doc_len[0]},"
                    f"{cfg.doc_len[1]}], {int(cfg.partial_frac * 100)}% of kept 32x32 blocks Bernoulli(0.5)), "
                    f"BLOCK_Q={BQ} BLOCK_K={BK}; (batch, head) units cut over the ranks, each rank classifies its own mask planes",
        "scaling": "strong", "n_gpus": world, "steps": steps, "warmup": warmup,
        "partition": "contiguous (batch, head) ranges with equal summed cost (sum of squared document lengths)"
                     if balance else "contiguous (batch, head) ranges with equal unit counts",
        "ms_per_step_max_over_ranks": max(ms), "ms_per_step_mean_over_ranks": statistics.mean(ms),
        "imbalance_max_over_mean": max(ms) / statistics.mean(ms),
        "effective_tflops": total_flops / (max(ms) * 1e-3) / 1e12,
        "frac_of_sustained_bf16_per_gpu": total_flops / (max(ms) * 1e-3) / 1e12 / world / peaks["bf16_tflops_sustained"],
        "per_rank": [{"rank": r["rank"], "units": r["units"], "classify_ms": r["classify_ms"], "attn_ms": r["attn_ms"],
                      "ms_per_step": r["ms_per_step"],
                      "attn_tflops": r["flops_per_step"] / (r["attn_ms"] * 1e-3) / 1e12 if r["attn_ms"] > 0 else None}
                     for r in recs],
        "verification": {"gather_bit_exact_all_ranks": all(r["gather_bit_exact"] for r in recs),
                         "gather_problem": f"B={vB} H={vH} S={vS}, cost-balanced cuts, all_gather over "
                                           f"{'NCCL' if world > 1 else 'one rank (no collective)'}",
                         "max_abs_err_vs_sdpa": max(r["err_max_vs_sdpa"] for r in recs),
                         "mean_abs_err_vs_sdpa": max(r["err_mean_vs_sdpa"] for r in recs),
                         "sdpa_rows": "one 128-row query block of one head per slab, every key, host SDPA"},
    }


# ------------------------------------------------------------------------------- decode-shaped case

def run_decode(args):
    """Kernel-only figures for a decode-shaped call -- 32 query rows per (batch, head) against a cache of
    32768 keys, a quarter of the 32-key blocks attended (per batch element) plus a causal edge.  The
    reference has no such path (README.md:61-65); the bound is HBM: the listed K and V blocks are read once."""
    import sparseattention_b200 as sa
    from sparseattention_b200 import _native

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    _native.load_library()
    peaks, peak_kind = load_peaks()
    B, H, Sq, Sk, D, BK = (args.batch or 8), 32, 32, 32768, 128, 32
    g = torch.Generator(device=dev).manual_seed(11)
    q = torch.randn((B, H, Sq, D), generator=g, device=dev, dtype=torch.bfloat16)
    k = torch.randn((B, H, Sk, D), generator=g, device=dev, dtype=torch.bfloat16)
    v = torch.randn((B, H, Sk, D), generator=g, device=dev, dtype=torch.bfloat16)
    keep = torch.rand((B, 1, 1, Sk // BK), generator=g, device=dev) < 0.25
    keep[..., 0] = True
    mask = keep.repeat_interleave(BK, dim=-1).expand(B, 1, Sq, Sk).clone()
    mask[..., Sk - Sq:] &= torch.ones((Sq, Sq), dtype=torch.bool, device=dev).tril()
    # the padded problem the call builds, once, to time the attention stage by itself
    q128 = torch.cat([q, q.new_zeros((B, H, 128 - Sq, D))], dim=2)
    mask128 = torch.cat([mask, mask.new_zeros((B, 1, 128 - Sq, Sk))], dim=2)
    md = sa.compute_mask_kernel(mask128.expand(B, H, 128, Sk), 128, BK)
    listed = int((md.unmasked_lens.sum(dtype=torch.int64) + md.masked_lens.sum(dtype=torch.int64)).item())
    kv_bytes = listed * BK * D * 2 * 2                      # K and V rows of the listed blocks, bf16
    io_bytes = kv_bytes + 2 * B * H * Sq * D * 2            # + Q read, O written
    res = {}
    res["call_ms"] = best_ms(lambda: sa.sparse_attention(q, k, v, mask, Sq, BK), n=7, warm=3)
    res["call_cached_ms"] = best_ms(lambda: sa.sparse_attention(q, k, v, mask, Sq, BK, cache=True), n=7, warm=3)
    sa.clear_mask_cache()
    res["attention_ms"] = best_ms(lambda: sa.sparse_attention(q128, k, v, mask128, 128, BK, mask_metadata=md), n=7, warm=3)
    res["attention_unsplit_ms"] = best_ms(
        lambda: sa.sparse_attention(q128, k, v, mask128, 128, BK, mask_metadata=md, splits=1), n=5, warm=2)
    # A call of this size is shorter than the host work of launching it: the device time is that of a
    # captured graph replayed back to back (what a decoding loop does).
    def replayed_ms(fn, reps=20):
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps
    res["attention_graph_ms"] = replayed_ms(lambda: sa.sparse_attention(q128, k, v, mask128, 128, BK, mask_metadata=md))
    res["attention_unsplit_graph_ms"] = replayed_ms(
        lambda: sa.sparse_attention(q128, k, v, mask128, 128, BK, mask_metadata=md, splits=1))
    res["generic_kernel_ms"] = best_ms(lambda: sa.sparse_attention(q, k, v, mask, Sq, BK, impl="simt"), n=3, warm=1)
    mask_e = mask.expand(B, H, Sq, Sk)
    res["torch_sdpa_bool_mask_ms"] = best_ms(
        lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask_e), n=5, warm=2)
    out = sa.sparse_attention(q, k, v, mask, Sq, BK)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask_e)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    gbs = io_bytes / (res["attention_graph_ms"] * 1e-3) / 1e9
    print(json.dumps({
        "workload": f"decode-shaped: B={B} H={H} Sq={Sq} Sk={Sk} D={D} bf16, 32-key blocks kept with p=0.25 per batch "
                    f"element + causal edge, lists at (128 padded, {BK})",
        "listed_block_fraction": listed / (B * H * (Sk // BK)),
        "ranges_per_unit": max(1, min(sms // (B * H), Sk // 512, 64)),
        **res,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "peak_source": peak_kind, "kernel": "attn_fwd_tc_kernel<bf16,128> + merge_splits_kernel",
                     "note": "bytes of the listed K and V blocks + Q + O / duration of the attention stage replayed "
                             "from a CUDA graph (CUDA events around 20 replays; K and V are larger than L2 at B >= 2)"},
        "max_abs_vs_torch_sdpa": float((out.float() - ref.float()).abs().max()),
    }))


# ------------------------------------------------------------------------------- backward pass

def run_backward(args):
    """Kernel-only figures for forward + backward through autograd (the reference has no backward pass,
    README.md:61-65): a slice of the headline shape, p = 0.5, against torch SDPA with the bool mask on the same GPU."""
    import sparseattention_b200 as sa
    import workloads
    from sparseattention_b200 import _native

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    _native.load_library()
    B, H, S, D, BQ, BK = (args.batch or 1), 8, 4096, 128, 128, 32
    q, k, v = (t.requires_grad_(True) for t in workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=5, device=dev))
    mask = workloads.random_block_mask(B, S, 0.5, 0.1, seed=6, device=dev)
    md = sa.compute_mask_kernel(mask.expand(B, H, S, S), BQ, BK)
    g = torch.randn((B, H, S, D), device=dev, dtype=torch.bfloat16)
    flops_fwd = workloads.computed_tile_flops(md.unmasked_lens, md.masked_lens, BQ, BK, D)

    def ours():
        out = sa.sparse_attention(q, k, v, mask, BQ, BK, mask_metadata=md)
        out.backward(g)
        q.grad = k.grad = v.grad = None

    mask_e = mask.expand(B, H, S, S)

    def sdpa():
        out = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask_e)
        out.backward(g)
        q.grad = k.grad = v.grad = None

    fwd_ms = best_ms(lambda: sa.sparse_attention(q.detach(), k.detach(), v.detach(), mask, BQ, BK, mask_metadata=md), n=5, warm=2)
    ours_ms = best_ms(ours, n=3, warm=1)
    sdpa_ms = best_ms(sdpa, n=3, warm=1)
    print(json.dumps({
        "workload": f"forward + backward: B={B} H={H} S={S} D={D} bf16, 32x32-block mask, drop p=0.5, lists at ({BQ},{BK})",
        "forward_ms": fwd_ms, "forward_plus_backward_ms": ours_ms, "backward_ms": ours_ms - fwd_ms,
        "backward_tflops_over_listed_tiles": 2.5 * flops_fwd / ((ours_ms - fwd_ms) * 1e-3) / 1e12,
        "torch_sdpa_bool_mask_forward_plus_backward_ms": sdpa_ms,
        "note": "backward = kv-major list transpose + dQ and dK/dV kernels on the tensor cores (warp-level MMA, fp32 accumulation); "
                "2.5 x the forward's FLOPs over the listed tiles",
    }))


# ------------------------------------------------------------------------------- GPU arm

def run_ours(args):
    import sparseattention_b200 as sa
    import workloads
    from sparseattention_b200 import _native

    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        args.gpus = world
    numa = bind_to_gpu_cpus(local)                 # before any pinned allocation
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
    flops_p, bytes_p, bits_bytes_p, mix, frac_unmasked = [], [], [], [], []
    for i in range(len(ps)):
        md = stage1(i)
        o = sa.sparse_attention(q, k, v, masks[i], BQ, BK, mask_metadata=md, impl="tcgen05", check_status=True)
        flops_p.append(workloads.computed_tile_flops(md.unmasked_lens, md.masked_lens, BQ, BK, D))
        lens_sum = int(md.unmasked_lens[:, 0].sum()) + int(md.masked_lens[:, 0].sum())
        bytes_p.append(workloads.classifier_bytes(planes, S, S, BQ, lens_sum))
        bits_bytes_p.append(float(planes) * S * S / 8.0)        # the packed plane stage 2 reads (written by stage 1)
        tiles = B * H * (S // BQ) * (S // BK)
        mix.append((float(md.unmasked_lens.sum()) / tiles, float(md.masked_lens.sum()) / tiles))
        frac_unmasked.append(float(masks[i].sum(dtype=torch.int64)) / masks[i].numel())
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

    for _ in range(warmup):
        step()
    barrier(world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    t_start.record()
    for s in range(args.steps):
        step(ev[s])
    t_end.record()
    barrier(world)
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = t_start.elapsed_time(t_end)

    # Stage 1 by itself, its launches back to back (one graph of the n_p calls, replayed): between two 2 ms
    # attention launches, a pair of events around a 30 us kernel also times the gap before it.
    cls_b2b_ms = None
    if rank == 0 and not args.profile and args.workload == "headline":
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            held = [stage1(i) for i in range(n_p)]
        graph.replay()
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(10):
            graph.replay()
        g1.record()
        torch.cuda.synchronize()
        cls_b2b_ms = g0.elapsed_time(g1) / 10.0          # all n_p masks once
        del held, graph

    cls_ms = [statistics.mean(ev[s][2 * i].elapsed_time(ev[s][2 * i + 1]) for s in range(args.steps)) for i in range(n_p)]
    att_ms = [statistics.mean(ev[s][2 * i + 1].elapsed_time(ev[s][2 * i + 2]) for s in range(args.steps)) for i in range(n_p)]
    att_all = [[ev[s][2 * i + 1].elapsed_time(ev[s][2 * i + 2]) for s in range(args.steps)] for i in range(n_p)]

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

    # ---- the caller's other list granularities on the p = 0.5 mask (stage 2 alone, lists passed in)
    granularities = []
    if 0.5 in ps:
        i5 = ps.index(0.5)
        for bq in (128, 64, 32):
            md = sa.compute_mask_kernel(masks_e[i5], bq, BK)
            t = best_ms(lambda: sa.sparse_attention(q, k, v, masks[i5], bq, BK, mask_metadata=md), n=5, warm=2)
            listed = float(md.unmasked_lens.sum(dtype=torch.int64) + md.masked_lens.sum(dtype=torch.int64))
            granularities.append({"BLOCK_Q": bq, "BLOCK_K": BK, "attn_ms": t,
                                  "listed_tile_fraction": listed / (B * H * (S // bq) * (S // BK))})
            del md

    # ---- end to end through the public entry points with host buffers
    host_q, host_k, host_v = (t.cpu().pin_memory() for t in (q, k, v))
    host_masks = [m.cpu().pin_memory() for m in masks]
    host_o = torch.empty((B, H, S, D), dtype=dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (host_q, host_k, host_v)) + sum(m.numel() for m in host_masks)
    d2h = n_p * host_o.numel() * host_o.element_size()

    # Three streams: host->device copies, compute (the caller's current stream), device->host
    # copies; the copies of one mask overlap the kernels of the previous one (PCIe is full duplex).
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dummy_o = torch.empty((B, H, S, D), dtype=dtype, device=dev)

    def e2e_step(compute=True):
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
            # the reference's call, stage 1 inside; the copy-only run sends back a buffer of the same size
            o = sa.sparse_attention(dq, dk, dv, dms[i], BQ, BK) if compute else dummy_o
            done = torch.cuda.Event()
            done.record(main)
            o.record_stream(s_out)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                host_o.copy_(o, non_blocking=True)

    def e2e_drain():
        main.wait_stream(s_in)
        main.wait_stream(s_out)                                  # the last result is on the host

    def e2e_time(n_steps, compute):
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        e2e_step(compute)
        e2e_drain()
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for _ in range(n_steps):
            e2e_step(compute)
        e2e_drain()
        e1.record()
        barrier(world)
        return e0.elapsed_time(e1)

    e2e_steps = max(1, min(args.steps, 5))
    e2e_ms = e2e_time(e2e_steps, True)
    copy_ms = e2e_time(e2e_steps, False)           # same buffers, streams and events, no kernels
    del host_q, host_k, host_v, host_masks, host_o, dummy_o

    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([elapsed_ms, e2e_ms, copy_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, copy_ms = float(t[0]), float(t[1]), float(t[2])
        f = torch.tensor([flops_step], device=dev, dtype=torch.float64)
        dist.all_reduce(f, op=dist.ReduceOp.SUM)
        flops_all = float(f[0])
    else:
        flops_all = flops_step

    # ---- same-GPU comparators (N = 1; outside every timed region of the metric)
    comparators = None
    if world == 1 and not args.no_comparators:
        comparators = gpu_comparators(q, k, v, masks, ps, flops_p)
    del q, k, v, masks, masks_e
    torch.cuda.empty_cache()

    # ---- the sharded multi-GPU configuration (strong scaling), every rank
    sharded = None
    if not args.no_sharded:
        try:
            sharded = run_sharded(rank, world, dev, max(1, min(args.steps, 5)), 2)
        except torch.cuda.OutOfMemoryError as e:
            sharded = {"unavailable": f"out of device memory: {e}"[:200]} if rank == 0 else None
        torch.cuda.empty_cache()

    if rank == 0:
        peaks, peak_kind = load_peaks()
        ms_per_step = elapsed_ms / args.steps
        value = flops_all / (ms_per_step * 1e-3) / 1e12
        att_total_ms = sum(att_ms)
        att_tflops = flops_step / (att_total_ms * 1e-3) / 1e12
        cls_total_ms = sum(cls_ms)
        cls_gbs = sum(bytes_p) / (cls_total_ms * 1e-3) / 1e9
        cls_gbs_with_plane = (sum(bytes_p) + sum(bits_bytes_p)) / (cls_total_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(), "l2": "inputs larger than L2 (Q,K,V 768 MiB, each mask 128 MiB)",
                       "flop_accounting": "4*D*BQ*BK per listed (non-skipped) tile, both stages timed",
                       "shard": "each rank owns a full (batch, head) shard of the workload"},
            "roofline": {"bound": "tensor", "achieved": att_tflops, "peak": peaks["bf16_tflops_sustained"],
                         "unit": "TFLOP/s", "frac": att_tflops / peaks["bf16_tflops_sustained"],
                         "frac_of_burst": att_tflops / peaks["bf16_tflops"],
                         "frac_of_nominal": att_tflops / NOMINAL["bf16_tflops"],
                         "traffic": 254.3e6 * B / 2.0, "traffic_unit": "bytes per launch (ncu capture at B=2, p=0.5, scaled by batch)",
                         "kernel": "attn_fwd_tc_kernel<bf16,128>", "peak_source": peak_kind + " (sustained bf16 matmul)",
                         "note": "FLOPs of the listed tiles of all six launches / sum of their durations (CUDA events)"},
            "roofline_classifier": {"bound": "hbm", "achieved": cls_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                    "frac": cls_gbs / peaks["hbm_gbs"],
                                    "frac_of_nominal": cls_gbs / NOMINAL["hbm_gbs"],
                                    "achieved_back_to_back": None if cls_b2b_ms is None else sum(bytes_p) / (cls_b2b_ms * 1e-3) / 1e9,
                                    "frac_back_to_back": None if cls_b2b_ms is None
                                    else sum(bytes_p) / (cls_b2b_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                    "frac_back_to_back_with_packed_plane": None if cls_b2b_ms is None
                                    else (sum(bytes_p) + sum(bits_bytes_p)) / (cls_b2b_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                    "us_per_mask_back_to_back": None if cls_b2b_ms is None else cls_b2b_ms * 1e3 / n_p,
                                    "achieved_with_packed_plane": cls_gbs_with_plane,
                                    "frac_with_packed_plane": cls_gbs_with_plane / peaks["hbm_gbs"],
                                    "traffic": 279.6e6 * B / 16.0,
                                    "traffic_unit": "bytes per launch (ncu capture at 16 mask planes: 268.6 MB read + "
                                                    "11.0 MB written, scaled by planes)",
                                    "kernel": "classify_kernel",
                                    "note": "algorithmic bytes (mask read once + lists; the 12.5 % of packed-plane writes "
                                            "are counted only in the *_with_packed_plane figures) / duration of the stage-1 "
                                            "calls between the attention launches of the timed steps (events around each: "
                                            "the gap before the kernel is in it); *_back_to_back: the same calls replayed "
                                            "from one CUDA graph, launch after launch"},
            "sweep": [{"p": p, "classify_ms": c, "attn_ms": a, "attn_ms_median": statistics.median(al),
                       "attn_ms_best": min(al), "attn_tflops": fl / (a * 1e-3) / 1e12,
                       "classify_gbs": by / (c * 1e-3) / 1e9, "full_frac": fm, "partial_frac": pm}
                      for p, c, a, al, fl, by, (fm, pm) in zip(ps, cls_ms, att_ms, att_all, flops_p, bytes_p, mix)],
            "list_granularities_p0.5": granularities,
            "e2e": {"value": flops_all / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps,
                    "copy_only_ms_per_step": copy_ms / e2e_steps,
                    "frac_of_copy_ceiling": copy_ms / e2e_ms,
                    "copy_gbs_per_direction_per_gpu": [h2d / (copy_ms / e2e_steps * 1e-3) / 1e9,
                                                       d2h / (copy_ms / e2e_steps * 1e-3) / 1e9],
                    "host_affinity": numa,
                    "note": "copy_only = the same pinned buffers, streams and events with the kernels left out: "
                            "what the host links allow at this N"},
            "gpu_launches": args.steps * n_p * 2,
            "clocks": clocks,
        }
        if sharded is not None:
            line["sharded"] = sharded
        if comparators is not None:
            line["comparators"] = comparators
        line["attention_results"] = ta_results(B, H, S, D, ps, frac_unmasked, att_ms, comparators)
        if args.results_json:
            with open(args.results_json, "w") as f:
                json.dump(line["attention_results"], f, indent=2)
        if world == 1 and not args.no_cpu_baseline:
            val, sec, desc, cores = cpu_sample(args.cpu_heads, 1, 1)
            line["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def ta_results(B, H, S, D, ps, frac_unmasked, sparse_ms, comparators):
    """The per-p records of the reference harness (test_attn.py:91-128: ``attention_results.json``) for this
    run: ``p`` there is the fraction of blocks KEPT (1 - drop probability), ``useful_flops`` is the dense
    FLOP count times the fraction of True mask elements (test_attn.py:105-108), and the sparse time is
    stage 2 alone with the lists passed in (test_attn.py:65)."""
    total_flops = 2 * 2 * B * H * S * S * D                                    # test_attn.py:84
    ref_ms = {r["p"]: r.get("ms") for r in (comparators or {}).get("sdpa_bool_mask", []) if "ms" in r}
    ext = (comparators or {}).get("reference_package", {})
    flex_ms = {r["p"]: r.get("flex_ms") for r in ext.get("rows", []) if r.get("flex_ms") is not None}
    tri_ms = {r["p"]: r.get("triton_attn_ms") for r in ext.get("rows", []) if r.get("triton_attn_ms") is not None}
    rows = []
    for p, fu, t in zip(ps, frac_unmasked, sparse_ms):
        useful = total_flops * fu
        row = {"p": 1.0 - p, "drop_p": p, "fraction_unmasked": fu, "useful_flops": useful,
               "sparse_time_ms": t, "sparse_tflops_per_sec": useful / (t / 1000) / 1e12}
        for name, table in (("ref", ref_ms), ("flex", flex_ms), ("reference_triton", tri_ms)):
            if p in table:
                row[f"{name}_time_ms"] = table[p]
                row[f"{name}_tflops_per_sec"] = useful / (table[p] / 1000) / 1e12
        rows.append(row)
    return {"config": {"shape": [B, H, S, S], "BLOCK_Q": BQ, "BLOCK_K": BK, "total_flops": total_flops},
            "results": rows}


def gpu_comparators(q, k, v, masks, ps, flops_p):
    """Same-GPU comparators of the reference's harness (test_attn.py:64-68), timed like the reference times
    them (CUDA events, best of a few runs after a warm-up): torch SDPA without a mask (the vendor's dense
    kernel) and with the bool mask, in this process; the reference's own Triton kernels and FlexAttention
    in a child process that imports the reference package from ``baseline/_ref`` (the same inputs are
    rebuilt there from the seeds).  The figures are not part of the metric."""
    import torch.nn.functional as F

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
    out["reference_package"] = reference_package_comparators(B, H, S, D, ps)
    return out


def reference_package_comparators(B, H, S, D, ps, timeout_s=420):
    """Runs ``baseline/reference_comparators.py`` (the reference's Triton kernels and FlexAttention on the
    headline inputs) in a child process and returns what it printed; ``unavailable`` with the reason when
    the reference package is not there, the child fails or runs out of time."""
    script = os.path.join(ROOT, "baseline", "reference_comparators.py")
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "sparseattention")):
        return {"unavailable": "baseline/_ref/sparseattention is not present on this machine"}
    cmd = [sys.executable, script, "--B", str(B), "--H", str(H), "--S", str(S), "--D", str(D),
           "--ps", ",".join(str(p) for p in ps)]
    rec = {"rows": []}
    by_p = {}

    def take(text):
        for ln in (text or "").splitlines():
            if ln.startswith("{"):
                part = json.loads(ln)
                if "row" in part:                  # rows of the same p (Triton part, Flex part) are merged
                    by_p.setdefault(part["row"]["p"], {}).update(part["row"])
                else:
                    rec.update(part)
        rec["rows"] = [by_p[p] for p in sorted(by_p)]

    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s)
        take(res.stdout)                           # the child prints one JSON object per finished part
        if res.returncode != 0:
            rec["unavailable"] = ("child exited with " + str(res.returncode) + ": " + res.stderr.strip()[-300:])
    except subprocess.TimeoutExpired as e:
        take(e.stdout.decode() if isinstance(e.stdout, bytes) else e.stdout)
        rec["unavailable"] = f"child did not finish within {timeout_s} s (parts that finished are kept)"
    except Exception as e:
        rec["unavailable"] = repr(e)[:300]
    return rec


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
    ap.add_argument("--no-comparators", action="store_true",
                    help="N=1: skip torch SDPA / FlexAttention / reference-Triton timings on the same inputs")
    ap.add_argument("--no-sharded", action="store_true", help="skip the sharded multi-GPU configuration")
    ap.add_argument("--results-json", default="", help="also write the attention_results record to this file")
    ap.add_argument("--profile", action="store_true",
                    help="profiling run: kernels only (no end-to-end leg, no CPU baseline, no warm-up floor)")
    ap.add_argument("--workload", default="headline", choices=["headline", "document", "composed", "scaling", "decode", "backward"],
                    help="headline = the benchmark line; the others print kernel-only figures for that configuration "
                         "(decode: 32 query rows against 32768 keys, one GPU)")
    ap.add_argument("--batch", type=int, default=0, help="profiling: override the batch size of the workload")
    ap.add_argument("--ps", default="", help="profiling: comma-separated subset of the drop probabilities")
    args = ap.parse_args()
    out = _quiet_stdout()
    sys.stdout = out
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.workload == "backward":
        run_backward(args)
    else:
        run_ours(args)
    out.flush()


if __name__ == "__main__":
    main()
