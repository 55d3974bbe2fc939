#!/usr/bin/env python
"""Benchmark of the quantized MoE feed-forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--layers L] [--slots S] [--sub-layers P] [--no-sub]
    (N > 1: python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...)

One JSON line on stdout (rank 0).  The headline workload is the decode configuration: a
stack of 40 MoE layers (2048 / 512 / 256 experts / top-8, F16 router, IQ3_XXS gate+up,
IQ4_XS down, Q8_0 shared expert, per-layer seeds), 16 concurrent slots per GPU with
independent N(0,1) hidden rows per layer.  A step is one pass of the rows through the 40
layers; value = tokens / second through the stack, summed over the GPUs (each GPU holds
the whole stack and decodes its own slots: weak scaling, no collective).  Weights are
seeded synthetic ggml blocks (no model file is needed).

Sub-objects of the same line: "prefill" - batched prefill of one layer at several chunk
sizes on the tensor cores (1 GPU), or the expert-parallel layer with experts sharded over
the N GPUs and NCCL all-to-all dispatch / combine (N > 1, strong scaling); "gemv" - the
dense dequant-GEMV sweep (1 GPU).

Timing: W >= 3 untimed steps, then K steps between two CUDA events on the launching
stream, bracketed by barrier + synchronize; max over ranks.  The working set of a step
(40 x ~140 MB of weights for decode, 8 rotating layers for prefill, > 250 MB of matrix
copies for GEMV) is larger than the 126 MB L2, so every step streams its weights from HBM.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

SEED_W, SEED_X = 42, 43


def measured_peaks():
    """HBM GB/s and bf16 TF/s from MEASURED_PEAKS.json (a copy benchmark and a cuBLAS GEMM run on the
    target GPUs), else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML read calls
    from a thread every 20 milliseconds (the region lasts tens of milliseconds, too short for
    a freshly started nvidia-smi to report in), nvidia-smi as the fallback.  Read-only."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc = gpu_index, [], None
        self.nvml = self.handle = self.t = None
        self.sm, self.mask, self.mx, self.stop_flag = [], 0, None, False
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in vis.split(",") if v.strip()]
            phys = int(ids[gpu_index]) if ids and all(v.strip().isdigit() for v in ids) and gpu_index < len(ids) else gpu_index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.mx = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def _poll(self):
        nv = self.nvml
        reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                self.mask |= int(reasons(self.handle))
            except Exception:
                pass
            time.sleep(0.02)

    def start(self):
        if self.nvml:
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.nvml:
            self.stop_flag = True
            self.t.join(timeout=1)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.mx,
                    "reasons": sorted(n for n, b in self.REASON_BITS if self.mask & b), "samples": len(self.sm),
                    "source": "nvml"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx = float(r[2])
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                    if r[col].lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ------------------------------------------------------------------ CPU arm (oracle port)

def cpu_moe_sample(syn, orc_mod, dims, n_slots, layers_sample, threads, router_type, gateup_type, down_type, cache=None):
    """Times the CPU path (quants.h-style dequant + scalar f32 loop, restated in
    oracle/qkm_oracle.cpp) on `layers_sample` layers x n_slots rows with `threads`
    host threads.  Returns seconds per (layer x n_slots rows).  `cache` (a dict) keeps the
    generated layers and inputs between calls, so that repeated steps time the same data without
    generating it again (349 MB per layer)."""
    orc = orc_mod.Oracle()
    total = 0.0
    for l in range(layers_sample):
        if cache is not None and l in cache:
            layer, x = cache[l]
        else:
            layer = syn.make_layer(dims, SEED_W, l, router_type, gateup_type, down_type)
            x = syn.random_x(n_slots, dims.n_embd, SEED_X + l)
            if cache is not None:
                cache[l] = (layer, x)
        t0 = time.perf_counter()
        orc.moe_layer(layer, x, acc=orc_mod.ACC_F32, threads=threads)
        total += time.perf_counter() - t0
    return total / layers_sample


def run_reference_arm(args, syn):
    """The reference's CPU implementation of the path (quants.h-style row dequantisation + scalar
    f32 loop, restated in oracle/; its own moeCpuRef is single-threaded and f64), timed on the
    host cores with all the threads the box has.  A step is the same workload as ours: n_slots
    rows through `layers` layers.  All layers are timed when the whole run fits a few minutes
    (N = 1); otherwise a step times a bounded sample of the layers and scales it, and says so."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    orc_mod = entry.oracle_module()
    orc_mod.build(ref=False)
    dims = syn.Dims()
    threads = orc_mod.Oracle().hardware_threads() or 1
    n_layers, n_slots = args.layers, args.slots * max(1, args.gpus)
    budget_s = 150.0
    cache = {}   # the layers are generated once (14 GB of host memory for 40 layers) and reused by every step
    t_layer = cpu_moe_sample(syn, orc_mod, dims, n_slots, 1, threads, syn.F16, syn.IQ3_XXS, syn.IQ4_XS, cache)   # probe, untimed
    total_steps = args.steps + args.warmup
    sample_layers = n_layers if t_layer * n_layers * total_steps <= budget_s else max(1, int(budget_s / (t_layer * total_steps)))
    sample_layers = min(sample_layers, n_layers)
    per_step = []
    for i in range(total_steps):
        t = cpu_moe_sample(syn, orc_mod, dims, n_slots, sample_layers, threads, syn.F16, syn.IQ3_XXS, syn.IQ4_XS, cache) * sample_layers
        if i >= args.warmup:
            per_step.append(t)
    sec_per_step = float(np.mean(per_step)) * n_layers / sample_layers
    value = n_slots / sec_per_step
    sample = (f"all {n_layers} layers x {n_slots} rows per step" if sample_layers == n_layers else
              f"{sample_layers} of {n_layers} layers x {n_slots} rows per step, scaled by layers")
    cfg = decode_config(args, n_slots)
    cfg["parallelism"] = parallelism_label(max(1, args.gpus), args.slots)
    line = {
        "impl": "reference", "metric": "moe_decode_tok_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "measured_all_layers": sample_layers == n_layers,
    }
    print(json.dumps(line), flush=True)


def parallelism_label(world, slots):
    return "1 GPU" if world == 1 else f"{world} replicas of the stack, {slots} slots each, no collective"


def decode_config(args, n_slots):
    return {"workload": f"moe_decode_stack: {args.layers} layers x {n_slots} slots, n_embd 2048, n_ff 512, "
                        "256 experts top-8, F16 router, IQ3_XXS gate/up, IQ4_XS down, Q8_0 shared",
            "layers": args.layers, "slots": n_slots, "l2": "working set per step >> 126 MB L2 (weights stream from HBM)"}


# ------------------------------------------------------------------ GPU arm

class Ranks:
    """Process-group plumbing: one rank per GPU under torchrun, a single process otherwise."""

    def __init__(self, torch):
        self.torch = torch
        self.rank, self.local_rank, self.world = dist_env()
        self.dev = torch.device("cuda", self.local_rank)
        torch.cuda.set_device(self.dev)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, v: float) -> float:
        if not self.dist:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, v: float) -> float:
        if not self.dist:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed(torch, R: Ranks, stream, fn, steps: int, warmup: int) -> float:
    """ms per step: warm-up, barrier + synchronize, CUDA events on the launching stream
    around exactly `steps` calls, barrier + synchronize, max over ranks."""
    for _ in range(warmup):
        fn()
    R.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    R.barrier()
    return R.max_over_ranks(e0.elapsed_time(e1) / steps)


def run_ours(args, pkg, syn):
    import torch
    R = Ranks(torch)
    dev, world, rank = R.dev, R.world, R.rank
    dims = syn.Dims()
    L, S = args.layers, args.slots
    orc_mod = entry.oracle_module()
    orc = orc_mod.Oracle()
    peaks = measured_peaks()

    # ---- weights: every rank holds the whole stack (14 GB of 180): decode slots are
    # independent sequences, so ranks are replicas for this workload and no collective is
    # on its data path.  The expert-parallel workloads below shard the experts instead.
    ctx = pkg.Context(dims, n_layer=L, max_tokens=S, device=R.local_rank)
    stream = torch.cuda.Stream(dev)   # a real stream: the stack is replayed as a CUDA graph
    ctx.set_stream(stream.cuda_stream)
    layers_keep = []
    x_all = np.empty((L, S, dims.n_embd), np.float32)
    ref_all = np.empty((L, S, dims.n_embd), np.float32)   # the oracle's output of every layer (checked below)
    nthr = orc.hardware_threads() or 1
    for l in range(L):
        layer = syn.make_layer(dims, SEED_W, l, syn.F16, syn.IQ3_XXS, syn.IQ4_XS)
        ctx.upload_layer(l, layer)
        x_all[l] = syn.random_x(S, dims.n_embd, SEED_X + 1000 * rank + l)
        ref_all[l] = orc.moe_layer(layer, x_all[l], threads=nthr)["y"]
        if l < args.sub_layers:
            layers_keep.append(layer)
    with torch.cuda.stream(stream):
        x_dev = torch.from_numpy(x_all).to(dev)
        y_dev = torch.empty_like(x_dev)
    x_pin = torch.from_numpy(x_all).pin_memory()
    y_pin = torch.empty_like(x_pin).pin_memory()

    def step():
        ctx.moe_decode_stack(0, L, x_dev, S, y_dev)

    # correctness of what is being timed: every layer of the stack against the oracle
    step(); R.barrier()
    y_host = y_dev.cpu().numpy()
    errs = [syn.rel_err_rows(y_host[l], ref_all[l]) for l in range(L)]
    err0 = float(max(errs))
    assert err0 < 1e-5, f"layer {int(np.argmax(errs))} output error {err0}"
    del ref_all

    # distinct experts per layer (for the algorithmic byte count), from the device's own routing
    distinct = []
    for l in range(L):
        ctx.moe_decode(l, x_dev[l], S, y_dev[l])
        ids = ctx.last_sel(S)["ids"][:, :dims.n_used]
        distinct.append(len(np.unique(ids)))
    bytes_step = sum(syn.layer_touched_bytes(dims, syn.F16, syn.IQ3_XXS, syn.IQ4_XS, u) for u in distinct)

    W = max(args.warmup, 3)
    for _ in range(W):
        step()
    # rank 0 alone samples its GPU's clocks: NVML calls from every rank at once contend for the driver's
    # locks and held back the graph launches of an 8-rank run (130 instead of 75 us per layer)
    sampler = ClockSampler(R.local_rank) if rank == 0 else None
    R.barrier()
    if sampler:
        sampler.start()
    n0 = ctx.launch_count()
    ms = timed(torch, R, stream, step, args.steps, 0)
    launches = ctx.launch_count() - n0
    clocks = sampler.stop() if sampler else None
    value = world * S / (ms * 1e-3)
    bytes_all = R.sum_over_ranks(float(bytes_step))

    # end to end: pinned host rows in, host rows out, every step (wall clock, max over ranks)
    for _ in range(2):
        ctx.moe_decode_stack_host(0, L, x_pin.data_ptr(), S, y_pin.data_ptr())
    R.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ctx.moe_decode_stack_host(0, L, x_pin.data_ptr(), S, y_pin.data_ptr())
    e2e_s = R.max_over_ranks((time.perf_counter() - t0) / args.steps)
    assert np.array_equal(y_pin[0].numpy(), y_dev[0].cpu().numpy())

    line = {
        "metric": "moe_decode_tok_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": decode_config(args, S * world),
        "hbm": {"algorithmic_bytes_per_step": bytes_all, "gbs": bytes_all / (ms * 1e-3) / 1e9,
                "gbs_per_gpu": bytes_all / world / (ms * 1e-3) / 1e9,
                "frac_of_measured_copy": bytes_all / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "frac_of_nominal_8TBs": bytes_all / world / (ms * 1e-3) / 8e12,
                "distinct_experts_per_layer_mean": float(np.mean(distinct))},
        "us_per_layer": ms * 1e3 / L,
        "e2e": {"value": world * S / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": int(x_pin.numel() * 4) * world,
                "d2h_bytes_per_step": int(y_pin.numel() * 4) * world, "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(launches) * world, "clocks": clocks, "parity": {"max_rel_err_over_all_layers": err0, "layers_checked": L},
    }
    line["config"]["parallelism"] = parallelism_label(world, S)

    # per-kernel timing of the dominant kernels over the same inputs (CUDA events, this stream)
    if rank == 0:
        kern = time_kernels(ctx, pkg, syn, torch, dev, stream, L, S, x_dev, distinct, dims)
        dom = max(kern.values(), key=lambda k: k["ms_per_layer"])
        line["roofline"] = {
            "bound": "hbm", "kernel": dom["name"], "achieved": dom["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": dom["gbs"] / peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy bandwidth",
            "frac_of_nominal_8TBs": dom["gbs"] / 8000.0, "traffic": ncu_traffic(dom["name"]),
            "bytes_per_launch": dom["bytes_per_launch"], "ms_per_launch": dom["ms_per_layer"]}
        line["kernels"] = kern
        threads = orc.hardware_threads() or 1
        if world == 1:
            cpu_sec_layer = cpu_moe_sample(syn, orc_mod, dims, S, 2, threads, syn.F16, syn.IQ3_XXS, syn.IQ4_XS)
            line["cpu_baseline"] = {"value": S / (cpu_sec_layer * L), "unit": "tok/s", "cores": threads, "kind": "port",
                                    "sample": f"2 of {L} layers x {S} rows on the host cores, scaled by layers"}
            # the reference's own CPU loop is single-threaded: the same path on one thread (4 rows x 1 layer, scaled)
            one = cpu_moe_sample(syn, orc_mod, dims, 4, 1, 1, syn.F16, syn.IQ3_XXS, syn.IQ4_XS)
            line["cpu_baseline"]["single_thread"] = {"value": 4 / (one * L), "unit": "tok/s", "cores": 1,
                                                     "sample": f"1 of {L} layers x 4 rows on one thread, scaled by layers"}
            line["decode_batch1"] = run_batch1(ctx, syn, torch, R, stream, L, dims, x_all, peaks, orc, layers_keep)
    R.barrier()
    ctx.close()
    del x_dev, y_dev
    torch.cuda.empty_cache()

    # ---- the other type mixes the reference loads (src/main.cpp:1283-1291): a Q6_K down tensor, IQ4_XS
    # gate/up tensors.  Same three-kernel decode sequence on their own tile layouts.  Four rotating
    # layers, same 16 slots.
    if not args.no_sub and world == 1:
        QL = 4
        for key, gt, dt, what in (("decode_q6k_down", syn.IQ3_XXS, syn.Q6_K, "Q6_K down tensors (decode_down_q6k_kernel)"),
                                  ("decode_iq4_gateup", syn.IQ4_XS, syn.IQ4_XS, "IQ4_XS gate/up tensors (decode_gateup_kernel<IQ4_XS>)")):
            cq = pkg.Context(dims, n_layer=QL, max_tokens=S, device=R.local_rank)
            sq = torch.cuda.Stream(dev)
            cq.set_stream(sq.cuda_stream)
            q_layers = [syn.make_layer(dims, SEED_W, 100 + l, syn.F16, gt, dt) for l in range(QL)]
            for l, ly in enumerate(q_layers):
                cq.upload_layer(l, ly)
            with torch.cuda.stream(sq):
                xq = torch.from_numpy(x_all[:QL].copy()).to(dev)
                yq = torch.empty_like(xq)
            cq.moe_decode_stack(0, QL, xq, S, yq); R.barrier()
            refq = orc.moe_layer(q_layers[0], x_all[0], threads=orc.hardware_threads())
            errq = syn.rel_err_rows(yq[0].cpu().numpy(), refq["y"])
            assert errq < 1e-5, f"{key}: layer output error {errq}"
            msq = timed(torch, R, sq, lambda: cq.moe_decode_stack(0, QL, xq, S, yq), args.steps, 3) / QL
            line[key] = {"us_per_layer": msq * 1e3, "tok_s_through_40_layers": S / (msq * 40e-3),
                         "rel_err_vs_oracle": errq, "layers_rotated": QL,
                         "note": f"working set {QL} layers x 0.4-0.5 GB > L2; {what}"}
            cq.close()
            del xq, yq, cq
            torch.cuda.empty_cache()

    # ---- the other configurations, as sub-objects of the same line
    if not args.no_sub:
        line["prefill"] = run_prefill_or_ep(args, pkg, syn, torch, R, orc, layers_keep, peaks)
        if world > 1:
            line["config"]["expert_parallel"] = {"ranks": world, "experts_per_rank": dims.n_expert // world,
                                                 "tokens": line["prefill"].get("summary")}
        if world == 1:
            line["gemv"] = run_gemv_sweep(args, pkg, syn, torch, R, orc, peaks)
    if rank == 0:
        print(json.dumps(line), flush=True)
    R.close()


def ncu_traffic(stage: str):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of a decode stage's
    kernel, from profiles/ncu_traffic.json - written when the ncu capture summarised under
    profiles/ was taken, with the commit it was taken at.  None when the file has no entry."""
    p = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        return json.load(open(p)).get(stage, {}).get("dram_bytes_per_launch")
    except Exception:
        return None


PREFILL_CHUNKS = (128, 256, 512, 2048, 4096)
TENSOR_FLOPS_PER_TOKEN = 56_623_104   # routed 8 x (gate, up, down) + shared expert, 2 x MACs


def run_prefill_or_ep(args, pkg, syn, torch, R: Ranks, orc, layers, peaks):
    """1 GPU: batched prefill (tcgen05 expert GEMMs) at several chunk sizes, rotating over
    `len(layers)` distinct layers so weights come from HBM.  N GPUs: the same token counts
    split over the ranks, experts sharded, rows exchanged by all-to-all (strong scaling)."""
    dims = syn.Dims()
    dev, world, rank = R.dev, R.world, R.rank
    PL = len(layers)
    Tmax = max(PREFILL_CHUNKS)
    per = dims.n_expert // world
    ctx = pkg.Context(dims, n_layer=PL, max_tokens=Tmax, device=R.local_rank,
                      expert_first=rank * per if world > 1 else 0, expert_count=per if world > 1 else 0)
    for l, layer in enumerate(layers):
        ctx.upload_layer(l, layer.expert_slice(rank * per, per) if world > 1 else layer)
    stream = torch.cuda.current_stream(dev)
    n_max = Tmax // world
    x_np = np.stack([syn.random_x(n_max, dims.n_embd, SEED_X + 77 + 1000 * rank + l) for l in range(PL)])
    x = torch.from_numpy(x_np).to(dev)
    y = torch.empty_like(x)
    ep = None
    if world > 1:
        from qwen_kernel_b200.expert_parallel import ExpertParallel
        ep = ExpertParallel(ctx, dims.n_embd, dims.n_used, max_local_tokens=n_max, max_recv_rows=Tmax, device=dev)
    out = {"layers_rotated": PL, "chunks": {}}
    # the peer-memory form (rows stored straight into the owners' buffers over NVLink, partial rows
    # summed while read back): every rank must have mapped every peer, else all ranks leave it out
    peer = None
    if world > 1:
        import torch.distributed as dist
        from qwen_kernel_b200.expert_parallel import PeerExpertParallel
        why = ""
        try:
            peer = PeerExpertParallel(ctx, max_local_tokens=n_max, device=dev, device_barrier=True)
        except Exception as e:   # noqa: BLE001  (reported in the JSON line)
            why = f"{type(e).__name__}: {e}"[:200]
        ok = torch.tensor([0 if peer is None else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            peer = None
            out["peer_memory_unavailable"] = why or "a peer rank could not map the buffers"
    steps, warm = max(3, args.steps // 4), 3
    # the unsharded layer on ONE GPU at the same token counts, timed by rank 0 inside this run
    # (the other ranks wait): the denominator of the expert-parallel speed-up
    one_gpu_us = {}
    if world > 1:
        if rank == 0:
            c1 = pkg.Context(dims, n_layer=PL, max_tokens=Tmax, device=R.local_rank)
            for l, layer in enumerate(layers):
                c1.upload_layer(l, layer)
            x1 = torch.from_numpy(np.stack([syn.random_x(Tmax, dims.n_embd, SEED_X + 555 + l) for l in range(PL)])).to(dev)
            y1 = torch.empty_like(x1)
            for T1 in (t for t in (128, 2048, 4096) if t in PREFILL_CHUNKS):
                def step1():
                    for l in range(PL):
                        c1.moe_prefill(l, x1[l], T1, y1[l])
                for _ in range(warm):
                    step1()
                torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(steps):
                    step1()
                e1.record(stream)
                torch.cuda.synchronize(dev)
                one_gpu_us[T1] = e0.elapsed_time(e1) / steps / PL * 1e3
            c1.close()
            del x1, y1
            torch.cuda.empty_cache()
        R.barrier()
    for T in PREFILL_CHUNKS:
        n = T // world
        if n == 0:
            continue

        def step():
            for l in range(PL):
                if ep:
                    ep.forward(l, x[l], n, y[l])
                else:
                    ctx.moe_prefill(l, x[l], n, y[l])

        step(); R.barrier()
        k = min(n, 512) if rank == 0 else min(n, 8)   # rank 0 checks all of its rows (up to 512), the others a few
        want = orc.moe_layer(layers[0], x_np[0, :k], threads=orc.hardware_threads())["y"]
        err = syn.rel_err_rows(y[0, :k].cpu().numpy(), want)
        assert err < 2e-2, f"prefill T={T}: error {err}"
        n0 = ctx.launch_count()
        ms = timed(torch, R, stream, step, steps, warm) / PL     # per layer
        entry_ = {"us_per_layer": ms * 1e3, "tok_s": T / (ms * 1e-3), "rel_err_vs_oracle": R.max_over_ranks(err),
                  "tensor_tflops": T * TENSOR_FLOPS_PER_TOKEN / (ms * 1e-3) / 1e12,
                  "launches_per_layer": (ctx.launch_count() - n0) / ((steps + warm) * PL)}
        entry_["tensor_tflops_per_gpu"] = entry_["tensor_tflops"] / world
        entry_["frac_of_measured_bf16_burst"] = entry_["tensor_tflops_per_gpu"] / peaks["bf16_tflops"]
        if ep:
            send, recv = ep.last_counts
            off = sum(send) - send[rank]
            entry_["rows_sent_off_gpu_per_rank"] = off
            entry_["nvlink_bytes_per_rank_per_layer"] = off * (dims.n_embd * 4 + 160) + off * dims.n_embd * 4
            entry_["exchange"] = "NCCL all-to-all"
        if peer:
            def step_peer():
                for l in range(PL):
                    peer.forward(l, x[l], n, y[l], slot_rows=n)

            y.zero_()
            step_peer(); R.barrier()
            err_p = syn.rel_err_rows(y[0, :k].cpu().numpy(), want)
            assert err_p < 2e-2, f"peer-memory expert parallel T={T}: error {err_p}"
            n0 = ctx.launch_count()
            ms_p = timed(torch, R, stream, step_peer, steps, warm) / PL
            entry_["peer_memory"] = {"us_per_layer": ms_p * 1e3, "tok_s": T / (ms_p * 1e-3),
                                     "rel_err_vs_oracle": R.max_over_ranks(err_p),
                                     "launches_per_layer": (ctx.launch_count() - n0) / ((steps + warm) * PL),
                                     "exchange": "rows and partial rows stored into peer-mapped buffers over NVLink, two flag barriers (own kernel) per layer, one library call per layer"}
            if ep:   # same rows as the all-to-all form, but f16 on the way out (f32 partial rows on the way back)
                entry_["peer_memory"]["nvlink_bytes_per_rank_per_layer"] = off * (dims.n_embd * 2 + 160) + off * dims.n_embd * 4
            try:
                ctx.sync()   # a barrier wait that ran out surfaces here; every rank goes on with the same calls
            except Exception as e:   # noqa: BLE001  (reported in the JSON line)
                entry_["peer_memory"]["barrier_status"] = str(e)[:160]
            peer.device_barrier = False
            ms_n = timed(torch, R, stream, step_peer, steps, warm) / PL
            peer.device_barrier = True
            entry_["peer_memory"]["us_per_layer_with_nccl_barriers"] = ms_n * 1e3
            if T in (128, 4096):   # where the time goes: the six calls of one layer between events, mean over the layers
                names = ("push", "barrier1", "experts", "barrier2", "pull")
                acc = dict.fromkeys(names, 0.0)
                for l in range(PL):
                    ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
                    calls = (lambda: ctx.ep_push(l, x[l], n, n), ctx.ep_barrier,
                             lambda: ctx.ep_forward_slots(l, n, n), ctx.ep_barrier, lambda: ctx.ep_pull(n, n, y[l]))
                    ev[0].record(stream)
                    for i, call in enumerate(calls):
                        call()
                        ev[i + 1].record(stream)
                    torch.cuda.synchronize(dev)
                    for i, nm in enumerate(names):
                        acc[nm] += ev[i].elapsed_time(ev[i + 1]) * 1e3 / PL
                entry_["peer_memory"]["stages_us"] = acc
            # the peer-memory form is the product path: its figures lead the entry, the all-to-all form sits beside them
            pm = entry_.pop("peer_memory")
            a2a = {k: entry_[k] for k in ("us_per_layer", "tok_s", "rel_err_vs_oracle", "launches_per_layer", "exchange")}
            entry_.update(pm)
            entry_["tensor_tflops"] = T * TENSOR_FLOPS_PER_TOKEN / (pm["us_per_layer"] * 1e-6) / 1e12
            entry_["tensor_tflops_per_gpu"] = entry_["tensor_tflops"] / world
            entry_["frac_of_measured_bf16_burst"] = entry_["tensor_tflops_per_gpu"] / peaks["bf16_tflops"]
            entry_["nccl_all_to_all"] = a2a
        if T in one_gpu_us:
            entry_["us_per_layer_1gpu_same_run"] = one_gpu_us[T]
            entry_["speedup_vs_1gpu"] = one_gpu_us[T] / entry_["us_per_layer"]
        out["chunks"][str(T)] = entry_
    if world == 1 and Tmax >= 2048:
        ctx.profile_enable(True)
        T = 2048
        acc = {}
        for l in range(PL):
            ctx.moe_prefill(l, x[l], T, y[l])
            for kk, v in ctx.profile_read().items():
                acc[kk] = acc.get(kk, 0.0) + v * 1e3 / PL
        ctx.profile_enable(False)
        out["stages_us_at_2048"] = acc
        gu = acc.get("moe.gu", 0.0)
        if gu > 0:
            fl = T * dims.n_used * 2 * 2 * dims.n_ff * dims.n_embd
            out["roofline"] = {"bound": "tensor", "kernel": "gateup_iq3_kernel at 2048 tokens",
                               "achieved": fl / (gu * 1e-6) / 1e12, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                               "frac": fl / (gu * 1e-6) / 1e12 / peaks["bf16_tflops"],
                               "peak_source": peaks["source"] + " cuBLAS bf16 burst", "traffic": None}
    out["workload"] = ("moe_prefill: one layer, chunks of T tokens, tcgen05 expert GEMMs" if world == 1 else
                       f"expert-parallel moe layer: T tokens over {world} GPUs ({per} experts each), rows stored into the "
                       "owners' peer-mapped buffers over NVLink (NCCL all-to-all form beside it)")
    out["scaling"] = "strong"
    if world > 1:   # the figures the scaling claim rests on, short enough to ride in the line's config object
        out["summary"] = {str(T): {k: out["chunks"][str(T)].get(k) for k in
                                   ("us_per_layer", "us_per_layer_1gpu_same_run", "speedup_vs_1gpu", "rel_err_vs_oracle", "stages_us")}
                          for T in (128, 2048, 4096) if str(T) in out["chunks"]}
    R.barrier()
    ctx.close()
    return out


GEMV_SHAPES = ((4096, 2048), (2048, 4096), (8192, 2048))


def run_gemv_sweep(args, pkg, syn, torch, R: Ranks, orc, peaks):
    """Dense dequant-GEMV, batch 1, per format and shape.  Each case rotates over enough
    copies of the matrix (distinct addresses) that a pass reads more than twice the L2."""
    dev = R.dev
    ctx = pkg.Context(syn.Dims(), n_layer=1, max_tokens=1, device=R.local_rank)
    stream = torch.cuda.Stream(dev)   # a real stream: each pass over the copies is replayed as a CUDA graph
    ctx.set_stream(stream.cuda_stream)
    torch.cuda.set_stream(stream)
    cases = [(t, m, k) for (m, k) in GEMV_SHAPES for t in (syn.Q8_0, syn.Q6_K, syn.IQ4_XS, syn.IQ3_XXS, syn.F16)]
    cases.append((syn.Q6_K, 151936, 2048))
    # the reference quotes its GEMV bandwidths on matrices of 96 MB and more: the same per format
    cases += [(t, 65536, 2048) for t in (syn.Q8_0, syn.Q6_K, syn.IQ4_XS, syn.IQ3_XXS, syn.F16)]
    names = {syn.Q8_0: "q8_0", syn.Q6_K: "q6_k", syn.IQ4_XS: "iq4_xs", syn.IQ3_XXS: "iq3_xxs", syn.F16: "f16"}
    out = {}
    for t, M, K in cases:
        W = syn.random_blocks(t, M, K, SEED_W + 5, "gemv")
        nbytes = W.nbytes
        stride = (nbytes + 255) // 256 * 256
        copies = max(1, min(64, -(-300_000_000 // stride)))
        buf = torch.zeros(copies * stride + 256, dtype=torch.uint8, device=dev)
        w_dev = torch.from_numpy(W).to(dev)
        for c in range(copies):
            buf[c * stride:c * stride + nbytes] = w_dev
        xv = syn.random_x(1, K, SEED_X + 9)
        x = torch.from_numpy(xv).to(dev)
        y = torch.empty(M, dtype=torch.float32, device=dev)
        base = buf.data_ptr()

        def step():
            for c in range(copies):
                ctx.gemv(t, base + c * stride, x, y, M, K, 1)

        step(); R.barrier()
        want = orc.gemv(t, W, xv.reshape(-1), M, K, threads=orc.hardware_threads())
        err = syn.rel_err_rows(y.cpu().numpy().reshape(1, -1), want.reshape(1, -1))
        assert err < 1e-5, f"gemv {names[t]} {M}x{K}: error {err}"
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        ms = timed(torch, R, stream, graph.replay, 5, 3) / copies
        del graph
        gb = syn.gemv_bytes(t, M, K)
        out[f"{names[t]}_{M}x{K}"] = {"us": ms * 1e3, "gbs": gb / (ms * 1e-3) / 1e9,
                                      "frac_of_measured_copy": gb / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "copies": copies}
        del buf, w_dev
    torch.cuda.set_stream(torch.cuda.default_stream(dev))
    ctx.set_stream(0)
    # dense prefill projections on the tensor cores: Y[n][M] = X[n][K] . W^T (compute-bound at these
    # n, so the matrix staying in L2 does not flatter the figure; the activations are 16-32 MB per call)
    for t, M, K, n in ((syn.Q8_0, 4096, 2048, 2048), (syn.IQ4_XS, 4096, 2048, 2048), (syn.Q8_0, 8192, 2048, 512)):
        W = syn.random_blocks(t, M, K, SEED_W + 6, "gemm")
        ctx.dense_upload(0, t, W, M, K)
        xg = torch.from_numpy(syn.random_x(n, K, SEED_X + 11)).to(dev)
        yg = torch.empty((n, M), dtype=torch.float32, device=dev)
        ctx.dense_gemm(0, xg, n, yg); R.barrier()
        want = orc.gemv(t, W, xg[0].cpu().numpy(), M, K, threads=orc.hardware_threads())
        err = syn.rel_err_rows(yg[:1].cpu().numpy(), want.reshape(1, -1))
        assert err < 2e-2, f"dense gemm {names[t]} {M}x{K}: error {err}"
        ms = timed(torch, R, torch.cuda.current_stream(dev), lambda: ctx.dense_gemm(0, xg, n, yg), 5, 3)
        out[f"gemm_{names[t]}_{M}x{K}_n{n}"] = {"us": ms * 1e3, "tflops": 2.0 * n * M * K / (ms * 1e-3) / 1e12,
                                                "frac_of_measured_bf16_burst": 2.0 * n * M * K / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    ctx.close()
    return out


def run_batch1(ctx, syn, torch, R, stream, L, dims, x_all, peaks, orc, layers_keep):
    """BASELINE configuration 0: one MoE layer, decode batch 1 (the reference's `qk moe <layer>`
    harness, src/main.cpp:1221-1243: us per layer and GB/s over the weight bytes one token
    touches).  The call rotates over all L layers of the stack (one token through each, replayed
    as a graph), so every layer's weights come from HBM, not from L2: a cold figure, as stated."""
    dev = R.dev
    with torch.cuda.stream(stream):
        x1 = torch.from_numpy(np.ascontiguousarray(x_all[:, :1])).to(dev)
        y1 = torch.empty_like(x1)
    ctx.moe_decode_stack(0, L, x1, 1, y1); R.barrier()
    ref = orc.moe_layer(layers_keep[0], x_all[0, :1])
    err = syn.rel_err_rows(y1[0].cpu().numpy(), ref["y"])
    assert err < 1e-5, f"batch-1 layer output error {err}"
    ms = timed(torch, R, stream, lambda: ctx.moe_decode_stack(0, L, x1, 1, y1), 20, 3) / L
    nbytes = syn.layer_touched_bytes(dims, syn.F16, syn.IQ3_XXS, syn.IQ4_XS, dims.n_used)
    return {"workload": f"one layer, one token; rotating over {L} layers so weights stream from HBM (cold)",
            "us_per_layer": ms * 1e3, "active_bytes_per_layer": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
            "frac_of_measured_copy": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "frac_of_nominal_8TBs": nbytes / (ms * 1e-3) / 8e12,
            "rel_err_vs_oracle": err}


def time_kernels(ctx, pkg, syn, torch, dev, stream, L, S, x_dev, distinct, dims, reps=5):
    """Average duration of every stage of the fused decode sequence (one launch per layer
    per pass), from CUDA events recorded on the launching stream between the stages
    (qkm_profile_*), with the algorithmic weight bytes each stage touches."""
    rb = syn.row_bytes
    mean_u = float(np.mean(distinct))
    # the shared expert's matrices ride inside the routed kernels of the fused sequence
    stage_bytes = {
        "moe.route": dims.n_expert * rb(syn.F16, dims.n_embd) + dims.n_embd * 4,
        "moe.gu": mean_u * 2 * dims.n_ff * rb(syn.IQ3_XXS, dims.n_embd) + 2 * dims.n_ff * rb(syn.Q8_0, dims.n_embd),
        "moe.dn": mean_u * dims.n_embd * rb(syn.IQ4_XS, dims.n_ff) + dims.n_embd * rb(syn.Q8_0, dims.n_ff),
    }
    y = torch.empty(S, dims.n_embd, device=dev)
    ctx.profile_enable(True)
    acc = {}
    for _ in range(reps):
        for l in range(L):
            ctx.moe_decode(l, x_dev[l], S, y)
            for k, v in ctx.profile_read().items():
                acc[k] = acc.get(k, 0.0) + v
    ctx.profile_enable(False)
    out = {}
    for k, v in acc.items():
        ms = v / (reps * L)
        nbytes = stage_bytes.get(k, 0)
        out[k] = {"name": k, "ms_per_layer": ms, "bytes_per_launch": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--slots", type=int, default=16, help="decode slots per GPU")
    ap.add_argument("--sub-layers", type=int, default=8, help="distinct layers the prefill / expert-parallel cases rotate over")
    ap.add_argument("--no-sub", action="store_true", help="only the headline decode workload")
    ap.add_argument("--prefill-tokens", default="", help="comma-separated chunk sizes of the prefill / expert-parallel cases "
                    "(default: 128,256,512,2048,4096); a single size keeps a profiler capture of their kernels small")
    args = ap.parse_args()
    args.sub_layers = max(1, min(args.sub_layers, args.layers))
    if args.prefill_tokens:
        global PREFILL_CHUNKS
        PREFILL_CHUNKS = tuple(sorted(int(v) for v in args.prefill_tokens.split(",") if v))
    pkg = entry.package()
    syn = pkg.synth
    if args.impl == "reference":
        return run_reference_arm(args, syn)
    pkg.load_library()  # fails loudly if the CUDA library was not built
    return run_ours(args, pkg, syn)


if __name__ == "__main__":
    main()
