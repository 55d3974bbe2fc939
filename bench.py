#!/usr/bin/env python
"""Benchmark of the quantized MoE feed-forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|prefill|gemv] [--layers L] [--slots S] [--tokens T]

One JSON line on stdout (rank 0).  The default workload is the decode
configuration: a stack of 40 MoE layers (2048 / 512 / 256 experts / top-8, F16
router, IQ3_XXS gate+up, IQ4_XS down, Q8_0 shared expert, per-layer seeds), 16
concurrent slots with independent N(0,1) hidden rows per layer.  A step is one
pass of the 16 rows through the 40 layers; value = tokens / second through the
stack.  Weights are seeded synthetic ggml blocks (no model file is needed).

Timing: W >= 3 untimed steps, then K steps between two CUDA events on the
launching stream, bracketed by barrier + synchronize; max over ranks.  The
working set of a step (about 40 x 143 MB of weights) is far larger than the
126 MB L2, so every step streams its weights from HBM.
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
    """HBM GB/s and bf16 TF/s measured on this pool (driver-written), else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
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
                "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ------------------------------------------------------------------ CPU arm (oracle port)

def cpu_moe_sample(syn, orc_mod, dims, n_slots, layers_sample, threads, router_type, gateup_type, down_type):
    """Times the CPU path (quants.h-style dequant + scalar f32 loop, restated in
    oracle/qkm_oracle.cpp) on `layers_sample` layers x n_slots rows with `threads`
    host threads.  Returns seconds per (layer x n_slots rows)."""
    orc = orc_mod.Oracle()
    total = 0.0
    for l in range(layers_sample):
        layer = syn.make_layer(dims, SEED_W, l, router_type, gateup_type, down_type)
        x = syn.random_x(n_slots, dims.n_embd, SEED_X + l)
        t0 = time.perf_counter()
        orc.moe_layer(layer, x, acc=orc_mod.ACC_F32, threads=threads)
        total += time.perf_counter() - t0
    return total / layers_sample


def run_reference_arm(args, syn):
    """The reference's CPU implementation of the path, timed on the host cores."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    orc_mod = entry.oracle_module()
    orc_mod.build(ref=False)
    dims = syn.Dims()
    threads = orc_mod.Oracle().hardware_threads() or 1
    n_layers, n_slots = args.layers, args.slots * max(1, args.gpus)
    sample_layers = 1
    per_layer = []
    for _ in range(args.warmup):
        cpu_moe_sample(syn, orc_mod, dims, n_slots, sample_layers, threads, syn.F16, syn.IQ3_XXS, syn.IQ4_XS)
    for _ in range(args.steps):
        per_layer.append(cpu_moe_sample(syn, orc_mod, dims, n_slots, sample_layers, threads, syn.F16, syn.IQ3_XXS, syn.IQ4_XS))
    sec_per_step = float(np.mean(per_layer)) * n_layers
    value = n_slots / sec_per_step
    line = {
        "impl": "reference", "metric": "moe_decode_tok_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": decode_config(args, n_slots),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"{sample_layers} of {n_layers} layers x {n_slots} rows per step, scaled by layers"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def decode_config(args, n_slots):
    return {"workload": f"moe_decode_stack: {args.layers} layers x {n_slots} slots, n_embd 2048, n_ff 512, "
                        "256 experts top-8, F16 router, IQ3_XXS gate/up, IQ4_XS down, Q8_0 shared",
            "layers": args.layers, "slots": n_slots, "l2": "working set per step >> 126 MB L2 (weights stream from HBM)"}


# ------------------------------------------------------------------ GPU arm

def run_decode(args, pkg, syn):
    import torch
    rank, local_rank, world = dist_env()
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dims = syn.Dims()
    L, S = args.layers, args.slots
    if world > 1:
        raise SystemExit("expert-parallel decode is launched through --workload ep (not built into this path yet)")

    ctx = pkg.Context(dims, n_layer=L, max_tokens=S, device=local_rank)
    stream = torch.cuda.Stream(dev)   # a real stream: the stack is replayed as a CUDA graph
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    orc_mod = entry.oracle_module()
    orc = orc_mod.Oracle()
    distinct, x_all = [], np.empty((L, S, dims.n_embd), np.float32)
    layer0 = None
    for l in range(L):
        layer = syn.make_layer(dims, SEED_W, l, syn.F16, syn.IQ3_XXS, syn.IQ4_XS)
        ctx.upload_layer(l, layer)
        x_all[l] = syn.random_x(S, dims.n_embd, SEED_X + l)
        if l == 0:
            layer0 = layer
    x_dev = torch.from_numpy(x_all).to(dev)
    y_dev = torch.empty_like(x_dev)
    x_pin = torch.from_numpy(x_all).pin_memory()
    y_pin = torch.empty_like(x_pin).pin_memory()

    def step():
        ctx.moe_decode_stack(0, L, x_dev, S, y_dev)

    def barrier():
        torch.cuda.synchronize(dev)

    # correctness of what is being timed: layer 0 against the oracle
    step(); barrier()
    ref0 = orc.moe_layer(layer0, x_all[0], threads=orc.hardware_threads())
    err0 = syn.rel_err_rows(y_dev[0].cpu().numpy(), ref0["y"])
    assert err0 < 1e-5, f"layer 0 output error {err0}"

    # distinct experts per layer (for the algorithmic byte count), from the device's own routing
    for l in range(L):
        ctx.moe_decode(l, x_dev[l], S, y_dev[l])
        ids = ctx.last_sel(S)["ids"][:, :dims.n_used]
        distinct.append(len(np.unique(ids)))
    bytes_step = sum(syn.layer_touched_bytes(dims, syn.F16, syn.IQ3_XXS, syn.IQ4_XS, u) for u in distinct)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = ctx.launch_count()
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    launches = ctx.launch_count() - n0
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    value = S / (ms * 1e-3)

    # end to end: pinned host rows in, host rows out, every step
    for _ in range(2):
        ctx.moe_decode_stack_host(0, L, x_pin.data_ptr(), S, y_pin.data_ptr())
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ctx.moe_decode_stack_host(0, L, x_pin.data_ptr(), S, y_pin.data_ptr())
    e2e_s = (time.perf_counter() - t0) / args.steps
    assert np.array_equal(y_pin[0].numpy(), y_dev[0].cpu().numpy())

    # per-kernel timing of the dominant kernels over the same inputs (CUDA events, this stream)
    kern = time_kernels(ctx, pkg, syn, torch, dev, stream, L, S, x_dev, distinct, dims)
    peaks = measured_peaks()
    dom = max(kern.values(), key=lambda k: k["ms_per_layer"])
    roof = {"bound": "hbm", "kernel": dom["name"], "achieved": dom["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": dom["gbs"] / peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy bandwidth",
            "frac_of_nominal_8TBs": dom["gbs"] / 8000.0, "traffic": None,
            "bytes_per_launch": dom["bytes_per_launch"], "ms_per_launch": dom["ms_per_layer"]}

    threads = orc.hardware_threads() or 1
    cpu_sec_layer = cpu_moe_sample(syn, orc_mod, dims, S, 2, threads, syn.F16, syn.IQ3_XXS, syn.IQ4_XS)
    cpu_val = S / (cpu_sec_layer * L)
    line = {
        "metric": "moe_decode_tok_s", "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": decode_config(args, S),
        "hbm": {"algorithmic_bytes_per_step": bytes_step, "gbs": bytes_step / (ms * 1e-3) / 1e9,
                "frac_of_measured_copy": bytes_step / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "frac_of_nominal_8TBs": bytes_step / (ms * 1e-3) / 8e12,
                "distinct_experts_per_layer_mean": float(np.mean(distinct))},
        "us_per_layer": ms * 1e3 / L,
        "roofline": roof, "kernels": kern,
        "cpu_baseline": {"value": cpu_val, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"2 of {L} layers x {S} rows on the host cores, scaled by layers"},
        "e2e": {"value": S / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": int(x_pin.numel() * 4),
                "d2h_bytes_per_step": int(y_pin.numel() * 4), "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(launches), "clocks": clocks, "parity": {"layer0_rel_err": err0},
    }
    print(json.dumps(line), flush=True)
    ctx.close()


def time_kernels(ctx, pkg, syn, torch, dev, stream, L, S, x_dev, distinct, dims, reps=5):
    """Average duration of every stage of the fused decode sequence (one launch per layer
    per pass), from CUDA events recorded on the launching stream between the stages
    (qkm_profile_*), with the algorithmic weight bytes each stage touches."""
    rb = syn.row_bytes
    mean_u = float(np.mean(distinct))
    stage_bytes = {
        "moe.route": dims.n_expert * rb(syn.F16, dims.n_embd) + dims.n_embd * 4,
        "moe.shared_gu": 2 * dims.n_ff * rb(syn.Q8_0, dims.n_embd),
        "moe.gu": mean_u * 2 * dims.n_ff * rb(syn.IQ3_XXS, dims.n_embd),
        "moe.dn": mean_u * dims.n_embd * rb(syn.IQ4_XS, dims.n_ff),
        "moe.shared_dn": dims.n_embd * rb(syn.Q8_0, dims.n_ff),
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
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "gemv"])
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--slots", type=int, default=16)
    ap.add_argument("--tokens", type=int, default=2048)
    args = ap.parse_args()
    pkg = entry.package()
    syn = pkg.synth
    if args.impl == "reference":
        return run_reference_arm(args, syn)
    pkg.load_library()  # fails loudly if the CUDA library was not built
    if args.workload == "decode":
        return run_decode(args, pkg, syn)
    raise SystemExit(f"workload {args.workload} not available yet")


if __name__ == "__main__":
    main()
