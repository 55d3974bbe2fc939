"""One NCCL rank of the multi-GPU expert-parallel test (started by test_gpu_ep.py, one process
per GPU): runs a layer through `PeerExpertParallel` (rows stored into peer-mapped buffers) and
through `ExpertParallel` (all-to-all) and checks this rank's rows against the unsharded oracle
layer.  Tolerance 2e-2 (tensor-core expert GEMMs) against the f64 oracle."""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import __graft_entry__ as entry  # noqa: E402

TOL = 2e-2


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--port", type=int, required=True)
    a = ap.parse_args()
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(a.port)
    torch.cuda.set_device(a.rank)
    dev = torch.device("cuda", a.rank)
    dist.init_process_group("nccl", rank=a.rank, world_size=a.world, device_id=dev)
    pkg = entry.package()
    syn = pkg.synth
    omod = entry.oracle_module()
    omod.build(ref=False)
    orc = omod.Oracle()
    from qwen_kernel_b200.expert_parallel import ExpertParallel, PeerExpertParallel

    dims = syn.Dims()
    per = dims.n_expert // a.world
    layers = [syn.make_layer(dims, seed=91, layer=l) for l in range(2)]
    cap = 160
    ctx = pkg.Context(dims, n_layer=2, max_tokens=cap * a.world, device=a.rank, expert_first=a.rank * per, expert_count=per)
    for l, layer in enumerate(layers):
        ctx.upload_layer(l, layer.expert_slice(a.rank * per, per))
    peer = PeerExpertParallel(ctx, max_local_tokens=cap, device=dev)
    a2a = ExpertParallel(ctx, dims.n_embd, dims.n_used, max_local_tokens=cap, max_recv_rows=cap * a.world, device=dev)
    worst = 0.0
    for T_all in (6 * a.world, 150 * a.world + 7):
        cut = [T_all * r // a.world for r in range(a.world + 1)]
        x_all = syn.random_x(T_all, dims.n_embd, seed=17 + T_all)
        lo, hi = cut[a.rank], cut[a.rank + 1]
        n = hi - lo
        rows = max(cut[r + 1] - cut[r] for r in range(a.world))
        x = torch.from_numpy(np.ascontiguousarray(x_all[lo:hi])).to(dev)
        y = torch.zeros_like(x)
        y2 = torch.zeros_like(x)
        for rep in range(3):              # back-to-back layers reuse the buffers
            for l in range(2):
                peer.device_barrier = bool(rep & 1)          # all-reduce barriers, then the library's own
                peer.forward(l, x, n, y, slot_rows=rows)
                a2a.forward(l, x, n, y2)
                want = orc.moe_layer(layers[l], x_all[lo:hi], threads=orc.hardware_threads())["y"]
                worst = max(worst, syn.rel_err_rows(y.cpu().numpy(), want), syn.rel_err_rows(y2.cpu().numpy(), want))
    ctx.sync()                                    # a device barrier that gave up would raise here
    ok = torch.tensor([worst], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MAX)
    if a.rank == 0:
        print("EP_GPU worst", float(ok.item()), flush=True)
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()
    sys.exit(0 if worst < TOL else 1)


if __name__ == "__main__":
    main()
