"""One gloo rank of the CPU expert-parallel test (started by test_ep_cpu.py):
runs `ExpertParallel.forward` with the oracle-backed engine and checks this rank's rows
against the unsharded oracle layer."""
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
from ep_cpu_engine import OracleEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("--tokens", type=int, default=12)
    ap.add_argument("--mode", choices=("alltoall", "peer"), default="alltoall")
    a = ap.parse_args()
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(a.port)
    dist.init_process_group("gloo", rank=a.rank, world_size=a.world)
    pkg = entry.package()
    syn = pkg.synth
    omod = entry.oracle_module()
    omod.build(ref=False)
    orc = omod.Oracle()
    from qwen_kernel_b200.expert_parallel import ExpertParallel, PeerExpertParallel, shard_range

    dims = syn.Dims(n_embd=256, n_ff=256, n_expert=16, n_used=4)
    layers = [syn.make_layer(dims, seed=77, layer=l) for l in range(2)]
    assert shard_range(dims.n_expert, a.rank, a.world) == (a.rank * dims.n_expert // a.world, dims.n_expert // a.world)
    # uneven token counts per rank, rank 1 may even have none
    T_all = a.tokens
    cut = [0] + [T_all * (r + 1) // a.world + (1 if r == 0 else 0) for r in range(a.world)]
    cut[-1] = T_all
    x_all = syn.random_x(T_all, dims.n_embd, seed=5)
    lo, hi = cut[a.rank], cut[a.rank + 1]
    n = hi - lo
    x = torch.from_numpy(np.ascontiguousarray(x_all[lo:hi]).copy()) if n else torch.zeros((1, dims.n_embd))
    y = torch.zeros((max(n, 1), dims.n_embd))
    eng = OracleEngine(orc, layers, a.rank, a.world)
    if a.mode == "peer":
        ep = PeerExpertParallel(eng, max_local_tokens=T_all, device="cpu")
    else:
        ep = ExpertParallel(eng, dims.n_embd, dims.n_used, max_local_tokens=T_all, max_recv_rows=T_all,
                            device="cpu")
    worst = 0.0
    n_most = max(cut[r + 1] - cut[r] for r in range(a.world))
    for l in range(2):
        if a.mode == "peer":
            ep.forward(l, x, n, y, slot_rows=n_most if l else None)   # once with the full slots, once tight
        else:
            ep.forward(l, x, n, y)
            send, recv = ep.last_counts
            assert len(send) == a.world and sum(send) <= n * min(a.world, dims.n_used)
        if n:
            want = orc.moe_layer(layers[l], x_all[lo:hi])["y"]
            got = y.numpy()[:n]
            rms = np.sqrt((want.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
            err = np.abs(got - want) / np.maximum(np.abs(want), rms)
            worst = max(worst, float(err.max()))
    ok = torch.tensor([1.0 if worst <= 1e-5 else 0.0, worst])
    gathered = [torch.zeros(2) for _ in range(a.world)]
    dist.all_gather(gathered, ok)
    if a.rank == 0:
        print("EP_CPU", [tuple(g.tolist()) for g in gathered], flush=True)
    dist.barrier()
    if a.mode == "peer":
        eng.close_peers()
    dist.destroy_process_group()
    sys.exit(0 if worst <= 1e-5 else 1)


if __name__ == "__main__":
    main()
