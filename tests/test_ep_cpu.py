"""Expert-parallel exchange logic on CPU: world_size-2 and -4 gloo ranks drive
`ExpertParallel` with an oracle-backed engine; every rank's rows must equal the unsharded
oracle layer within the f32 decode tolerance (1e-5, row-scaled)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world,tokens,mode", [(2, 12, "alltoall"), (4, 9, "alltoall"), (2, 1, "alltoall"),
                                               (2, 12, "peer"), (4, 9, "peer"), (2, 1, "peer")])
def test_expert_parallel_gloo(world, tokens, mode, orc):  # `orc` builds the oracle once, before the ranks start
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "ep_worker.py"), "--rank", str(r), "--world",
                               str(world), "--port", str(port), "--tokens", str(tokens), "--mode", mode],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out[-3000:]}"
    assert "EP_CPU" in outs[0]


def test_plan_send_order():
    from ep_cpu_engine import plan_send, INVALID
    ids = np.zeros((3, 16), np.uint32)
    ids[0, :2] = [0, 5]      # ranks 0 and 1 (4 experts per rank)
    ids[1, :2] = [6, 7]      # rank 1 only
    ids[2, :2] = [12, 1]     # ranks 3 and 0
    counts, send_tok, send_pos = plan_send(ids, 2, 4, 4)
    assert counts == [2, 2, 0, 1]
    assert send_tok.tolist() == [0, 2, 0, 1, 2]
    assert send_pos[1].tolist() == [INVALID, 3, INVALID, INVALID]
    assert send_pos[2].tolist() == [1, INVALID, INVALID, 4]
