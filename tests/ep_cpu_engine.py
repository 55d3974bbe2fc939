"""A CPU engine with the interface `ExpertParallel` drives (ep_dispatch / ep_shared /
ep_expert_forward / ep_combine), computing with the oracle.  Test infrastructure only: it
lets the exchange logic (send order, split sizes, combine order) run as gloo ranks without a
GPU, and documents the contract of the four calls in plain numpy."""
import numpy as np

INVALID = 0xFFFFFFFF


def plan_send(ids: np.ndarray, n_used: int, experts_per_rank: int, n_ranks: int):
    """counts[r], send_tok (rank by rank, ascending token), send_pos[t][r]."""
    T = ids.shape[0]
    owner = ids[:, :n_used] // experts_per_rank
    counts, send_tok = [], []
    send_pos = np.full((T, n_ranks), INVALID, np.uint32)
    for r in range(n_ranks):
        toks = np.nonzero((owner == r).any(axis=1))[0]
        for t in toks:
            send_pos[t, r] = len(send_tok)
            send_tok.append(int(t))
        counts.append(len(toks))
    return counts, np.asarray(send_tok, np.int64), send_pos


class OracleEngine:
    def __init__(self, orc, layers, rank: int, world: int):
        self.orc, self.layers, self.rank, self.world = orc, layers, rank, world
        d = layers[0].dims
        self.dims = d
        self.per = d.n_expert // world
        self.slices = [L.expert_slice(rank * self.per, self.per) for L in layers]
        self.sel = self.send_pos = self.y2 = None

    def ep_dispatch(self, layer, x, n, n_ranks, xsend, selsend):
        assert n_ranks == self.world
        xn = x.numpy()[:n]
        self.sel, _ = self.orc.route(self.layers[layer], xn)
        counts, send_tok, self.send_pos = plan_send(self.sel["ids"], self.dims.n_used, self.per, n_ranks)
        k = len(send_tok)
        xsend.numpy()[:k] = xn[send_tok]
        selsend.numpy()[:k] = self.sel[send_tok].view(np.uint8).reshape(k, 160)
        return counts

    def ep_dispatch_dev(self, layer, x, n, n_ranks, xsend, selsend, counts_dev):
        counts = self.ep_dispatch(layer, x, n, n_ranks, xsend, selsend)
        counts_dev.numpy()[:] = np.asarray(counts, np.int32)

    def ep_shared(self, layer, x, n):
        # shared expert only: a selection whose experts all live outside the one-expert slice
        d = self.dims
        lone = self.layers[layer].expert_slice(0, 1)
        sel = self.sel.copy()
        sel["ids"][:, :d.n_used] = 1
        self.y2 = self.orc.moe_layer(lone, x.numpy()[:n], sel_in=sel, with_shared=True)["y"]

    def ep_expert_forward(self, layer, xrecv, selrecv, n_recv, partial):
        if n_recv == 0:
            return
        from conftest import entry
        sel = selrecv.numpy()[:n_recv].reshape(-1).view(entry.package().SEL_DTYPE).copy()
        out = self.orc.moe_layer(self.slices[layer], xrecv.numpy()[:n_recv], sel_in=sel, with_shared=False)
        partial.numpy()[:n_recv] = out["y"]

    def ep_combine(self, n, n_ranks, back, y):
        b = back.numpy()
        out = np.zeros((n, self.dims.n_embd), np.float32)
        for r in range(n_ranks):
            for t in range(n):
                p = self.send_pos[t, r]
                if p != INVALID:
                    out[t] += b[p]
        out += self.y2
        y.numpy()[:n] = out
