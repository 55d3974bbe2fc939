"""A CPU engine with the interface `ExpertParallel` drives (ep_dispatch / ep_shared /
ep_expert_forward / ep_combine) and the one `PeerExpertParallel` drives (ep_peer_* / ep_push /
ep_forward_slots / ep_pull, with POSIX shared memory standing in for peer-mapped device
buffers), computing with the oracle.  Test infrastructure only: it
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

    # ---- peer-memory form: receive buffers live in shared memory, "handles" are their names
    def ep_peer_setup(self, n_ranks, rank, slot_cap):
        from multiprocessing import shared_memory
        assert (n_ranks, rank) == (self.world, self.rank)
        E, rows = self.dims.n_embd, n_ranks * slot_cap
        self.cap = slot_cap
        self.shm = [shared_memory.SharedMemory(create=True, size=max(nb, 1)) for nb in (rows * E * 4, rows * 160, rows * E * 4)]
        self.peer_shm = {}
        self.peers = {rank: self._views(self.shm, rows)}
        self.peers[rank][1][:] = 0xFF

    def _views(self, shm, rows):
        E = self.dims.n_embd
        return (np.ndarray((rows, E), np.float32, shm[0].buf), np.ndarray((rows, 160), np.uint8, shm[1].buf),
                np.ndarray((rows, E), np.float32, shm[2].buf))

    def ep_peer_export(self) -> bytes:
        return b"".join(s.name.encode().ljust(64, b"\0") for s in self.shm)

    def ep_peer_import(self, peer, handles: bytes):
        from multiprocessing import shared_memory
        names = [handles[64 * i:64 * i + 64].rstrip(b"\0").decode() for i in range(3)]
        self.peer_shm[peer] = [shared_memory.SharedMemory(name=nm) for nm in names]
        self.peers[peer] = self._views(self.peer_shm[peer], self.world * self.cap)

    def _need(self, n):
        owner = self.sel["ids"][:n, :self.dims.n_used] // self.per
        return np.stack([(owner == r).any(axis=1) for r in range(self.world)], axis=1)   # [n][ranks]

    def ep_push(self, layer, x, n, slot_rows):
        xn = x.numpy()[:n]
        self.sel, _ = self.orc.route(self.layers[layer], xn)
        need = self._need(n) if n else np.zeros((0, self.world), bool)
        empty = np.zeros(160, np.uint8)
        empty[:64] = 0xFF
        base = self.rank * slot_rows
        for d in range(self.world):
            xr, sr, _ = self.peers[d]
            for i in range(slot_rows):
                if i < n and need[i, d]:
                    xr[base + i] = xn[i]
                    sr[base + i] = self.sel[i:i + 1].view(np.uint8).reshape(160)
                else:
                    sr[base + i] = empty
                    if i < n and d == self.rank:      # own rows always travel: the shared expert reads them
                        xr[base + i] = xn[i]
                        sr[base + i, 64:] = self.sel[i:i + 1].view(np.uint8).reshape(160)[64:]

    def ep_forward_slots(self, layer, slot_rows, n_shared=None):
        from conftest import entry
        xr, sr, _ = self.peers[self.rank]
        rows = self.world * slot_rows
        sel = sr[:rows].copy().reshape(-1).view(entry.package().SEL_DTYPE)
        live = (sel["ids"][:, :self.dims.n_used] < self.dims.n_expert).any(axis=1)
        pr = np.zeros((rows, self.dims.n_embd), np.float32)
        if live.any():
            idx = np.nonzero(live)[0]
            out = self.orc.moe_layer(self.slices[layer], np.ascontiguousarray(xr[idx]), sel_in=sel[idx].copy(), with_shared=False)
            pr[idx] = out["y"]
        self.shared_in_partial = n_shared is not None
        if n_shared:
            own = slice(self.rank * slot_rows, self.rank * slot_rows + n_shared)
            sh = sel[own].copy()
            sh["ids"][:, :self.dims.n_used] = 1       # experts outside the one-expert slice: shared only
            lone = self.layers[layer].expert_slice(0, 1)
            pr[own] += self.orc.moe_layer(lone, np.ascontiguousarray(xr[own]), sel_in=sh, with_shared=True)["y"]
            live[own] = True
        # every live partial row goes to its source rank's return buffer, at (this rank, token)
        for r in np.nonzero(live)[0]:
            src, i = divmod(int(r), slot_rows)
            self.peers[src][2][self.rank * slot_rows + i] = pr[r]

    def ep_pull(self, n, slot_rows, y):
        if n == 0:
            return
        need = self._need(n)
        if self.shared_in_partial:
            need[:, self.rank] = True
        back = self.peers[self.rank][2]
        out = np.zeros((n, self.dims.n_embd), np.float32)
        for d in range(self.world):
            for t in range(n):
                if need[t, d]:
                    out[t] += back[d * slot_rows + t]
        if not self.shared_in_partial:
            out += self.y2
        y.numpy()[:n] = out

    def close_peers(self):
        self.peers = {}
        for lst in self.peer_shm.values():
            for s in lst:
                s.close()
        for s in getattr(self, "shm", []):
            s.close()
            s.unlink()
