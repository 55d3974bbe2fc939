"""Expert-parallel MoE layer across the GPUs of one node: one process per GPU, experts
sharded contiguously (rank r of G owns experts [r*E/G, (r+1)*E/G)), tokens data-parallel,
one all-to-all each way per layer.

The reference engine is single-GPU; what is kept from it is the per-(token, expert)
arithmetic (src/main.cpp:1351-1369) and the buffer formats (the 160-byte selection record,
f32 rows).  A token's row travels once to every rank that owns at least one of its selected
experts; that rank returns one partial row, already weighted and summed over its experts.

The engine object does the compute on this rank's device: `qwen_kernel_b200.Context` opened
with this rank's expert range (its `ep_*` methods call the C ABI's `qkm_ep_*`).  The
exchange is `torch.distributed.all_to_all_single` with split sizes: NCCL over NVLink between
GPUs; tests run the same code over gloo with an engine that computes on the CPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

SEL_BYTES = 160


def shard_range(n_expert: int, rank: int, world: int):
    """(expert_first, expert_count) of `rank`: equal contiguous shards."""
    if n_expert % world:
        raise ValueError(f"n_expert {n_expert} is not divisible by {world} ranks")
    per = n_expert // world
    return rank * per, per


class ExpertParallel:
    """Runs MoE layers over a process group.  All buffers are allocated once."""

    def __init__(self, engine, n_embd: int, n_used: int, max_local_tokens: int, max_recv_rows: int,
                 device, group=None):
        self.engine, self.group = engine, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n_embd, self.device = n_embd, device
        fan = min(self.world, n_used)
        send_rows = max_local_tokens * fan
        self.max_local, self.max_recv = max_local_tokens, max_recv_rows
        f32, u8 = torch.float32, torch.uint8
        self.xsend = torch.empty((send_rows, n_embd), dtype=f32, device=device)
        self.selsend = torch.empty((send_rows, SEL_BYTES), dtype=u8, device=device)
        self.back = torch.empty((send_rows, n_embd), dtype=f32, device=device)
        self.xrecv = torch.empty((max_recv_rows, n_embd), dtype=f32, device=device)
        self.selrecv = torch.empty((max_recv_rows, SEL_BYTES), dtype=u8, device=device)
        self.partial = torch.empty((max_recv_rows, n_embd), dtype=f32, device=device)
        self.counts_dev = torch.zeros(2 * self.world, dtype=torch.int32, device=device)   # sent | received
        self.last_counts = None

    def forward(self, layer: int, x: torch.Tensor, n: int, y: torch.Tensor) -> None:
        """y[:n] = MoE layer `layer` of the n local rows x[:n] (all ranks call this together)."""
        if n > self.max_local:
            raise ValueError(f"{n} local tokens exceed the {self.max_local} this object was sized for")
        eng, W = self.engine, self.world
        # rows per destination stay on the device, are exchanged, and come to the host once
        eng.ep_dispatch_dev(layer, x, n, W, self.xsend, self.selsend, self.counts_dev[:W])
        dist.all_to_all_single(self.counts_dev[W:], self.counts_dev[:W], group=self.group)
        both = [int(v) for v in self.counts_dev.tolist()]
        send, recv = both[:W], both[W:]
        n_send, n_recv = sum(send), sum(recv)
        # an overflow is decided by all ranks together: a rank that raised alone would leave its
        # peers blocked in the next collective
        over = torch.tensor([max(0, n_recv - self.max_recv)], dtype=torch.int32, device=self.device)
        dist.all_reduce(over, op=dist.ReduceOp.MAX, group=self.group)
        if int(over.item()) > 0:
            raise RuntimeError(f"rank {self.rank}: {n_recv} rows arrive here, the buffers hold {self.max_recv}; "
                               f"the fullest rank is {int(over.item())} rows over (every rank raises)")
        self.last_counts = (send, recv)
        w1 = dist.all_to_all_single(self.xrecv[:n_recv], self.xsend[:n_send], recv, send, group=self.group, async_op=True)
        w2 = dist.all_to_all_single(self.selrecv[:n_recv], self.selsend[:n_send], recv, send, group=self.group, async_op=True)
        eng.ep_shared(layer, x, n)          # overlaps the exchange
        w1.wait()
        w2.wait()
        eng.ep_expert_forward(layer, self.xrecv, self.selrecv, n_recv, self.partial)
        dist.all_to_all_single(self.back[:n_send], self.partial[:n_recv], send, recv, group=self.group)
        eng.ep_combine(n, W, self.back, y)


class PeerExpertParallel:
    """The same layer with no all-to-all: every rank's receive buffers are mapped on every
    rank (CUDA IPC over NVLink), tokens' rows are stored straight into the owners' buffers by
    the push kernel and the partial rows are summed while they are read back from them
    (`qkm_ep_push` / `qkm_ep_forward_slots` / `qkm_ep_pull`).  Nothing comes to the host and
    no counts travel; the only synchronisation is two barriers per layer, which also order the
    reuse of the buffers by the next layer.  With `device_barrier=True` the barriers are the
    library's own kernel over the same peer mappings (`qkm_ep_barrier`, bounded wait) and a layer
    is ONE call into the library (`qkm_ep_peer_layer`); otherwise each is a one-word all-reduce
    of the process group on the compute stream.  The device barrier needs every rank on its own
    GPU and all ranks issuing the same sequence of calls.

    The engine must launch on the stream the process group's collectives synchronise with
    (torch's current stream): the constructor and every forward() point the engine at it.
    After a device barrier's bounded wait has run out, y is undefined from that layer on until
    the engine's sync() has reported the timeout; with `device_barrier=True` call `sync()` at the
    end of a step (see `end_step`)."""

    HANDLE_BYTES = 192

    def __init__(self, engine, max_local_tokens: int, device, group=None, device_barrier: bool = False,
                 timeout_ms: int = 2000):
        self.engine, self.group = engine, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.max_local, self.device = max_local_tokens, device
        self.device_barrier, self.timeout_ms = device_barrier, timeout_ms
        self._follow_current_stream()
        engine.ep_peer_setup(self.world, self.rank, max_local_tokens)
        mine = torch.frombuffer(bytearray(engine.ep_peer_export()), dtype=torch.uint8).to(device)
        if mine.numel() != self.HANDLE_BYTES:
            raise ValueError("engine exported handles of the wrong size")
        every = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(every, mine, group=group)
        for r, h in enumerate(every):
            if r != self.rank:
                engine.ep_peer_import(r, bytes(h.cpu().numpy().tobytes()))
        self._word = torch.zeros(1, dtype=torch.int32, device=device)
        self.barrier()

    def _follow_current_stream(self) -> None:
        """The one-word all-reduces that order the phases run on torch's current stream; the
        engine's kernels must run there too, or the barriers order nothing."""
        if hasattr(self.engine, "set_stream") and torch.cuda.is_available() and torch.device(self.device).type == "cuda":
            self.engine.set_stream(torch.cuda.current_stream(self.device).cuda_stream)

    def barrier(self) -> None:
        dist.all_reduce(self._word, group=self.group)

    def end_step(self) -> None:
        """End of a step with the library's own barriers: brings a barrier wait that ran out to
        the host (raises the engine's timeout error); outputs since that layer are invalid."""
        if self.device_barrier:
            self.engine.sync()

    def forward(self, layer: int, x: torch.Tensor, n: int, y: torch.Tensor, slot_rows: int | None = None) -> None:
        """y[:n] = MoE layer `layer` of the n local rows x[:n].  All ranks call this together
        with the same slot_rows (>= every rank's n; default: the size given at construction)."""
        rows = self.max_local if slot_rows is None else slot_rows
        if n > rows or rows > self.max_local:
            raise ValueError(f"{n} local tokens / {rows} slot rows exceed the {self.max_local} this object was sized for")
        eng = self.engine
        self._follow_current_stream()
        if self.device_barrier:
            eng.ep_peer_layer(layer, x, n, rows, y, self.timeout_ms)
            return
        eng.ep_push(layer, x, n, rows)
        self.barrier()                      # every rank's rows have landed
        eng.ep_forward_slots(layer, rows, n)   # the shared expert of the local rows rides along
        self.barrier()                      # every rank's partial rows are written
        eng.ep_pull(n, rows, y)
