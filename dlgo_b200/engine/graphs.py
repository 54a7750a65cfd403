"""CUDA graphs for decode steps.

A decode step is a hundred-odd small launches; at one token per sequence the
GPU work of each is a few microseconds, so the launches themselves bound the
step.  One graph per batch size and reach replays the whole step from persistent
input buffers (token ids, positions, slots).  Nothing inside the graph may depend
on the sequences' lengths through the host: grids are sized for the graph's reach
(the longest sequence it is asked to serve: 4,096 positions, 16,384, ... up to the
cache's capacity) and every kernel reads lengths and pages from device memory.
"""
from __future__ import annotations

from typing import Any, List, Optional, Sequence

import torch

from ..csrc import kernels
from .runtime import StepContext


# Captured steps kept per engine, one per batch size and reach (a batch that drains one sequence at a time asks
# for every size once); each holds its fp32 logits [batch, vocab], so their number is bounded and the least recently used
# goes first.  Intermediates of all captures share one memory pool: they never run at the same time.
MAX_GRAPHS = 24
FIRST_REACH = 4096


def reach_bucket(reach: int, max_seq_len: int) -> int:
    """The reach a captured step is sized for when its longest sequence ends at ``reach`` positions: 4,096,
    16,384, 65,536, ... but no more than the cache holds per sequence.  A context limit of 131,072 would
    otherwise size every step for 2,048 pages a sequence, and a sequence of a few hundred tokens would be
    cut into dozens of mostly empty slices that meet again through scratch memory and a second kernel."""
    b = FIRST_REACH
    while b < reach and b < max_seq_len:
        b *= 4
    return min(b, max_seq_len)


class NotOnHost:
    """Stands where a captured step has no host-side value (slots, start positions): a replay serves
    whatever sequences the step brings, so a part must read ``ctx.seq_slot`` and ``ctx.token_pos`` on
    the device instead.  Any use of it says so."""

    def __init__(self, what: str):
        self._what = what

    def _refuse(self, *a: Any, **k: Any):
        raise RuntimeError(f"{self._what} is not known on the host inside a captured decode step: read the "
                           "device tensors ctx.seq_slot / ctx.token_pos (or build the engine with cuda_graphs=False)")

    __iter__ = __len__ = __getitem__ = __bool__ = __index__ = _refuse


class DecodeGraph:
    def __init__(self, engine: Any, batch: int, reach: int):
        rt = engine.runtime
        dev = rt.device
        self.batch = batch
        self.reach = reach
        self.meta = torch.zeros((3, batch), dtype=torch.int32, device=dev)   # ids, positions, slots
        self.host = torch.zeros((3, batch), dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()     # a view: the step's inputs are written here without tensor construction
        self.token_seq = torch.arange(batch, dtype=torch.int32, device=dev)
        self.want_rows = torch.arange(batch, dtype=torch.int32, device=dev)
        self.ctx = StepContext(
            runtime=rt, n_tokens=batch, n_seqs=batch, token_ids=self.meta[0], token_pos=self.meta[1],
            token_seq=self.token_seq, seq_slot=self.meta[2], seq_slots_host=NotOnHost("a sequence's slot"),
            seq_start_host=NotOnHost("a sequence's start position"),
            seq_ntok_host=[1] * batch, decode=True, max_len=reach, captured=True,
            capacity=reach, want_identity=True)
        # one token per sequence: the tile table is the same for every replay (built before capture: a
        # capture may not copy from pageable host memory)
        self.ctx._tiles[(1, False)] = (torch.stack([self.token_seq, self.token_seq, torch.ones_like(self.token_seq)],
                                                   dim=1).contiguous(), batch, 1)
        self.graph = torch.cuda.CUDAGraph()
        self.logits = None
        self.engine = engine
        self._dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
        # copy of the inputs, "buffer free" event and graph launch as one native call (csrc/hoststep.cu)
        self._native = kernels.HostStep()
        self._exec = None
        # a second capture of the same step that begins with the copy of its inputs out of the pinned buffer
        # and ends with the argmax and the copy of the ids into pinned memory, for greedy runs (made when
        # first asked for)
        self.greedy_graph = None
        self.greedy_exec = None
        self.greedy_kernels = 0
        self.ids_dev = torch.zeros((batch,), dtype=torch.int32, device=dev)
        self.ids_host = torch.zeros((batch,), dtype=torch.int32).pin_memory()
        # captures per sampler configuration that end with the filters and the draw, for sampled runs; the
        # draw's inputs (seed, request and draw indices, recent tokens, token counts) come out of one pinned
        # buffer, so that one capture serves every seed and every set of requests
        self.sampled = {}
        self.draw_host = None
        self.draw_dev = None

    def capture(self) -> None:
        eng = self.engine
        # Warm-up runs on a side stream (lazy initialisations must not land in the capture).  It runs the
        # step for real: keys and values land where the step itself writes them again, but fixed-size
        # state would be advanced twice, so the batch's state is put back afterwards.
        slots = [int(v) for v in self.host_np[2]]
        saved = eng.cache.state.snapshot(slots) if eng.cache.state.tensors else None
        s = torch.cuda.Stream(device=eng.runtime.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            eng.model.forward(self.ctx, eng.cache, self.want_rows)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        if saved is not None:
            eng.cache.state.restore(slots, saved)
        before = kernels.LAUNCHES
        with torch.cuda.graph(self.graph, pool=eng.graph_pool()):
            self.logits = eng.model.forward(self.ctx, eng.cache, self.want_rows)
        self.kernels_per_replay = kernels.LAUNCHES - before
        self._exec = self.graph.raw_cuda_graph_exec()

    def capture_greedy(self) -> None:
        eng = self.engine
        torch.cuda.synchronize()
        before = kernels.LAUNCHES
        self.greedy_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.greedy_graph, pool=eng.graph_pool()):
            self.meta.copy_(self.host, non_blocking=True)      # the step's inputs out of the pinned buffer
            logits = eng.model.forward(self.ctx, eng.cache, self.want_rows)
            kernels.argmax(logits, self.ids_dev)
            self.ids_host.copy_(self.ids_dev, non_blocking=True)
        self.greedy_kernels = kernels.LAUNCHES - before
        self.greedy_exec = self.greedy_graph.raw_cuda_graph_exec()

    def capture_sampled(self, cfg: Any) -> tuple:
        """(graph exec, kernels per replay) of the step followed by ``cfg``'s filters and draw."""
        from ..sampling.sampler import RECENT_WINDOW, draw_on_device, temperature_rows
        hit = self.sampled.get(cfg)
        if hit is not None:
            return hit[1], hit[2]
        if len(self.sampled) >= 4:
            self.sampled.pop(next(iter(self.sampled)))      # (a handful of configurations at a time)
        eng, b, w = self.engine, self.batch, RECENT_WINDOW
        dev = eng.runtime.device
        if self.draw_host is None:
            self.draw_host = torch.zeros((2 + 3 * b + b * w,), dtype=torch.int32).pin_memory()
            self.draw_host[2 + 2 * b:2 + 2 * b + b * w] = -1
            self.draw_dev = torch.zeros((2 + 2 * b + b * w,), dtype=torch.int32, device=dev)
        d = self.draw_dev
        requests, draws, recent = d[2:2 + b], d[2 + b:2 + 2 * b], d[2 + 2 * b:].view(b, w)
        temperature = temperature_rows(cfg, b, dev)
        torch.cuda.synchronize()
        before = kernels.LAUNCHES
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=eng.graph_pool()):
            self.meta.copy_(self.host, non_blocking=True)
            d.copy_(self.draw_host[:d.numel()], non_blocking=True)
            logits = eng.model.forward(self.ctx, eng.cache, self.want_rows)
            draw_on_device(logits, cfg, requests, draws, recent, 0, seed_dev=d[0:2], out=self.ids_dev,
                           temperature=temperature)
            self.ids_host.copy_(self.ids_dev, non_blocking=True)
        n = kernels.LAUNCHES - before
        self.sampled[cfg] = (graph, graph.raw_cuda_graph_exec(), n, temperature)
        return self.sampled[cfg][1], n

    def run(self, slots: Sequence[int], token_ids: Sequence[int], starts: Sequence[int]) -> torch.Tensor:
        self._native.wait()      # the previous step's copy out of the pinned buffer has finished
        h = self.host_np
        h[0, :] = token_ids
        h[1, :] = starts
        h[2, :] = slots
        self._native.launch(self.meta, self.host, self._exec, self._dev_index)
        kernels.LAUNCHES += self.kernels_per_replay
        return self.logits


def greedy_with_graph(engine: Any, slots: List[int], token_ids: List[int], starts: List[int], n_steps: int,
                      stop_ids: Sequence[int]) -> List[List[int]]:
    """Up to ``n_steps`` greedy decode steps through the graph of this batch size in one native call;
    the ids chosen, a list per step (fewer than ``n_steps`` if a sequence chose a stop id)."""
    b = len(slots)
    g = graph_for(engine, slots, token_ids, starts, max(starts) + n_steps)
    if g.greedy_exec is None:
        g.capture_greedy()
    g._native.wait()
    h = g.host_np
    h[0, :] = token_ids
    h[1, :] = starts
    h[2, :] = slots
    return kernels.greedy_run_graph(g.host, g.greedy_exec, g.ids_host, stop_ids, n_steps, g._dev_index,
                                    g.greedy_kernels)


def sampled_with_graph(engine: Any, slots: List[int], token_ids: List[int], starts: List[int], n_steps: int,
                       stop_ids: Sequence[int], cfg: Any, seed: int, requests: Sequence[int], draws: Sequence[int],
                       recents: Sequence[Sequence[int]]) -> List[List[int]]:
    """:func:`greedy_with_graph` with ``cfg``'s filters and draw instead of the argmax: ``requests[i]`` and
    ``draws[i]`` key the uniform numbers of sequence i (the draw index advances with every step), and
    ``recents[i]`` are its latest tokens, oldest first, for the repetition penalty."""
    from ..sampling.sampler import RECENT_WINDOW
    b, w = len(slots), RECENT_WINDOW
    g = graph_for(engine, slots, token_ids, starts, max(starts) + n_steps)
    graph_exec, n_kernels = g.capture_sampled(cfg)
    g._native.wait()
    h = g.host_np
    h[0, :] = token_ids
    h[1, :] = starts
    h[2, :] = slots
    dh = g.draw_host.numpy()
    seed &= (1 << 64) - 1
    dh[0:2] = [((seed & 0xFFFFFFFF) ^ 0x80000000) - 0x80000000, ((seed >> 32) ^ 0x80000000) - 0x80000000]
    dh[2:2 + b] = list(requests)
    dh[2 + b:2 + 2 * b] = list(draws)
    rec = dh[2 + 2 * b:2 + 2 * b + b * w].reshape(b, w)
    cnt = dh[2 + 2 * b + b * w:]
    for i, r in enumerate(recents):
        r = list(r)[-w:]
        rec[i, :len(r)] = r
        rec[i, len(r):] = -1
        cnt[i] = len(r)                 # the oldest lies first: a full window wraps to it
    return kernels.sampled_run_graph(g.host, graph_exec, g.ids_host, stop_ids, n_steps, g.draw_host, w,
                                     g._dev_index, n_kernels)


def graph_for(engine: Any, slots: List[int], token_ids: List[int], starts: List[int],
              reach: Optional[int] = None) -> DecodeGraph:
    """The captured step of this batch size whose grids cover sequences of up to ``reach`` positions (default:
    the longest sequence after one step), made when first asked for."""
    b = len(slots)
    key = (b, reach_bucket(max(starts) + 1 if reach is None else reach, engine.max_seq_len))
    g = engine._graphs.get(key)
    if g is not None:
        engine._graphs.move_to_end(key)
    if g is None:
        while len(engine._graphs) >= MAX_GRAPHS:
            engine._graphs.popitem(last=False)      # the one that was used longest ago
        g = DecodeGraph(engine, b, key[1])
        # the warm-up before the capture runs the step for real, on whatever the buffers hold: give it
        # this step's inputs so that it writes where this step writes anyway
        g.host_np[0, :] = token_ids
        g.host_np[1, :] = starts
        g.host_np[2, :] = slots
        g.meta.copy_(g.host)
        g.capture()
        engine._graphs[key] = g
    return g


def decode_with_graph(engine: Any, slots: List[int], token_ids: List[int], starts: List[int],
                      reach: Optional[int] = None) -> torch.Tensor:
    """Logits [batch, vocab] of one decode step, through the graph of this batch size (and ``reach``, see
    :func:`graph_for`).

    The returned tensor is the graph's output buffer: it is overwritten by the next
    decode step of the same batch size.
    """
    return graph_for(engine, slots, token_ids, starts, reach).run(slots, token_ids, starts)
