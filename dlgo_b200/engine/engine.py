"""The engine: one model, one cache, one step function.

``step`` is the only way tokens reach the model.  It takes a batch of
sequences, each with its next tokens (a whole prompt, or one token, or anything
between), runs exactly those tokens as one packed batch against the cache, and
returns fp32 logits at the wanted places.  The reference has two functions for
its single sequence, ``Forward(token, pos)`` (models/llm/forward.go:123) and
``ForwardBatch(tokens, startPos)`` (models/llm/forward_batch.go:78); both are
this step with a batch of one.

Nothing is padded: sequences of unequal length are packed one after another, so
there is no padding that could change a result.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Dict, List, Optional, Sequence

import torch

from ..cache.book import CacheError
from ..cache.kv_cache import KVCache, PAGE_SIZE
from ..config.registry import load_config
from ..weights.loader import DictSource, WeightSource
from .graphs import decode_with_graph, greedy_with_graph, sampled_with_graph
from .model import CausalLM
from .runtime import Runtime, build_context


class StepError(ValueError):
    """A step the engine refuses (bad token id, unknown slot, sequence too long)."""


class Engine:
    def __init__(self, model_dir: Optional[str] = None, dtype="bfloat16", device="cuda:0",
                 max_tokens: Optional[int] = None, max_seq_len: Optional[int] = None, cuda_graphs: bool = True,
                 default_batch: int = 1, spec: Any = None, tensors: Optional[Dict[str, torch.Tensor]] = None,
                 max_slots: Optional[int] = None):
        """``max_tokens``: positions live sequences may hold in total (each sequence's count
        rounded up to a multiple of 64); it sizes the cache.  ``max_seq_len``: longest single
        sequence, clamped to the model's context like the reference's ``maxSeqLen``
        (models/llm/generate.go:56-58).  ``max_slots``: sequences that may be live at once (default:
        one per page of the cache, but no more than keep a group's page table within 64 MB).

        A model comes from ``model_dir`` (config.json chooses the architecture), or from an
        :class:`ArchitectureSpec` and its tensors given in memory (``spec``, ``tensors``)."""
        self.runtime = Runtime(device, dtype)
        if spec is None:
            if model_dir is None:
                raise ValueError("give a model folder, or a spec with its tensors")
            self.config = load_config(model_dir)
            self.spec = self.config.architecture_spec()
        else:
            self.config = None
            self.spec = spec
        self.model = CausalLM(self.spec)
        with torch.cuda.device(self.runtime.device):
            if tensors is not None:
                source = DictSource(tensors, self.runtime.device)
            else:
                source = WeightSource(model_dir, self.runtime.device)
            self.model.load_weights(source, self.runtime)
            source.release()
        self._note_stand_ins()
        context = self.spec.max_positions
        if max_seq_len is None or max_seq_len <= 0 or max_seq_len > context:
            max_seq_len = context
        needs, borrows, states = self.model.cache_needs()
        if max_tokens is None or max_tokens <= 0:
            # room for `default_batch` sequences of full length, within half of the free memory
            per_position = sum(2 * n.num_kv_heads * n.head_dim for n, b in zip(needs, borrows)
                               if n is not None and b is None) * (2 if self.runtime.dtype == torch.bfloat16 else 4)
            free, _ = torch.cuda.mem_get_info(self.runtime.device)
            fits = max(PAGE_SIZE, int(free * 0.5) // max(per_position, 1))
            max_tokens = max(min(max_seq_len * max(default_batch, 1), fits), min(max_seq_len, fits))
        n_pages = max(1, (max_tokens + PAGE_SIZE - 1) // PAGE_SIZE)
        if max_slots is None or max_slots <= 0:
            # a live sequence holds at least one page, so more slots than pages are never used; a slot's row
            # of the page table has one entry per page of the longest sequence
            row_bytes = 4 * ((min(max_seq_len, n_pages * PAGE_SIZE) + PAGE_SIZE - 1) // PAGE_SIZE)
            max_slots = min(n_pages, max(default_batch, 256, (64 << 20) // row_bytes))
        self.cache = KVCache(needs, borrows, states, max_tokens, max_seq_len, self.runtime.dtype, self.runtime.device,
                             PAGE_SIZE, n_slots=max_slots)
        self.max_seq_len = self.cache.max_seq_len
        self.vocab_size = self.spec.vocab_size
        self.cuda_graphs = cuda_graphs
        self._graphs: "OrderedDict[tuple, object]" = OrderedDict()    # (batch size, reach) -> captured step
        self._graph_pool = None
        self.launches_last_step = 0

    def _note_stand_ins(self) -> None:
        """One line on stderr when a bfloat16 model's sizes land on the slower stand-in kernels (never a wrong
        result, but a user should know why it is slow)."""
        if self.runtime.dtype != torch.bfloat16:
            return
        import sys
        notes = set()
        for blk in self.model.blocks:
            for part in blk.parts().values():
                for v in vars(part).values():
                    if hasattr(v, "_tc") and hasattr(v, "in_features") and v._tc is None:
                        notes.add(f"contractions over {v.in_features} inputs (no multiple of 8) run on the fp32 pipes")
                hd = getattr(part, "head_dim", None)
                if hd is not None and hasattr(part, "num_kv_heads") and hd not in (64, 128):
                    notes.add(f"attention with heads of {hd} runs on the general kernels (tensor-core kernels take 64 and 128)")
        if notes:
            print("[dlgo_b200] note: " + "; ".join(sorted(notes)), file=sys.stderr, flush=True)

    def graph_pool(self):
        """The memory pool that all captured steps of this engine share."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    # -------------------------------------------------------------------- slots
    def take_slot(self) -> int:
        return self.cache.take_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # --------------------------------------------------------------------- step
    def _validate(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
                  want: Optional[Sequence[Sequence[int]]]) -> None:
        if len(slots) != len(tokens):
            raise StepError(f"{len(slots)} slots for {len(tokens)} token lists")
        if len(set(slots)) != len(slots):
            raise StepError("a slot appears twice in one step")
        if want is not None and len(want) != len(tokens):
            raise StepError(f"{len(want)} want lists for {len(tokens)} sequences")
        V = self.vocab_size
        for i, (s, tk) in enumerate(zip(slots, tokens)):
            if len(tk) == 0:
                raise StepError(f"sequence {i} (slot {s}) brings no token")
            bad = [t for t in tk if not 0 <= int(t) < V]
            if bad:
                raise StepError(f"sequence {i} (slot {s}): token id {bad[0]} is outside the vocabulary [0, {V})")
            cur = self.cache.length(s)
            if cur + len(tk) > self.max_seq_len:
                raise StepError(
                    f"sequence {i} (slot {s}) would reach {cur + len(tk)} positions; the limit is {self.max_seq_len}")
            if want is not None:
                for w in want[i]:
                    if not 0 <= int(w) < len(tk):
                        raise StepError(f"sequence {i}: wanted place {w} is outside its {len(tk)} tokens")
        short = self.cache.pages_short(slots, [len(t) for t in tokens])
        if short is not None:
            raise StepError(short)      # refused before anything changes, like every other check

    @torch.no_grad()
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Run ``tokens[i]`` as the next tokens of the sequence in ``slots[i]``.

        ``want[i]`` lists the places among ``tokens[i]`` whose logits are asked for
        (default: the last).  Returns ``[wanted, vocab]`` fp32 on the device, in the
        order of the sequences and of ``want``; ``None`` if nothing is wanted.
        """
        slots = [int(s) for s in slots]
        if want is None and self.cuda_graphs and all(len(t) == 1 for t in tokens) and len(slots) == len(tokens):
            fast = self._decode_step(slots, tokens)
            if fast is not None:
                return fast
        self._validate(slots, tokens, want)
        ntok = [len(t) for t in tokens]
        starts = [self.cache.length(s) for s in slots]
        rows: List[int] = []
        off = 0
        for i, n in enumerate(ntok):
            rows.extend(off + int(w) for w in (want[i] if want is not None else [n - 1]))
            off += n
        with torch.cuda.device(self.runtime.device):
            self.cache.reserve(slots, ntok)
            decode = all(n == 1 for n in ntok)
            last_only = want is None or all(list(w) == [0] for w in want)
            if decode and self.cuda_graphs and last_only:
                logits = decode_with_graph(self, slots, [int(t[0]) for t in tokens], starts)
            else:
                ctx = build_context(self.runtime, tokens, slots, starts, self.max_seq_len)
                ctx.want_identity = rows == list(range(ctx.n_tokens))
                want_rows = (torch.tensor(rows, dtype=torch.int32).to(self.runtime.device, non_blocking=True)
                             if rows else None)
                logits = self.model.forward(ctx, self.cache, want_rows)
            self.cache.commit(slots, ntok)
        return logits

    def _decode_step(self, slots: List[int], tokens: Sequence[Sequence[int]]) -> Optional[torch.Tensor]:
        """One token per sequence, logits of each: the same checks and the same work as the general
        path with less host time (a decode step's GPU work is under a millisecond).  ``None`` hands
        an input that fails a check over to the general path, which names the fault."""
        V, limit = self.vocab_size, self.max_seq_len
        lengths = self.cache.book._len
        ids = []
        starts = []
        for s, tk in zip(slots, tokens):
            t = int(tk[0])
            cur = lengths.get(s)
            if cur is None or not 0 <= t < V or cur + 1 > limit:
                return None
            ids.append(t)
            starts.append(cur)
        if len(set(slots)) != len(slots):
            return None
        ones = [1] * len(slots)
        dev = self.runtime.device
        if torch.cuda.current_device() != (dev.index or 0):
            with torch.cuda.device(dev):
                self.cache.reserve(slots, ones)
                logits = decode_with_graph(self, slots, ids, starts)
        else:
            self.cache.reserve(slots, ones)
            logits = decode_with_graph(self, slots, ids, starts)
        for s in slots:
            lengths[s] += 1
        return logits

    @torch.no_grad()
    def sampled_run(self, slots: Sequence[int], tokens: Sequence[int], n_steps: int, stop_ids: Sequence[int],
                    sampler: Any, seed: int, requests: Sequence[int], draws: Sequence[int],
                    recents: Sequence[Sequence[int]]) -> Optional[List[List[int]]]:
        """:meth:`greedy_run` with a sampler configuration's filters and draw in the place of the argmax
        (``sampler`` is not greedy).  ``requests[i]`` and ``draws[i]`` key sequence i's uniform numbers, the
        draw index advancing by one per step; ``recents[i]`` are its latest tokens, oldest first."""
        return self.greedy_run(slots, tokens, n_steps, stop_ids, (sampler, seed, requests, draws, recents))

    def greedy_run(self, slots: Sequence[int], tokens: Sequence[int], n_steps: int,
                   stop_ids: Sequence[int] = (), _draw: Optional[tuple] = None) -> Optional[List[List[int]]]:
        """Run ``tokens[i]`` as the next token of the sequence in ``slots[i]`` and go on greedily, every
        sequence one token per step, for up to ``n_steps`` steps without returning in between (the steps,
        the argmax and the copies of the ids are one native call).  Returns the ids chosen, a list per
        step; the run ends with the step in which a sequence chose one of ``stop_ids``.  ``None`` when
        this engine cannot do it (no CUDA graphs, or the cache lacks room for ``n_steps`` positions):
        the caller then steps one by one."""
        if not self.cuda_graphs or n_steps <= 0:
            return None
        slots = [int(s) for s in slots]
        ids = [int(t) for t in tokens]
        V, limit = self.vocab_size, self.max_seq_len
        lengths = self.cache.book._len
        if len(slots) != len(ids) or len(set(slots)) != len(slots):
            raise StepError("greedy_run: one token per distinct slot")
        starts = []
        for s, t in zip(slots, ids):
            cur = lengths.get(s)
            if cur is None:
                raise StepError(f"slot {s} is not held")
            if not 0 <= t < V:
                raise StepError(f"token id {t} is outside the vocabulary [0, {V})")
            if cur + n_steps > limit:
                raise StepError(f"slot {s} would reach {cur + n_steps} positions; the limit is {limit}")
            starts.append(cur)
        with torch.cuda.device(self.runtime.device):
            try:
                self.cache.reserve(slots, [n_steps] * len(slots))     # pages for the whole run, mirrored once
            except CacheError:
                return None             # no room for the whole run; nothing was taken (all or nothing)
            if _draw is None:
                out = greedy_with_graph(self, slots, ids, starts, n_steps, stop_ids)
            else:
                out = sampled_with_graph(self, slots, ids, starts, n_steps, stop_ids, *_draw)
        self.cache.commit(slots, [len(out)] * len(slots))
        return out

    # ------------------------------------------------------------------ summary
    def weight_bytes(self) -> int:
        """Bytes of weights a decode step reads once (embedding table excluded unless it is the head)."""
        seen = set()
        total = 0

        def add(t: Optional[torch.Tensor]) -> None:
            nonlocal total
            if t is None or t.data_ptr() in seen:
                return
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()

        for blk in self.model.blocks:
            for part in blk.parts().values():
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor):
                        add(v)
                    elif hasattr(v, "weight") and isinstance(getattr(v, "weight"), torch.Tensor):
                        add(v.weight)
        add(getattr(self.model.final_norm, "weight", None))
        proj = getattr(self.model.head, "proj", None)
        add(getattr(proj, "weight", None))
        return total
