"""The generation loop: requests in, token ids out.

The reference generates for one sequence (models/llm/generate.go:84-153):
reject an empty or over-long prompt (:85-90), reset the cache (:97-100), run the
whole prompt (:110), sample (:113), then loop: stop at the context limit
(:122), stop if the last token is EOS or a stop token (:126-133), run that one
token, sample again, at most ``MaxTokens`` tokens.

Here the same loop runs over batches of requests.  A batch's prompts, of unequal
lengths, go through ONE step; then every sequence that is still going brings one
token per step.  A sequence that ends leaves the batch at once and its slot is
given back; the others go on.  When a batch is done the next one starts, in the
slots the last one freed, until no request is left.

The loop decides; it computes nothing.  It drives a *backend* with four calls
(``take_slot``, ``free_slot``, ``pages_free``/``pages_for`` for admission, and
``step_and_sample``), so its decisions can be tested against a scripted backend
without a GPU.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Protocol, Sequence, Tuple

from ..sampling.sampler import RECENT_WINDOW, SamplerConfig


@dataclass(frozen=True)
class GenerateConfig:
    """Defaults follow the reference's ``DefaultGenerateConfig`` (models/llm/generate.go:25-31)."""

    max_tokens: int = 256
    sampler: SamplerConfig = field(default_factory=SamplerConfig)
    seed: int = -1                       # < 0: seeded from the clock
    stop_token_ids: Tuple[int, ...] = ()  # in addition to the model's own
    ignore_eos: bool = False             # benchmarks: never stop on a token
    include_stop: bool = False           # keep the stop token in the output


@dataclass
class GenerateResult:
    """What the reference's ``GenerateResult`` reports (models/llm/generate.go:192-200), per call."""

    tokens: List[List[int]]
    prompt_tokens: int
    output_tokens: int
    prefill_ms: float
    generate_ms: float
    batches: int
    steps: int

    @property
    def tokens_per_sec(self) -> float:
        return self.output_tokens / (self.generate_ms / 1e3) if self.generate_ms > 0 else 0.0


class Backend(Protocol):
    max_seq_len: int

    def take_slot(self) -> int: ...
    def free_slot(self, slot: int) -> None: ...
    def pages_free(self) -> int: ...
    def slots_free(self) -> int: ...
    def pages_for(self, n_positions: int) -> int: ...
    def step_and_sample(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], requests: Sequence[int],
                        draws: Sequence[int], sampler: SamplerConfig, seed: int,
                        recent: Sequence[Sequence[int]]) -> List[int]: ...
    # optional: ``greedy_steps(slots, last_tokens, n_steps, stop_ids) -> per-step lists of ids | None``:
    # up to n_steps greedy decode steps of the same sequences in one call, ending with the step in
    # which a sequence chose a stop id


class GenerationError(ValueError):
    pass


@dataclass
class _Live:
    request: int
    slot: int
    length: int                 # positions held (prompt + tokens already run)
    out: List[int] = field(default_factory=list)
    recent: List[int] = field(default_factory=list)
    last: int = -1


class GenerationLoop:
    def __init__(self, backend: Backend, model_stop_ids: Sequence[int] = (), max_batch: int = 64):
        if max_batch <= 0:
            raise GenerationError("max_batch must be positive")
        self.backend = backend
        self.model_stop_ids = tuple(int(t) for t in model_stop_ids)
        self.max_batch = max_batch

    # ------------------------------------------------------------------ admission
    def plan_batches(self, prompt_lens: Sequence[int], max_tokens: int) -> List[List[int]]:
        """Requests in order, cut into batches that fit the slots and the pages.

        A request is admitted with room for its whole run (prompt + tokens it may still
        bring), so a batch never runs out of cache halfway.
        """
        batches: List[List[int]] = []
        cur: List[int] = []
        pages = 0
        total_pages = self.backend.pages_free()
        slots = self.backend.slots_free()
        limit = self.backend.max_seq_len
        for i, n in enumerate(prompt_lens):
            need = self.backend.pages_for(min(limit, n + max(max_tokens - 1, 0)))
            if need > total_pages:
                raise GenerationError(
                    f"request {i} needs {need} cache pages for {n} prompt tokens and up to {max_tokens} new ones; "
                    f"the cache has {total_pages}")
            if cur and (len(cur) >= min(self.max_batch, slots) or pages + need > total_pages):
                batches.append(cur)
                cur, pages = [], 0
            cur.append(i)
            pages += need
        if cur:
            batches.append(cur)
        return batches

    # ----------------------------------------------------------------------- run
    def run(self, prompts: Sequence[Sequence[int]], cfg: GenerateConfig,
            on_token: Optional[Callable[[int, int], None]] = None) -> GenerateResult:
        """Generate for every prompt; ``on_token(request index, token id)`` is called per emitted token."""
        if len(prompts) == 0:
            return GenerateResult([], 0, 0, 0.0, 0.0, 0, 0)
        limit = self.backend.max_seq_len
        for i, p in enumerate(prompts):
            if len(p) == 0:
                raise GenerationError(f"request {i}: empty prompt")
            if len(p) >= limit:
                raise GenerationError(f"request {i}: prompt too long: {len(p)} tokens (max {limit})")
        if cfg.max_tokens <= 0:
            raise GenerationError("max_tokens must be positive")
        seed = cfg.seed if cfg.seed >= 0 else time.time_ns() & 0x7FFFFFFFFFFFFFFF
        stops = set() if cfg.ignore_eos else set(self.model_stop_ids) | set(int(t) for t in cfg.stop_token_ids)
        outputs: List[List[int]] = [[] for _ in prompts]
        prefill_ms = generate_ms = 0.0
        steps = 0
        batches = self.plan_batches([len(p) for p in prompts], cfg.max_tokens)
        for batch in batches:
            live = [_Live(request=i, slot=self.backend.take_slot(), length=0) for i in batch]
            try:
                t0 = time.perf_counter()
                feed: List[Sequence[int]] = [prompts[s.request] for s in live]
                first = True
                def account(sampled: Sequence[int]) -> None:
                    """One step's chosen tokens: outputs, stop tokens, who goes on."""
                    nonlocal live, feed
                    still: List[_Live] = []
                    for s, fed, tok in zip(live, feed, sampled):
                        s.length += len(fed)
                        tok = int(tok)
                        stop = tok in stops
                        if not stop or cfg.include_stop:
                            s.out.append(tok)
                            s.recent.append(tok)
                            if len(s.recent) > RECENT_WINDOW:
                                del s.recent[0]
                            if on_token is not None:
                                on_token(s.request, tok)
                        # the next step would put `tok` at position s.length: it must fit, and
                        # the reference stops one short of the limit (generate.go:122)
                        done = stop or len(s.out) >= cfg.max_tokens or s.length >= limit - 1
                        if done:
                            outputs[s.request] = s.out
                            self.backend.free_slot(s.slot)
                            s.slot = -1
                        else:
                            s.last = tok
                            still.append(s)
                    live = still
                    feed = [[s.last] for s in live]

                greedy_steps = getattr(self.backend, "greedy_steps", None)
                sampled_steps = getattr(self.backend, "sampled_steps", None)
                many_steps = greedy_steps if cfg.sampler.greedy else sampled_steps
                while live:
                    if not first and many_steps is not None and on_token is None:
                        # Decoding with nobody listening token by token: the backend may run several
                        # steps in one call.  As many as every sequence can take before it ends by
                        # count, so that only a stop token can end one earlier, and the backend
                        # returns with the step in which one appeared.
                        n = min(min(cfg.max_tokens - len(s.out), limit - 1 - s.length) for s in live)
                        chunk = None
                        if n > 1 and cfg.sampler.greedy:
                            chunk = greedy_steps([s.slot for s in live], [s.last for s in live], n, sorted(stops))
                        elif n > 1:
                            chunk = sampled_steps([s.slot for s in live], [s.last for s in live], n, sorted(stops),
                                                  cfg.sampler, seed, [s.request for s in live],
                                                  [len(s.out) for s in live], [s.recent for s in live])
                        if chunk is not None:
                            head = chunk[:-1]
                            if len(head) > 1 and all(stops.isdisjoint(row) for row in head):
                                # Only the run's last step can end a sequence (by a stop token, or by count:
                                # n was chosen so).  The steps before it just append, a sequence at a time
                                # instead of a token at a time.
                                for s, col in zip(live, zip(*head)):
                                    s.length += len(col)
                                    s.out.extend(col)
                                    s.recent = (s.recent + list(col))[-RECENT_WINDOW:]
                                    s.last = int(col[-1])
                                steps += len(head)
                                feed = [[s.last] for s in live]
                                chunk = chunk[-1:]
                            for sampled in chunk:
                                steps += 1
                                account(sampled)
                            continue
                    sampled = self.backend.step_and_sample(
                        [s.slot for s in live], feed, [s.request for s in live], [len(s.out) for s in live],
                        cfg.sampler, seed, [s.recent for s in live])
                    steps += 1
                    if first:
                        prefill_ms += (time.perf_counter() - t0) * 1e3
                        t0 = time.perf_counter()
                        first = False
                    account(sampled)
                generate_ms += (time.perf_counter() - t0) * 1e3
            finally:
                for s in live:
                    if s.slot >= 0:
                        self.backend.free_slot(s.slot)
        return GenerateResult(
            tokens=outputs, prompt_tokens=sum(len(p) for p in prompts),
            output_tokens=sum(len(o) for o in outputs), prefill_ms=prefill_ms, generate_ms=generate_ms,
            batches=len(batches), steps=steps)
