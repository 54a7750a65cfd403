"""The generation loop's decisions, against a scripted backend (no GPU)."""
from typing import Dict, List

import pytest

from dlgo_b200.engine.generate import GenerateConfig, GenerationError, GenerationLoop
from dlgo_b200.sampling.sampler import SamplerConfig


class ScriptedBackend:
    """Sequences "generate" a function of their request index and draw count; slots and pages are counted."""

    def __init__(self, n_slots=4, n_pages=16, page_size=64, max_seq_len=256, script=None):
        self.max_seq_len = max_seq_len
        self.page_size = page_size
        self.n_pages = n_pages
        self.free_slots = list(range(n_slots))
        self.held: Dict[int, int] = {}          # slot -> positions held
        self.calls: List[dict] = []
        self.script = script or (lambda request, draw: 100 + 10 * request + draw)
        self.freed: List[int] = []

    def take_slot(self):
        s = self.free_slots.pop(0)
        self.held[s] = 0
        return s

    def free_slot(self, slot):
        assert slot in self.held, "slot freed twice or never taken"
        del self.held[slot]
        self.free_slots.append(slot)
        self.freed.append(slot)

    def pages_free(self):
        return self.n_pages - sum(self.pages_for(n) for n in self.held.values())

    def slots_free(self):
        return len(self.free_slots)

    def pages_for(self, n):
        return (n + self.page_size - 1) // self.page_size

    def step_and_sample(self, slots, tokens, requests, draws, sampler, seed, recent):
        self.calls.append(dict(slots=list(slots), tokens=[list(t) for t in tokens], requests=list(requests),
                               draws=list(draws), recent=[list(r) for r in recent], seed=seed))
        for s, t in zip(slots, tokens):
            self.held[s] += len(t)
            assert self.held[s] <= self.max_seq_len
        return [self.script(r, d) for r, d in zip(requests, draws)]


GREEDY = SamplerConfig.greedy_config()


def test_prompts_go_in_one_step_then_one_token_each():
    be = ScriptedBackend()
    res = GenerationLoop(be).run([[1, 2, 3], [4], [5, 6]], GenerateConfig(max_tokens=3, sampler=GREEDY, seed=5))
    assert res.tokens == [[100, 101, 102], [110, 111, 112], [120, 121, 122]]
    assert be.calls[0]["tokens"] == [[1, 2, 3], [4], [5, 6]]
    assert be.calls[1]["tokens"] == [[100], [110], [120]] and be.calls[1]["draws"] == [1, 1, 1]
    assert len(be.calls) == 3 and res.steps == 3 and res.batches == 1
    assert res.prompt_tokens == 6 and res.output_tokens == 9
    assert be.held == {} and sorted(be.free_slots) == [0, 1, 2, 3]
    assert all(c["seed"] == 5 for c in be.calls)


def test_stop_token_ends_one_sequence_early_and_is_left_out():
    script = lambda r, d: 7 if (r == 1 and d == 1) else 100 + 10 * r + d
    be = ScriptedBackend(script=script)
    loop = GenerationLoop(be, model_stop_ids=[7])
    res = loop.run([[1], [2], [3]], GenerateConfig(max_tokens=4, sampler=GREEDY, seed=0))
    assert res.tokens[1] == [110]                       # stopped at its second draw, stop token not returned
    assert res.tokens[0] == [100, 101, 102, 103] and res.tokens[2] == [120, 121, 122, 123]
    assert be.calls[2]["requests"] == [0, 2]            # the batch shrank; the others went on
    assert be.freed[0] == be.calls[0]["slots"][1]       # its slot came back first
    res2 = loop.run([[1], [2], [3]], GenerateConfig(max_tokens=4, sampler=GREEDY, seed=0, include_stop=True))
    assert res2.tokens[1] == [110, 7]
    res3 = loop.run([[1], [2]], GenerateConfig(max_tokens=3, sampler=GREEDY, seed=0, ignore_eos=True))
    assert res3.tokens[1] == [110, 7, 112]


def test_extra_stop_tokens_and_a_stop_on_the_first_token():
    be = ScriptedBackend(script=lambda r, d: 9)
    res = GenerationLoop(be).run([[1, 2]], GenerateConfig(max_tokens=5, sampler=GREEDY, seed=0, stop_token_ids=(9,)))
    assert res.tokens == [[]] and len(be.calls) == 1 and be.held == {}


def test_batches_one_after_another_reuse_slots():
    be = ScriptedBackend(n_slots=2)
    res = GenerationLoop(be, max_batch=8).run([[i + 1] for i in range(5)], GenerateConfig(max_tokens=2, sampler=GREEDY, seed=0))
    assert res.batches == 3 and [len(t) for t in res.tokens] == [2] * 5
    assert res.tokens[4] == [140, 141]
    firsts = [c for c in be.calls if c["draws"][0] == 0]
    assert [c["requests"] for c in firsts] == [[0, 1], [2, 3], [4]]
    assert set(firsts[1]["slots"]) == set(firsts[0]["slots"])      # the same slots, used again
    assert be.held == {}


def test_admission_by_pages_and_a_request_too_large():
    be = ScriptedBackend(n_slots=8, n_pages=4, page_size=64, max_seq_len=256)
    loop = GenerationLoop(be)
    # each request may reach 100 + 29 = 129 positions -> 3 pages; only one fits at a time
    assert loop.plan_batches([100, 100, 100], 30) == [[0], [1], [2]]
    assert loop.plan_batches([10, 10, 10, 10, 10], 30) == [[0, 1, 2, 3], [4]]
    be2 = ScriptedBackend(n_slots=8, n_pages=2, max_seq_len=256)
    with pytest.raises(GenerationError, match="cache pages"):
        GenerationLoop(be2).plan_batches([200], 30)


def test_limits_and_errors():
    be = ScriptedBackend(max_seq_len=8)
    loop = GenerationLoop(be)
    with pytest.raises(GenerationError, match="empty prompt"):
        loop.run([[]], GenerateConfig(sampler=GREEDY))
    with pytest.raises(GenerationError, match="too long"):
        loop.run([[1] * 8], GenerateConfig(sampler=GREEDY))
    with pytest.raises(GenerationError, match="max_tokens"):
        loop.run([[1]], GenerateConfig(max_tokens=0, sampler=GREEDY))
    # prompt of 5 in a context of 8: tokens land at positions 5 and 6, then the loop stops one short
    # of the limit as the reference does (models/llm/generate.go:122)
    res = loop.run([[1] * 5], GenerateConfig(max_tokens=100, sampler=GREEDY, seed=0))
    assert len(res.tokens[0]) == 3 and be.held == {}
    assert loop.run([], GenerateConfig(sampler=GREEDY)).tokens == []


def test_recent_tokens_window_and_stream_callback():
    be = ScriptedBackend(max_seq_len=512, n_pages=64)
    seen = []
    res = GenerationLoop(be).run([[1], [2]], GenerateConfig(max_tokens=70, sampler=GREEDY, seed=0),
                                 on_token=lambda r, t: seen.append((r, t)))
    assert len(seen) == 140 and seen[0] == (0, 100) and seen[1] == (1, 110)
    assert [t for r, t in seen if r == 1] == res.tokens[1]
    last = be.calls[-1]["recent"][0]
    assert len(last) == 64 and last == res.tokens[0][-65:-1]       # sliding window of 64 (generate.go:143)


def test_slots_come_back_when_the_backend_fails():
    class Boom(ScriptedBackend):
        def step_and_sample(self, *a, **k):
            if len(self.calls) == 2:
                raise RuntimeError("boom")
            return super().step_and_sample(*a, **k)
    be = Boom()
    with pytest.raises(RuntimeError):
        GenerationLoop(be).run([[1], [2]], GenerateConfig(max_tokens=10, sampler=GREEDY, seed=0))
    assert be.held == {}


def test_seed_from_the_clock_when_negative():
    be = ScriptedBackend()
    GenerationLoop(be).run([[1]], GenerateConfig(max_tokens=1, sampler=GREEDY, seed=-1))
    assert be.calls[0]["seed"] >= 0


class MultiStepBackend(ScriptedBackend):
    """A backend that also offers several greedy steps in one call; it has to be told which request
    sits in which slot, so it remembers the requests of the prompt step."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.request_of: Dict[int, int] = {}
        self.draw_of: Dict[int, int] = {}
        self.multi_calls: List[dict] = []

    def step_and_sample(self, slots, tokens, requests, draws, sampler, seed, recent):
        for s, r, d in zip(slots, requests, draws):
            self.request_of[s] = r
            self.draw_of[s] = d + 1
        return super().step_and_sample(slots, tokens, requests, draws, sampler, seed, recent)

    def greedy_steps(self, slots, tokens, n_steps, stop_ids):
        self.multi_calls.append(dict(slots=list(slots), tokens=list(tokens), n=n_steps, stops=list(stop_ids)))
        out = []
        for _ in range(n_steps):
            ids = []
            for s in slots:
                self.held[s] += 1
                assert self.held[s] <= self.max_seq_len
                ids.append(self.script(self.request_of[s], self.draw_of[s]))
                self.draw_of[s] += 1
            out.append(ids)
            if any(i in stop_ids for i in ids):
                break
        return out


class MultiSampledBackend(MultiStepBackend):
    """... and several sampled steps in one call: it checks what the loop tells it about each sequence."""

    def sampled_steps(self, slots, tokens, n_steps, stop_ids, sampler, seed, requests, draws, recent):
        assert not sampler.greedy and seed >= 0
        for s, r, d, rec in zip(slots, requests, draws, recent):
            assert self.request_of[s] == r and self.draw_of[s] == d, "request and draw index of every sequence"
            assert len(rec) <= 64 and (d == 0 or len(rec) > 0)
        self.sampled_calls = getattr(self, "sampled_calls", 0) + 1
        return self.greedy_steps(slots, tokens, n_steps, stop_ids)


def test_several_sampled_steps_in_one_backend_call_change_no_decision():
    script = lambda r, d: 7 if (r == 1 and d == 2) else 100 + 10 * r + d
    prompts = [[1, 2], [3], [4, 5, 6]]
    sampler = SamplerConfig(temperature=0.7, top_k=40, top_p=0.9, min_p=0.0, repetition_penalty=1.1)
    for kw in (dict(), dict(include_stop=True), dict(ignore_eos=True)):
        cfg = GenerateConfig(max_tokens=6, sampler=sampler, seed=3, **kw)
        plain = GenerationLoop(ScriptedBackend(script=script), model_stop_ids=[7]).run(prompts, cfg)
        be = MultiSampledBackend(script=script)
        multi = GenerationLoop(be, model_stop_ids=[7]).run(prompts, cfg)
        assert multi.tokens == plain.tokens and multi.steps == plain.steps
        assert be.held == {} and be.sampled_calls >= 1 and len(be.calls) == 1
        # somebody listening token by token: one step per call
        be2 = MultiSampledBackend(script=script)
        seen = []
        GenerationLoop(be2, model_stop_ids=[7]).run(prompts, cfg, lambda r, t: seen.append((r, t)))
        assert not hasattr(be2, "sampled_calls") and len(be2.calls) > 1


def test_several_greedy_steps_in_one_backend_call_change_no_decision():
    script = lambda r, d: 7 if (r == 1 and d == 2) else 100 + 10 * r + d
    prompts = [[1, 2], [3], [4, 5, 6]]
    for kw in (dict(), dict(include_stop=True), dict(ignore_eos=True)):
        cfg = GenerateConfig(max_tokens=6, sampler=GREEDY, seed=0, **kw)
        plain = GenerationLoop(ScriptedBackend(script=script), model_stop_ids=[7]).run(prompts, cfg)
        be = MultiStepBackend(script=script)
        multi = GenerationLoop(be, model_stop_ids=[7]).run(prompts, cfg)
        assert multi.tokens == plain.tokens and multi.steps == plain.steps and multi.output_tokens == plain.output_tokens
        assert be.held == {} and sorted(be.free_slots) == [0, 1, 2, 3]
        assert len(be.calls) == 1 and be.multi_calls            # the prompts one step, the rest in runs
        if not kw:
            # the run asked for 5 more steps came back after 2 (request 1 chose the stop token); the
            # two others went on in a second run of 3
            assert [c["n"] for c in be.multi_calls] == [5, 3] and be.multi_calls[1]["slots"] == [0, 2]
    # with a listener, or when sampling, the loop steps one by one
    be = MultiStepBackend(script=script)
    seen = []
    GenerationLoop(be).run(prompts, GenerateConfig(max_tokens=3, sampler=GREEDY, seed=0), lambda r, t: seen.append((r, t)))
    assert not be.multi_calls and len(seen) == 9
    be = MultiStepBackend(script=script)
    GenerationLoop(be).run(prompts, GenerateConfig(max_tokens=3, sampler=SamplerConfig.plain_temperature(0.8), seed=0))
    assert not be.multi_calls
    # the sequence limit bounds a run like max_tokens does
    be = MultiStepBackend(max_seq_len=8, script=script)
    res = GenerationLoop(be).run([[1, 2, 3]], GenerateConfig(max_tokens=50, sampler=GREEDY, seed=0))
    assert len(res.tokens[0]) == 5 and be.multi_calls[0]["n"] == 4


def test_captured_steps_are_sized_for_a_reach_not_for_the_whole_context():
    from dlgo_b200.engine.graphs import reach_bucket
    assert reach_bucket(1, 131072) == 4096 and reach_bucket(4096, 131072) == 4096
    assert reach_bucket(4097, 131072) == 16384 and reach_bucket(70000, 131072) == 131072
    assert reach_bucket(131072, 131072) == 131072
    # a cache that holds less than the first reach: one size, the cache's
    assert reach_bucket(10, 1024) == 1024 and reach_bucket(1024, 1024) == 1024
    assert reach_bucket(5000, 6000) == 6000
