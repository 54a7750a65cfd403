"""The engine against the plain implementation, in 32-bit and in bfloat16, under every way of
cutting the work: whole requests, last tokens one by one, unequal batches with slot reuse, long
decoding, first tokens, and generation through the entry point.  Needs a GPU."""
import os

import pytest
import torch

import plain_llama as P
import traces as T
from tiny_configs import TINY, assert_close, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
# request lengths: page edges (64, 65, 128, 129), a single token, lengths across original_max_position (64)
LENGTHS = {"A": [5, 17, 32, 64, 100], "B": [1, 9, 70, 130, 200], "C": [3, 65, 129, 300, 64], "Bsharp": [2, 40, 128, 250]}
_engines = {}


def vocab_of(name):
    return TINY[name.replace("sharp", "")]["cfg"]["vocab_size"]


def requests_of(name):
    return {f"{name}{i}": random_tokens(n, vocab_of(name), 100 + i) for i, n in enumerate(LENGTHS[name])}


def engine_for(model_dirs, name, dtype, graphs=True, max_tokens=1536):
    from dlgo_b200.engine.engine import Engine
    key = (name, dtype, graphs, max_tokens)
    if key not in _engines:
        e = Engine(model_dirs[name], dtype=dtype, max_tokens=max_tokens, cuda_graphs=graphs)
        e.cache.poison()      # whatever was never written, or was given back, reads as NaN
        _engines[key] = e
    return _engines[key]


def check(name, model_dirs, dtype, steps, outs, reqs, what):
    got = T.collect(steps, outs, reqs)
    for rid, toks in reqs.items():
        assert_close(got[rid], plain_logits(model_dirs[name], toks), dtype, f"{what} {rid} ({len(toks)} tokens, {dtype})")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "Bsharp"])
def test_each_request_alone_and_whole(model_dirs, name, dtype):
    eng = engine_for(model_dirs, name, dtype)
    reqs = requests_of(name)
    steps = T.whole(reqs)
    check(name, model_dirs, dtype, steps, T.run_in_process(eng, steps), reqs, "whole")
    eng.cache.book.check()
    assert eng.cache.book.live_slots() == []


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "Bsharp"])
def test_last_32_tokens_one_by_one(model_dirs, name, dtype, graphs):
    eng = engine_for(model_dirs, name, dtype, graphs)
    reqs = requests_of(name)
    steps = T.tail_one_by_one(reqs, 32)
    check(name, model_dirs, dtype, steps, T.run_in_process(eng, steps), reqs, "tail")
    assert eng.cache.book.live_slots() == []


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "Bsharp"])
def test_unequal_batches_one_after_another(model_dirs, name, dtype, graphs):
    # a cache just large enough for one batch at a time: the second batch runs in the first one's pages
    reqs = requests_of(name)
    lens = sorted((len(t) for t in reqs.values()), reverse=True)
    need = sum((n + 63) // 64 * 64 for n in lens[:3])
    eng = engine_for(model_dirs, name, dtype, graphs, max_tokens=max(need, 64 * ((max(lens) + 63) // 64)) + 64)
    for rep, decode in enumerate([(32, 5, 17, 1, 40), (3, 33, 0, 12, 7)]):
        steps = T.batched(reqs, 3, decode)
        check(name, model_dirs, dtype, steps, T.run_in_process(eng, steps), reqs, f"batched#{rep}")
        eng.cache.book.check()
        assert eng.cache.book.live_slots() == []


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_composition_changes_nothing_in_float32_beyond_rounding(model_dirs, dtype):
    # the same request alone and inside two different batches
    eng = engine_for(model_dirs, "B", dtype)
    reqs = requests_of("B")
    alone = T.collect(T.whole(reqs), T.run_in_process(eng, T.whole(reqs)), reqs)
    st = T.batched(reqs, 5, (1, 1, 1, 1, 1))
    together = T.collect(st, T.run_in_process(eng, st), reqs)
    tol = 2e-6 if dtype == "float32" else 2e-2
    for rid in reqs:
        scale = float(alone[rid].abs().max())
        assert float((alone[rid] - together[rid]).abs().max()) <= tol * scale, rid


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model_dirs, dtype):
    # 4 prompt tokens, then 500 tokens one by one, across seven page edges, through the graph
    eng = engine_for(model_dirs, "C", dtype)
    reqs = {"long": random_tokens(504, vocab_of("C"), 9)}
    steps = T.tail_one_by_one(reqs, 500)
    check("C", model_dirs, dtype, steps, T.run_in_process(eng, steps), reqs, "long decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C"])
def test_requests_fed_in_pieces_of_several_tokens(model_dirs, name, dtype):
    # several tokens at a time on top of a cache that is not empty, unequal pieces side by side
    eng = engine_for(model_dirs, name, dtype)
    reqs = requests_of(name)
    steps = T.chunked(reqs, (37, 1, 64, 5, 70))
    check(name, model_dirs, dtype, steps, T.run_in_process(eng, steps), reqs, "pieces")


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_behind_a_prompt_of_more_than_64_pages(tmp_path_factory, dtype):
    # 4,090 prompt tokens, then fourteen tokens one by one across position 4,096 (the end of page 64): the
    # captured step sized for 4,096 positions hands over to the one sized for the whole cache, whose decode
    # attention cuts a sequence into more slices than a cluster holds and combines them through scratch memory
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.engine.engine import Engine
    from dlgo_b200.weights import write_random_model
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=128, num_hidden_layers=1, intermediate_size=192,
               num_attention_heads=2, num_key_value_heads=1, head_dim=64, vocab_size=300, rope_theta=500000.0,
               rms_norm_eps=1e-5, max_position_embeddings=8192, tie_word_embeddings=True)
    d = _long_dir.get("d")
    if d is None:
        d = _long_dir["d"] = str(tmp_path_factory.mktemp("long_context"))
        write_random_model(config_from_dict(cfg), 12, d)
    n_prompt, n_more = 4090, 14
    toks = random_tokens(n_prompt + n_more, 300, 21)
    eng = Engine(d, dtype=dtype, max_tokens=4608, max_seq_len=8192)
    eng.cache.poison()
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:n_prompt], "want": [0, 2047, n_prompt - 1]}], "end": []}]
    for j in range(n_prompt, n_prompt + n_more):
        steps.append({"step": len(steps), "entries": [{"id": "x", "tokens": [toks[j]], "want": [0]}],
                      "end": ["x"] if j == n_prompt + n_more - 1 else []})
    outs = T.run_in_process(eng, steps)
    assert list(eng._graphs) == [(1, 4096), (1, eng.max_seq_len)] and eng.max_seq_len == 4608
    ref = plain_logits(d, toks)
    got = torch.cat([outs[i] for i in range(1 + n_more)])
    assert_close(got, ref[[0, 2047, n_prompt - 1] + list(range(n_prompt, n_prompt + n_more))], dtype,
                 f"long context ({dtype})")
    # the same tokens chosen greedily in one native run across the boundary as step by step
    slot = eng.take_slot()
    first = int(eng.step([slot], [toks[:n_prompt]]).argmax())
    run = eng.greedy_run([slot], [first], 12)
    eng.free_slot(slot)
    slot = eng.take_slot()
    tok = int(eng.step([slot], [toks[:n_prompt]]).argmax())
    single = []
    for _ in range(12):
        tok = int(eng.step([slot], [[tok]]).argmax())
        single.append(tok)
    eng.free_slot(slot)
    assert run is not None and [r[0] for r in run] == single


_long_dir = {}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    # every token from the very first one by one: position 0, the first decoded token, the second
    eng = engine_for(model_dirs, name, dtype)
    reqs = {"f1": random_tokens(1, vocab_of(name), 1), "f2": random_tokens(2, vocab_of(name), 2),
            "f6": random_tokens(6, vocab_of(name), 3)}
    steps = T.tail_one_by_one(reqs, 1000)
    check(name, model_dirs, dtype, steps, T.run_in_process(eng, steps), reqs, "first tokens")
    st2 = T.batched(reqs, 3, (5, 1, 0))
    check(name, model_dirs, dtype, st2, T.run_in_process(eng, st2), reqs, "first tokens batched")


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(model_dirs, dtype, tmp_path):
    # the program a user runs, line by line on its standard input, with a poisoned cache
    reqs = requests_of("B")
    steps = T.batched(reqs, 2, (32, 3, 10))
    outs = T.run_program(model_dirs["B"], dtype, steps, str(tmp_path / "out"), 512, vocab_of("B"),
                         env={"DLGO_CACHE_POISON": "1"})
    check("B", model_dirs, dtype, steps, outs, reqs, "trace_run")
    same = T.run_in_process(engine_for(model_dirs, "B", dtype, True, 512), steps)
    for k in outs:
        assert torch.equal(outs[k], same[k]), f"step {k}: the program and the library disagree"


def test_step_refuses_what_it_cannot_run(model_dirs):
    from dlgo_b200.cache import CacheError
    from dlgo_b200.engine.engine import StepError
    eng = engine_for(model_dirs, "A", "float32")
    s = eng.take_slot()
    with pytest.raises(StepError, match="vocabulary"):
        eng.step([s], [[1, 256]])
    with pytest.raises(StepError, match="no token"):
        eng.step([s], [[]])
    with pytest.raises(StepError, match="twice"):
        eng.step([s, s], [[1], [2]])
    with pytest.raises(StepError, match="limit"):
        eng.step([s], [[1] * 129])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([s], [[1, 2]], [[2]])
    with pytest.raises(CacheError):
        eng.step([s + 1], [[1]])
    assert eng.step([s], [[1, 2, 3]], [[]]) is None and eng.length(s) == 3
    eng.free_slot(s)
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(model_dirs, name, dtype):
    import dlgo_b200
    llm = dlgo_b200.load_llm(model_dirs[name], dtype=dtype, max_tokens=1024)
    cfg, w = P.read_model(model_dirs[name])
    lens = [5, 17, 32] if name == "A" else [1, 9, 70]
    prompts = [random_tokens(n, vocab_of(name), 40 + n) for n in lens]
    n_new = 16 if name == "A" else 24
    got = llm.generate(prompts, max_tokens=n_new, greedy=True, ignore_eos=True)
    for p, g in zip(prompts, got):
        assert len(g) == n_new
        want = P.greedy_generate(cfg, w, p, n_new)
        if g != want:
            # a different token is admissible only at a near tie of the plain logits
            k = next(i for i in range(n_new) if g[i] != want[i])
            lg = P.forward(cfg, w, p + want[:k])[-1]
            gap = float(lg[want[k]] - lg[g[k]])
            assert dtype == "bfloat16" and gap < 2e-2 * float(lg.abs().max()), (
                f"{name} {dtype}: token {k} is {g[k]}, plain says {want[k]} (gap {gap:.3e})")
    # one prompt alone gives what it gave inside the batch
    assert llm.generate(prompts[1], max_tokens=n_new, greedy=True, ignore_eos=True) == got[1]
    info = llm.model_info()
    assert info.layers == cfg["num_hidden_layers"] and info.vocab_size == cfg["vocab_size"]


def test_temperature_generation_is_seeded_and_independent_of_the_batch(model_dirs):
    import dlgo_b200
    llm = dlgo_b200.load_llm(model_dirs["B"], dtype="float32", max_tokens=1024)
    prompts = [random_tokens(n, 384, 60 + n) for n in (1, 9, 70, 130)]
    opts = dict(max_tokens=24, temperature=0.8, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=7, ignore_eos=True)
    a = llm.generate(prompts, **opts)
    assert a == llm.generate(prompts, **opts)
    assert a != llm.generate(prompts, **{**opts, "seed": 8})
    seen = []
    llm.generate_stream(prompts[:2], lambda r, t: seen.append((r, t)), **opts)
    assert [t for r, t in seen if r == 1] == a[1]
    # the plain sampler, fed the plain logits and the same counter-based uniforms, picks the same tokens
    cfg, w = P.read_model(model_dirs["B"])
    seq = list(prompts[1])
    for d in range(6):
        lg = P.forward(cfg, w, seq)[-1]
        tok = P.sample_temperature(lg, 0.8, P.philox_uniform(7, d, 1))
        assert tok == a[1][d], f"draw {d}"
        seq.append(tok)
    filt = llm.generate(prompts, max_tokens=8, temperature=0.7, top_k=40, top_p=0.9, seed=3, ignore_eos=True)
    assert filt == llm.generate(prompts, max_tokens=8, temperature=0.7, top_k=40, top_p=0.9, seed=3, ignore_eos=True)
    res = llm.benchmark(prompts, max_tokens=4, greedy=True, ignore_eos=True)
    assert res.output_tokens == 16 and res.tokens_per_sec > 0 and "tok/s" in str(res)


@pytest.mark.parametrize("dtype", DTYPES)
def test_several_greedy_steps_in_one_native_call(model_dirs, dtype):
    # Engine.greedy_run against the same steps taken one by one: same ids, same cache lengths; a stop id
    # ends the run with the step in which it was chosen
    from dlgo_b200.csrc import kernels
    from dlgo_b200.engine.engine import Engine
    eng = Engine(model_dirs["C"], dtype=dtype, max_tokens=1536)
    prompts = [random_tokens(n, vocab_of("C"), 40 + i) for i, n in enumerate([60, 3, 130])]

    def start():
        slots = [eng.take_slot() for _ in prompts]
        first = kernels.argmax(eng.step(slots, prompts)).cpu().tolist()
        return slots, first

    slots, first = start()
    one_by_one, cur = [], first
    for _ in range(70):                                          # across a page edge for every sequence
        cur = kernels.argmax(eng.step(slots, [[t] for t in cur])).cpu().tolist()
        one_by_one.append(cur)
    lens_a = [eng.length(s) for s in slots]
    for s in slots:
        eng.free_slot(s)
    slots, first2 = start()
    assert first2 == first
    run = eng.greedy_run(slots, first, 70)
    assert run == one_by_one and [eng.length(s) for s in slots] == lens_a
    for s in slots:
        eng.free_slot(s)
    # a stop id: the id sequence 1 chose at its 5th step
    stop = one_by_one[4][1]
    expect = next(i for i, ids in enumerate(one_by_one) if stop in ids) + 1
    slots, _ = start()
    run = eng.greedy_run(slots, first, 70, [stop])
    assert len(run) == expect and run == one_by_one[:expect]
    assert [eng.length(s) for s in slots] == [len(p) + expect for p in prompts]
    # and the run goes on from there like the single steps
    more = eng.greedy_run(slots, run[-1], 3)
    assert more == one_by_one[expect:expect + 3]
    for s in slots:
        eng.free_slot(s)
    eng.cache.book.check()
    with pytest.raises(Exception):
        eng.greedy_run([0], [5], 10)                              # a slot that is not held


def test_sampled_steps_in_one_native_call_draw_what_single_steps_draw(model_dirs):
    """Sampled generation with nobody listening token by token runs many steps per native call (a captured
    step that ends with the filters and the draw; draw indices and the repetition penalty's window advance
    in that call): the same tokens as stepping one by one, with every filter on, past a full window of 64
    recent tokens, with sequences that end at different times, and with a second seed through the same
    capture."""
    import dlgo_b200
    llm = dlgo_b200.load_llm(model_dirs["B"], dtype="float32", max_tokens=1536)
    prompts = [random_tokens(n, 384, 90 + n) for n in (3, 40, 70)]
    for seed in (5, 6):
        opts = dict(max_tokens=90, temperature=0.7, top_k=40, top_p=0.9, min_p=0.02, repetition_penalty=1.3, seed=seed)
        stepped = [[] for _ in prompts]
        llm.generate_stream(prompts, lambda r, t: stepped[r].append(t), **opts)      # one step per call
        native = llm.generate(prompts, **opts)
        assert native == stepped, f"seed {seed}"
    plain_t = dict(max_tokens=30, temperature=1.1, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=11, ignore_eos=True)
    stepped = [[] for _ in prompts]
    llm.generate_stream(prompts, lambda r, t: stepped[r].append(t), **plain_t)
    assert llm.generate(prompts, **plain_t) == stepped
    llm.engine.cache.book.check()
    assert llm.engine.cache.book.live_slots() == []



def _cli(*args):
    import subprocess
    import sys
    from traces import ROOT
    p = subprocess.run([sys.executable, "-m", "dlgo_b200", *args], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    return p.stdout, p.stderr


def test_the_command_line_generates_what_the_python_entry_point_does(model_dirs):
    # `python -m dlgo_b200 generate` as a user runs it (the reference's counterpart:
    # examples/simple_chat/main.go:19-22 over dlgo.go:51-115), greedy and sampled, plain and streamed
    import dlgo_b200
    d = model_dirs["B"]
    p1, p2 = random_tokens(9, 384, 41), random_tokens(3, 384, 42)
    ids = [",".join(map(str, p1)), " ".join(map(str, p2))]
    llm = dlgo_b200.load_llm(d, dtype="bfloat16")
    out, err = _cli("generate", d, "--prompt-ids", ids[0], "--prompt-ids", ids[1], "--max-tokens", "6", "--greedy",
                    "--ignore-eos")
    assert "Model: LlamaForCausalLM (3 layers" in err
    want = llm.generate([p1, p2], max_tokens=6, greedy=True, ignore_eos=True)
    assert [[int(t) for t in line.split()] for line in out.strip().splitlines()] == want
    out, _ = _cli("generate", d, "--prompt-ids", ids[0], "--prompt-ids", ids[1], "--max-tokens", "5", "--temp", "0.8",
                  "--seed", "7", "--stream", "--ignore-eos")
    want = llm.generate([p1, p2], max_tokens=5, temperature=0.8, seed=7, ignore_eos=True)
    seen = [[], []]
    for line in out.strip().splitlines():
        r, t = line.split("\t")
        seen[int(r)].append(int(t))
    assert seen == want
    out, err = _cli("generate", d, "--prompt-ids", ids[1], "--max-tokens", "4", "--greedy", "--bench", "--ctx", "64",
                    "--dtype", "float32", "--ignore-eos")
    assert len(out.split()) == 4 and "tok/s" in err and "prompt tokens: 3" in err
    # per-kernel timing a user can switch on (the reference's DLGO_PROFILE): same tokens, a table on stderr
    out2, err = _cli("generate", d, "--prompt-ids", ids[1], "--max-tokens", "4", "--greedy", "--profile", "--dtype",
                     "float32", "--ignore-eos")
    assert out2.split() == out.split()
    assert "kernel entry point" in err and "gemm_simt" in err and "rmsnorm" in err


@pytest.mark.parametrize("dtype", DTYPES)
def test_interleaved_rotation_pairs_from_the_configuration(tmp_path, dtype):
    # config.json's rope_interleaved (the reference's own pairing for this architecture, ops/rope.go:26-31):
    # the same weights give other logits than with split-half pairs, and the engine follows the plain
    # implementation in both, prompts and single tokens
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.engine.engine import Engine
    from dlgo_b200.weights import write_random_model
    cfg = dict(TINY["B"]["cfg"], rope_interleaved=True)
    d = write_random_model(config_from_dict(cfg), 1, str(tmp_path / "inter"), std=0.05)
    reqs = {"i0": random_tokens(70, 384, 5), "i1": random_tokens(9, 384, 6)}
    eng = Engine(d, dtype=dtype, max_tokens=512)
    steps = T.tail_one_by_one(reqs, 8)
    got = T.collect(steps, T.run_in_process(eng, steps), reqs)
    pc, w = P.read_model(d)
    assert pc["rope_interleaved"] is True
    for rid, toks in reqs.items():
        ref = P.forward(pc, w, toks)
        assert_close(got[rid], ref, dtype, f"interleaved {rid}")
        other = P.forward(dict(pc, rope_interleaved=False), w, toks)
        assert float((ref - other).abs().max()) > 1e-3 * float(ref.abs().max()) or len(toks) < 2
