"""Each part of a layer alone, a model whose layers differ and whose run order repeats and borrows,
and toy parts that are registered from here without a change to the framework: a mixer with state of
its own, a feed-forward with routing, a position encoding.  Needs a GPU."""
import dataclasses
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype, ref):
    return (2e-5 if dtype == "float32" else 3e-2) * max(1.0, float(ref.abs().max()))


def runtime(dtype):
    from dlgo_b200.engine.runtime import Runtime
    return Runtime("cuda:0", dtype)


def bf16_exact(*shape, scale=1.0):
    return (torch.randn(*shape) * scale).to(torch.bfloat16).float()


def make_ctx(rt, cache, seqs):
    """seqs: list of (slot, tokens).  Reserves cache room and returns the step's context."""
    from dlgo_b200.engine.runtime import build_context
    slots = [s for s, _ in seqs]
    starts = [cache.length(s) for s in slots]
    cache.reserve(slots, [len(t) for _, t in seqs])
    return build_context(rt, [t for _, t in seqs], slots, starts, cache.max_seq_len)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_embedding_head_alone(dtype):
    from dlgo_b200.parts import registry as R
    from dlgo_b200.config.spec import PartSpec
    rt = runtime(dtype)
    torch.manual_seed(0)
    w = 1 + 0.1 * bf16_exact(72)
    norm = R.NORMS.build(PartSpec("rmsnorm", {"size": 72, "eps": 2e-6}))
    assert norm.param_specs()["weight"].shape == (72,) and norm.param_specs()["weight"].init == "one_plus_normal"
    norm.load(lambda n: {"weight": w.to(DEV)}[n], rt)
    x = torch.randn(9, 72)
    ref = P.rmsnorm(x, w, 2e-6)
    assert float((norm.forward(x.to(DEV)).float().cpu() - ref).abs().max()) <= tol(dtype, ref)
    table = bf16_exact(33, 72)
    emb = R.EMBEDDINGS.build(PartSpec("token_embedding", {"vocab_size": 33, "hidden_size": 72}))
    emb.load(lambda n: table.to(DEV).to(torch.bfloat16), rt)
    ids = torch.tensor([0, 32, 7], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), table[[0, 32, 7]])
    head = R.HEADS.build(PartSpec("linear_head", {"vocab_size": 33, "hidden_size": 72, "tied_to": "e.weight"}))
    assert head.param_specs() == {}
    head.load(lambda n: table.to(DEV).to(torch.bfloat16), rt)
    xa = bf16_exact(4, 72)
    lg = head.forward(xa.to(DEV).to(DT[dtype]))
    assert lg.dtype == torch.float32
    assert float((lg.cpu() - xa @ table.t()).abs().max()) <= tol(dtype, xa @ table.t())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_alone(dtype):
    from dlgo_b200.parts import registry as R
    from dlgo_b200.config.spec import PartSpec
    rt = runtime(dtype)
    torch.manual_seed(1)
    d, f = 40, 104
    w = {"gate_proj.weight": bf16_exact(f, d, scale=0.3), "up_proj.weight": bf16_exact(f, d, scale=0.3),
         "down_proj.weight": bf16_exact(d, f, scale=0.3)}
    ffn = R.FEED_FORWARDS.build(PartSpec("swiglu", {"hidden_size": d, "intermediate_size": f}))
    assert {k: v.shape for k, v in ffn.param_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    ffn.load(lambda n: w[n].to(DEV).to(torch.bfloat16), rt)
    x = bf16_exact(11, d)
    res = torch.randn(11, d)
    out = res.clone().to(DEV)
    ffn.forward(x.to(DEV).to(DT[dtype]), out, None)
    ref = res + P.feed_forward(x, w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"])
    assert float((out.cpu() - ref).abs().max()) <= tol(dtype, ref)


def plain_mixer(x, w, hq, hkv, hd, freqs, window=None, k_from=None):
    """Attention part in plain form for one whole sequence: projections, rotation, attention, output."""
    q, k, v = P.linear(x, w["q_proj.weight"]), P.linear(x, w["k_proj.weight"]), P.linear(x, w["v_proj.weight"])
    for p in range(x.shape[0]):
        for h in range(hq):
            q[p, h * hd:(h + 1) * hd] = P.rope(q[p, h * hd:(h + 1) * hd], p, freqs) if freqs else q[p, h * hd:(h + 1) * hd]
        for h in range(hkv):
            k[p, h * hd:(h + 1) * hd] = P.rope(k[p, h * hd:(h + 1) * hd], p, freqs) if freqs else k[p, h * hd:(h + 1) * hd]
    if k_from is not None:
        k, v = k_from
    return P.linear(P.attention(q, k, v, hq, hkv, hd, window), w["o_proj.weight"]), (k, v)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,rope", [(None, True), (70, True), (None, False)])
def test_attention_mixer_alone(dtype, window, rope):
    from dlgo_b200.cache.kv_cache import KVCache
    from dlgo_b200.config.spec import PartSpec
    from dlgo_b200.parts import registry as R
    rt = runtime(dtype)
    torch.manual_seed(2)
    d, hq, hkv, hd = 56, 6, 2, 16
    mixer = R.MIXERS.build(PartSpec("gqa_attention", dict(
        hidden_size=d, num_heads=hq, num_kv_heads=hkv, head_dim=hd, scale=hd ** -0.5, window=window,
        position_encoding="rope" if rope else None, cache_group="g")))
    need = mixer.cache_need()
    assert (need.group, need.num_kv_heads, need.head_dim, need.window) == ("g", hkv, hd, window)
    w = {"q_proj.weight": bf16_exact(hq * hd, d, scale=0.5), "k_proj.weight": bf16_exact(hkv * hd, d, scale=0.5),
         "v_proj.weight": bf16_exact(hkv * hd, d, scale=0.3), "o_proj.weight": bf16_exact(d, hq * hd, scale=0.3)}
    mixer.load(lambda n: w[n].to(DEV).to(torch.bfloat16), rt)
    pe = R.POSITION_ENCODINGS.build(PartSpec("rotary", dict(head_dim=hd, rotary_dim=hd, theta=100.0, max_positions=256)))
    pe.prepare(rt)
    cache = KVCache([need], [None], {}, max_tokens=512, max_seq_len=256, dtype=rt.dtype, device=DEV)
    cache.poison()
    L = 150
    x = bf16_exact(L, d)
    freqs = P.rope_frequencies(hd, 100.0, None) if rope else None
    ref, _ = plain_mixer(x, w, hq, hkv, hd, freqs, window)
    slot = cache.take_slot()
    got = torch.zeros(L, d, device=DEV)
    # a prompt of 100, a chunk of 18, then one token at a time
    cuts = [(0, 100), (100, 118)] + [(i, i + 1) for i in range(118, L)]
    for a, b in cuts:
        ctx = make_ctx(rt, cache, [(slot, [0] * (b - a))])
        mixer.forward(x[a:b].to(DEV).to(DT[dtype]), got[a:b], ctx, cache.view(0), None, {"rope": pe})
        ctx.settle(got[a:b])      # a part may leave its last sum to the next reader of the residual
        cache.commit([slot], [b - a])
    assert float((got.cpu() - ref).abs().max()) <= tol(dtype, ref)
    if window:
        assert cache.book.table("g", slot)[0] == -1      # the page behind the window was given back


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_alone(dtype, model_dirs):
    # one pre-norm block of tiny model B against the plain layer function
    from dlgo_b200.cache.kv_cache import KVCache
    from dlgo_b200.config import load_config
    from dlgo_b200.engine.model import CausalLM
    from dlgo_b200.weights import WeightSource
    rt = runtime(dtype)
    cfgobj = load_config(model_dirs["B"])
    model = CausalLM(cfgobj.architecture_spec())
    src = WeightSource(model_dirs["B"], DEV)
    model.load_weights(src, rt)
    cfg, w = P.read_model(model_dirs["B"])
    x = torch.randn(90, 96)
    ref = P.layer(x, w, "model.layers.1.", cfg, P.rope_frequencies(32, cfg["rope_theta"], cfg["rope_scaling"]))
    needs, borrows, states = model.cache_needs()
    cache = KVCache(needs, borrows, states, 256, 256, rt.dtype, DEV)
    slot = cache.take_slot()
    res = x.clone().to(DEV)
    ctx = make_ctx(rt, cache, [(slot, [0] * 90)])
    model.blocks[1].forward(res, ctx, cache.view(1), None, model.positions)
    assert float((res.cpu() - ref).abs().max()) <= tol(dtype, ref)


# ------------------------------------------------ a model whose layers differ, run in an order of its own
def mixed_spec():
    from dlgo_b200.config.spec import ArchitectureSpec, LayerSpec, PartSpec, RunEntry
    d, V = 48, 100
    names = {"mixer": "attn.", "ffn": "ff.", "mixer_norm": "n1.", "ffn_norm": "n2."}
    l0 = LayerSpec("layers.0.", "prenorm",
                   PartSpec("gqa_attention", dict(hidden_size=d, num_heads=3, num_kv_heads=3, head_dim=16, scale=0.25,
                                                  window=40, position_encoding="rope_a", cache_group="win")),
                   PartSpec("swiglu", dict(hidden_size=d, intermediate_size=72)),
                   {"mixer_norm": PartSpec("rmsnorm", dict(size=d, eps=1e-5)),
                    "ffn_norm": PartSpec("rmsnorm", dict(size=d, eps=1e-5))}, names)
    l1 = LayerSpec("layers.1.", "prenorm",
                   PartSpec("gqa_attention", dict(hidden_size=d, num_heads=4, num_kv_heads=1, head_dim=32,
                                                  scale=32 ** -0.5, window=None, position_encoding="rope_b",
                                                  cache_group="full")),
                   PartSpec("swiglu", dict(hidden_size=d, intermediate_size=56)),
                   {"mixer_norm": PartSpec("rmsnorm", dict(size=d, eps=1e-3)),
                    "ffn_norm": PartSpec("rmsnorm", dict(size=d, eps=1e-6))}, names)
    return ArchitectureSpec(
        name="MixedTest", hidden_size=d, vocab_size=V, max_positions=192,
        embedding=PartSpec("token_embedding", dict(vocab_size=V, hidden_size=d)), embedding_prefix="emb.",
        layers=[l0, l1], order=[RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_of=1)],
        final_norm=PartSpec("rmsnorm", dict(size=d, eps=1e-5)), final_norm_prefix="final.",
        head=PartSpec("linear_head", dict(vocab_size=V, hidden_size=d, tied_to=None)), head_prefix="head.",
        position_encodings={
            "rope_a": PartSpec("rotary", dict(head_dim=16, rotary_dim=16, theta=1e4, max_positions=192)),
            "rope_b": PartSpec("rotary", dict(head_dim=32, rotary_dim=16, theta=1e3, max_positions=192))},
        bos_token_id=None, stop_token_ids=())


def random_tensors(spec, seed, scale=0.15):
    from dlgo_b200.engine.model import CausalLM
    torch.manual_seed(seed)
    out = {}
    for name, ps in sorted(CausalLM(spec).expected_tensors().items()):
        t = torch.randn(ps.shape) * scale
        out[name] = (t + 1.0 if ps.init == "one_plus_normal" else t).to(torch.bfloat16)
    return out


def plain_mixed(tensors, tokens):
    w = {k: v.float() for k, v in tensors.items()}
    x = P.embedding(w["emb.weight"], tokens)
    fa, fb = P.rope_frequencies(16, 1e4, None), P.rope_frequencies(16, 1e3, None)

    def sub(prefix):
        return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}

    def run(layer, x, freqs, hq, hkv, hd, window, eps1, eps2, k_from=None):
        p = f"layers.{layer}."
        a, kv = plain_mixer(P.rmsnorm(x, w[p + "n1.weight"], eps1), sub(p + "attn."), hq, hkv, hd, freqs, window, k_from)
        r = x + a
        ff = sub(p + "ff.")
        y = P.feed_forward(P.rmsnorm(r, w[p + "n2.weight"], eps2), ff["gate_proj.weight"], ff["up_proj.weight"],
                           ff["down_proj.weight"])
        return r + y, kv

    x, _ = run(0, x, fa, 3, 3, 16, 40, 1e-5, 1e-5)
    x, kv1 = run(1, x, fb, 4, 1, 32, None, 1e-3, 1e-6)
    x, _ = run(0, x, fa, 3, 3, 16, 40, 1e-5, 1e-5)          # the same layer again, a cache of its own
    x, _ = run(1, x, fb, 4, 1, 32, None, 1e-3, 1e-6, k_from=kv1)   # reads the keys and values of entry 1
    return P.linear(P.rmsnorm(x, w["final.weight"], 1e-5), w["head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_that_differ_in_an_order_that_repeats_and_borrows(dtype):
    import traces as T
    from dlgo_b200.engine.engine import Engine
    spec = mixed_spec()
    tensors = random_tensors(spec, 3)
    eng = Engine(spec=spec, tensors=tensors, dtype=dtype, max_tokens=512)
    eng.cache.poison()
    assert sorted(eng.cache.storage) == ["full", "win"]
    assert eng.cache.storage["win"].shape[0] == 2 and eng.cache.storage["full"].shape[0] == 1
    g = torch.Generator().manual_seed(4)
    reqs = {f"m{i}": torch.randint(0, 100, (n,), generator=g).tolist() for i, n in enumerate([150, 7, 66])}
    refs = {r: plain_mixed(tensors, t) for r, t in reqs.items()}
    for steps in (T.whole(reqs), T.tail_one_by_one(reqs, 32), T.batched(reqs, 3, (32, 3, 20))):
        got = T.collect(steps, T.run_in_process(eng, steps), reqs)
        for r in reqs:
            assert float((got[r] - refs[r]).abs().max()) <= tol(dtype, refs[r]), r
    eng.cache.book.check()
    assert eng.cache.book.groups["win"].pool.n_free == eng.cache.n_pages


# ------------------------------------------------ a toy mixer with state of its own, defined here
def register_toy():
    from dlgo_b200.parts import Mixer, ParamSpec, StateNeed, register_mixer

    class DecaySum(Mixer):
        """y_t = W . s_t with s_t = decay * s_{t-1} + x_t: no cache of keys, a fixed-size state per sequence."""

        def __init__(self, hidden_size, decay):
            super().__init__(hidden_size=hidden_size, decay=decay)
            self.d, self.decay = hidden_size, decay

        def param_specs(self):
            return {"mix.weight": ParamSpec((self.d, self.d))}

        def state_need(self):
            return StateNeed((self.d,), torch.float32)

        def load(self, get, runtime):
            self.w = get("mix.weight").float()

        def forward(self, x, residual, ctx, cache, state, positions):
            assert cache is None and state is not None
            if ctx.decode:
                # one token per sequence: slots come from the device (a captured step has no host copy of them)
                slots = ctx.seq_slot.long()
                s = self.decay * state[slots] + x.float()
                state[slots] = s
                residual += s @ self.w.t()
                return
            off = 0
            for slot, n in zip(ctx.seq_slots_host, ctx.seq_ntok_host):
                for j in range(n):
                    state[slot] = self.decay * state[slot] + x[off + j].float()
                    residual[off + j] += self.w @ state[slot]
                off += n

    register_mixer("toy_decay_sum", DecaySum, replace=True)


def toy_spec():
    from dlgo_b200.config.spec import PartSpec
    spec = mixed_spec()
    l0 = dataclasses.replace(spec.layers[0], mixer=PartSpec("toy_decay_sum", dict(hidden_size=48, decay=0.5)))
    from dlgo_b200.config.spec import RunEntry
    return dataclasses.replace(spec, name="ToyTest", layers=[l0, spec.layers[1]], order=[RunEntry(0), RunEntry(1)])


def plain_toy(tensors, tokens):
    w = {k: v.float() for k, v in tensors.items()}
    x = P.embedding(w["emb.weight"], tokens)
    xn = P.rmsnorm(x, w["layers.0.n1.weight"], 1e-5)
    s = torch.zeros(48)
    a = torch.zeros_like(x)
    for t in range(x.shape[0]):
        s = 0.5 * s + xn[t]
        a[t] = w["layers.0.attn.mix.weight"] @ s
    r = x + a
    y = P.feed_forward(P.rmsnorm(r, w["layers.0.n2.weight"], 1e-5), w["layers.0.ff.gate_proj.weight"],
                       w["layers.0.ff.up_proj.weight"], w["layers.0.ff.down_proj.weight"])
    x = r + y
    sub = {k[len("layers.1.attn."):]: v for k, v in w.items() if k.startswith("layers.1.attn.")}
    a, _ = plain_mixer(P.rmsnorm(x, w["layers.1.n1.weight"], 1e-3), sub, 4, 1, 32, P.rope_frequencies(16, 1e3, None))
    r = x + a
    y = P.feed_forward(P.rmsnorm(r, w["layers.1.n2.weight"], 1e-6), w["layers.1.ff.gate_proj.weight"],
                       w["layers.1.ff.up_proj.weight"], w["layers.1.ff.down_proj.weight"])
    return P.linear(P.rmsnorm(r + y, w["final.weight"], 1e-5), w["head.weight"])


def test_a_toy_mixer_with_state_is_registered_built_and_stepped():
    import traces as T
    from dlgo_b200.engine.engine import Engine
    register_toy()
    spec = toy_spec()
    tensors = random_tensors(spec, 5)
    assert "layers.0.attn.mix.weight" in tensors and "layers.0.attn.q_proj.weight" not in tensors
    eng = Engine(spec=spec, tensors=tensors, dtype="float32", max_tokens=384)     # decode steps replay a graph
    assert list(eng.cache.state.tensors) == [0] and eng.cache.state.tensors[0].shape[1:] == (48,)
    assert sorted(eng.cache.storage) == ["full"] and eng.cache.storage["full"].shape[0] == 1
    g = torch.Generator().manual_seed(6)
    reqs = {f"t{i}": torch.randint(0, 100, (n,), generator=g).tolist() for i, n in enumerate([40, 3, 70, 9])}
    refs = {r: plain_toy(tensors, t) for r, t in reqs.items()}
    # batches of two, one after another: the second batch takes the first one's slots, whose state must be zero again
    for steps in (T.whole(reqs), T.batched(reqs, 2, (8, 2, 30, 5))):
        got = T.collect(steps, T.run_in_process(eng, steps), reqs)
        for r in reqs:
            assert float((got[r] - refs[r]).abs().max()) <= 5e-5 * max(1.0, float(refs[r].abs().max())), r
    assert eng._graphs, "the decode steps should have gone through a captured graph"
    # a part that asks the captured step for host-side slots is told where to look instead
    with pytest.raises(RuntimeError, match="ctx.seq_slot"):
        list(next(iter(eng._graphs.values())).ctx.seq_slots_host)


# ------------------------------------------------ a block with norms after its parts too, defined here
def register_sandwich():
    from dlgo_b200.parts import Block, register_block

    class SandwichBlock(Block):
        """r = x + post_mixer_norm(mixer(mixer_norm(x))); x = r + post_ffn_norm(ffn(ffn_norm(r))): four norms
        (the reference's PostAttnNorm / PostFFNNorm wiring, models/llm/forward.go:158-182)."""

        def forward(self, residual, ctx, cache, state, positions):
            n = self.norms
            for pre, part, post, args in ((n["mixer_norm"], self.mixer, n["post_mixer_norm"], (cache, state, positions)),
                                          (n["ffn_norm"], self.ffn, n["post_ffn_norm"], ())):
                branch = torch.zeros_like(residual)
                if part is self.mixer:
                    part.forward(pre.forward(residual), branch, ctx, *args)
                else:
                    part.forward(pre.forward(residual), branch, ctx)
                ctx.settle(branch)              # slices a contraction may have left unsummed
                residual += post.forward(branch).float()

    register_block("toy_sandwich", SandwichBlock, replace=True)


def sandwich_spec():
    from dlgo_b200.config.spec import PartSpec, RunEntry
    spec = mixed_spec()
    l1 = spec.layers[1]
    norms = dict(l1.norms)
    norms["post_mixer_norm"] = PartSpec("rmsnorm", dict(size=48, eps=1e-4))
    norms["post_ffn_norm"] = PartSpec("rmsnorm", dict(size=48, eps=1e-2))
    names = dict(l1.names)
    names.update(post_mixer_norm="p1.", post_ffn_norm="p2.")
    l1 = dataclasses.replace(l1, block="toy_sandwich", norms=norms, names=names)
    return dataclasses.replace(spec, name="SandwichTest", layers=[l1], order=[RunEntry(0), RunEntry(0)])


def plain_sandwich(tensors, tokens):
    w = {k: v.float() for k, v in tensors.items()}
    x = P.embedding(w["emb.weight"], tokens)
    sub = {k[len("layers.1.attn."):]: v for k, v in w.items() if k.startswith("layers.1.attn.")}
    for _ in range(2):
        a, _ = plain_mixer(P.rmsnorm(x, w["layers.1.n1.weight"], 1e-3), sub, 4, 1, 32,
                           P.rope_frequencies(16, 1e3, None))
        r = x + P.rmsnorm(a, w["layers.1.p1.weight"], 1e-4)
        y = P.feed_forward(P.rmsnorm(r, w["layers.1.n2.weight"], 1e-6), w["layers.1.ff.gate_proj.weight"],
                           w["layers.1.ff.up_proj.weight"], w["layers.1.ff.down_proj.weight"])
        x = r + P.rmsnorm(y, w["layers.1.p2.weight"], 1e-2)
    return P.linear(P.rmsnorm(x, w["final.weight"], 1e-5), w["head.weight"])


def test_a_block_with_four_norms_needs_no_change_to_the_framework():
    import traces as T
    from dlgo_b200.engine.engine import Engine
    register_sandwich()
    spec = sandwich_spec()
    tensors = random_tensors(spec, 12)
    assert {"layers.1.p1.weight", "layers.1.p2.weight", "layers.1.n1.weight", "layers.1.n2.weight"} <= set(tensors)
    eng = Engine(spec=spec, tensors=tensors, dtype="float32", max_tokens=384)
    per_layer = sum(v.numel() * 4 for k, v in tensors.items() if k.startswith("layers.1."))
    # every norm of the block is counted (and, at most, a few bytes of the parts' own constants)
    assert 0 <= eng.weight_bytes() - (per_layer + 4 * (48 + 100 * 48)) <= 64
    g = torch.Generator().manual_seed(13)
    reqs = {f"s{i}": torch.randint(0, 100, (n,), generator=g).tolist() for i, n in enumerate([45, 6, 80])}
    refs = {r: plain_sandwich(tensors, t) for r, t in reqs.items()}
    for steps in (T.whole(reqs), T.tail_one_by_one(reqs, 16), T.batched(reqs, 2, (8, 2, 30))):
        got = T.collect(steps, T.run_in_process(eng, steps), reqs)
        for r in reqs:
            assert float((got[r] - refs[r]).abs().max()) <= 1e-4 * max(1.0, float(refs[r].abs().max())), r


# ---------------- a toy feed-forward with routing and a toy position encoding, both defined here
def register_routed_and_positions():
    from dlgo_b200.parts import (FeedForward, Mixer, ParamSpec, PositionEncoding, register_feed_forward,
                                 register_mixer, register_position_encoding)

    class Top1Experts(FeedForward):
        """Each token goes to the expert whose router logit is largest (fp32 logits, first maximum):
        y = down_e(relu(up_e x))."""

        def __init__(self, hidden_size, n_experts, expert_size):
            super().__init__(hidden_size=hidden_size, n_experts=n_experts, expert_size=expert_size)
            self.d, self.e, self.f = hidden_size, n_experts, expert_size

        def param_specs(self):
            out = {"router.weight": ParamSpec((self.e, self.d))}
            for i in range(self.e):
                out[f"experts.{i}.up.weight"] = ParamSpec((self.f, self.d))
                out[f"experts.{i}.down.weight"] = ParamSpec((self.d, self.f))
            return out

        def load(self, get, runtime):
            self.router = get("router.weight").float()
            self.up = [get(f"experts.{i}.up.weight").float() for i in range(self.e)]
            self.down = [get(f"experts.{i}.down.weight").float() for i in range(self.e)]

        def forward(self, x, residual, ctx):
            xf = x.float()
            choice = (xf @ self.router.t()).argmax(dim=1)
            for i in range(self.e):
                rows = (choice == i).nonzero().flatten()
                if rows.numel():
                    residual[rows] += torch.relu(xf[rows] @ self.up[i].t()) @ self.down[i].t()

    class SineTable(PositionEncoding):
        """table[p, i] = sin(p / period ** (i / dim)): whoever names it scales its input by 1 + table[p]."""

        def __init__(self, dim, period, max_positions):
            super().__init__(dim=dim, period=period, max_positions=max_positions)
            self.dim, self.period, self.max_positions = dim, period, max_positions
            self.table = None

        def prepare(self, runtime):
            p = torch.arange(self.max_positions, dtype=torch.float64)[:, None]
            i = torch.arange(self.dim, dtype=torch.float64)[None, :]
            self.table = torch.sin(p / self.period ** (i / self.dim)).float().to(runtime.device)

    class PositionGate(Mixer):
        """y_t = W . (x_t * (1 + table[pos_t])): no cache, no state, only the position of each token."""

        def __init__(self, hidden_size, position_encoding):
            super().__init__(hidden_size=hidden_size, position_encoding=position_encoding)
            self.d, self.pe = hidden_size, position_encoding

        def param_specs(self):
            return {"gate.weight": ParamSpec((self.d, self.d))}

        def load(self, get, runtime):
            self.w = get("gate.weight").float()

        def forward(self, x, residual, ctx, cache, state, positions):
            assert cache is None and state is None
            t = positions[self.pe].table[ctx.token_pos.long()]
            residual += (x.float() * (1.0 + t)) @ self.w.t()

    register_feed_forward("toy_top1_experts", Top1Experts, replace=True)
    register_position_encoding("toy_sine_table", SineTable, replace=True)
    register_mixer("toy_position_gate", PositionGate, replace=True)


def routed_spec():
    from dlgo_b200.config.spec import PartSpec, RunEntry
    spec = mixed_spec()
    l0 = dataclasses.replace(spec.layers[0],
                             mixer=PartSpec("toy_position_gate", dict(hidden_size=48, position_encoding="sine")),
                             ffn=PartSpec("toy_top1_experts", dict(hidden_size=48, n_experts=3, expert_size=20)))
    pes = dict(spec.position_encodings)
    pes["sine"] = PartSpec("toy_sine_table", dict(dim=48, period=50.0, max_positions=192))
    return dataclasses.replace(spec, name="RoutedTest", layers=[l0, spec.layers[1]], order=[RunEntry(0), RunEntry(1)],
                               position_encodings=pes)


def plain_routed(tensors, tokens):
    w = {k: v.float() for k, v in tensors.items()}
    x = P.embedding(w["emb.weight"], tokens)
    n = x.shape[0]
    xn = P.rmsnorm(x, w["layers.0.n1.weight"], 1e-5)
    pos = torch.arange(n, dtype=torch.float64)[:, None]
    table = torch.sin(pos / 50.0 ** (torch.arange(48, dtype=torch.float64)[None, :] / 48)).float()
    r = x + (xn * (1.0 + table)) @ w["layers.0.attn.gate.weight"].t()
    xn = P.rmsnorm(r, w["layers.0.n2.weight"], 1e-5)
    y = torch.zeros_like(r)
    used = set()
    for t in range(n):
        e = P.argmax(w["layers.0.ff.router.weight"] @ xn[t])
        used.add(e)
        y[t] = w[f"layers.0.ff.experts.{e}.down.weight"] @ torch.relu(w[f"layers.0.ff.experts.{e}.up.weight"] @ xn[t])
    x = r + y
    sub = {k[len("layers.1.attn."):]: v for k, v in w.items() if k.startswith("layers.1.attn.")}
    a, _ = plain_mixer(P.rmsnorm(x, w["layers.1.n1.weight"], 1e-3), sub, 4, 1, 32, P.rope_frequencies(16, 1e3, None))
    r = x + a
    y = P.feed_forward(P.rmsnorm(r, w["layers.1.n2.weight"], 1e-6), w["layers.1.ff.gate_proj.weight"],
                       w["layers.1.ff.up_proj.weight"], w["layers.1.ff.down_proj.weight"])
    return P.linear(P.rmsnorm(r + y, w["final.weight"], 1e-5), w["head.weight"]), used


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_need_no_change_to_the_framework():
    import traces as T
    from dlgo_b200.engine.engine import Engine
    register_routed_and_positions()
    spec = routed_spec()
    tensors = random_tensors(spec, 8)
    assert "layers.0.ff.experts.2.down.weight" in tensors and "layers.0.ff.gate_proj.weight" not in tensors
    eng = Engine(spec=spec, tensors=tensors, dtype="float32", max_tokens=384, cuda_graphs=False)
    assert sorted(eng.cache.storage) == ["full"] and not eng.cache.state.tensors
    g = torch.Generator().manual_seed(9)
    reqs = {f"r{i}": torch.randint(0, 100, (n,), generator=g).tolist() for i, n in enumerate([50, 4, 90])}
    refs, used = {}, set()
    for r_, t in reqs.items():
        refs[r_], u = plain_routed(tensors, t)
        used |= u
    assert len(used) == 3, "the inputs should reach every expert"
    # positions matter in every cutting: whole, the tail token by token, and batches of unequal lengths
    for steps in (T.whole(reqs), T.tail_one_by_one(reqs, 16), T.batched(reqs, 2, (8, 2, 30))):
        got = T.collect(steps, T.run_in_process(eng, steps), reqs)
        for r_ in reqs:
            assert float((got[r_] - refs[r_]).abs().max()) <= 5e-5 * max(1.0, float(refs[r_].abs().max())), r_
