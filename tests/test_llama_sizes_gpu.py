"""The engine at the layer sizes of Llama 3.2 1B (hidden 2048, 32/8 heads of 64, feed-forward 8192,
vocabulary 128256, llama3 rope scaling factor 32, tied head) with FOUR layers instead of sixteen so
that the plain implementation stays within a minute on the CPU.  These sizes take the kernels the
tiny models never reach: the tensor-core prompt attention (head size 64), 128 x 256 GEMM tiles over
many tiles, K-slices, a vocabulary that is no multiple of any tile.  The same at the layer sizes of
Llama 3.2 3B and Llama 3.1 8B (heads of 128, three and four query heads per kv head, an untied head).
Needs a GPU."""
import pytest
import torch

import plain_llama as P
import traces as T

pytestmark = pytest.mark.gpu

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, num_hidden_layers=4, intermediate_size=8192,
           num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=128256, rope_theta=500000.0,
           rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                             original_max_position_embeddings=8192),
           rms_norm_eps=1e-5, max_position_embeddings=131072, tie_word_embeddings=True)
# Llama 3.1 8B layer sizes (hidden 4096, 32/8 heads of 128, feed-forward 14336, untied head, rope factor 8),
# two layers and a 32000 vocabulary to keep the plain implementation quick: head size 128 everywhere
CFG_8B = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=2, intermediate_size=14336,
              num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=32000, rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=8192),
              rms_norm_eps=1e-5, max_position_embeddings=131072, tie_word_embeddings=False)
# Llama 3.2 3B layer sizes (hidden 3072, 24/8 heads of 128: three query heads per kv head, feed-forward 8192, tied),
# two layers and a 32000 vocabulary
CFG_3B = dict(architectures=["LlamaForCausalLM"], hidden_size=3072, num_hidden_layers=2, intermediate_size=8192,
              num_attention_heads=24, num_key_value_heads=8, head_dim=128, vocab_size=32000, rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=8192),
              rms_norm_eps=1e-5, max_position_embeddings=131072, tie_word_embeddings=True)
ROWS = [0, 1, 63, 64, 127, 128, 141] + list(range(142, 150))       # places compared (the last 8 are decoded)


def build(tmp_path_factory, CFG, seed):
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.weights import write_random_model
    d = str(tmp_path_factory.mktemp("llama_sizes"))
    write_random_model(config_from_dict(CFG), seed, d, device="cuda")
    g = torch.Generator().manual_seed(3)
    reqs = {"long": torch.randint(0, CFG["vocab_size"], (150,), generator=g).tolist(),
            "short": torch.randint(0, CFG["vocab_size"], (21,), generator=g).tolist()}
    cfg, w = P.read_model(d)
    freqs = P.rope_frequencies(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
    refs = {}
    for rid, toks in reqs.items():
        x = P.embedding(w["model.embed_tokens.weight"], toks)
        for i in range(cfg["num_hidden_layers"]):
            x = P.layer(x, w, f"model.layers.{i}.", cfg, freqs)
        rows = [r for r in ROWS if r < len(toks)] if rid == "long" else list(range(len(toks)))
        xn = P.rmsnorm(x[rows], w["model.norm.weight"], cfg["rms_norm_eps"])
        head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
        refs[rid] = (rows, P.linear(xn, head))
    del w
    return d, reqs, refs


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    return build(tmp_path_factory, CFG, 2)


@pytest.fixture(scope="module")
def big8(tmp_path_factory):
    return build(tmp_path_factory, CFG_8B, 5)


@pytest.fixture(scope="module")
def big3(tmp_path_factory):
    return build(tmp_path_factory, CFG_3B, 4)


def run(engine, reqs, refs, dtype, what):
    long_rows = refs["long"][0]
    n = len(reqs["long"])
    # whole: both requests in one step; then the long one again with its last 8 tokens one by one
    steps = [{"step": 0, "entries": [{"id": "long", "tokens": reqs["long"], "want": long_rows},
                                      {"id": "short", "tokens": reqs["short"], "want": list(range(len(reqs["short"])))}],
              "end": ["long", "short"]},
             {"step": 1, "entries": [{"id": "l2", "tokens": reqs["long"][:n - 8], "want": [r for r in long_rows if r < n - 8]}],
              "end": []}]
    for j in range(n - 8, n):
        steps.append({"step": len(steps), "entries": [{"id": "l2", "tokens": [reqs["long"][j]], "want": [0]}],
                      "end": ["l2"] if j == n - 1 else []})
    outs = T.run_in_process(engine, steps)
    tol = 1e-4 if dtype == "float32" else 3e-2
    ref_long, ref_short = refs["long"][1], refs["short"][1]
    scale = float(ref_long.abs().max())

    def close(got, ref, name):
        assert torch.isfinite(got).all(), name
        err = float((got - ref).abs().max())
        assert err <= tol * scale, f"{what} {name} ({dtype}): max abs diff {err:.3e} > {tol * scale:.3e}"

    close(outs[0][:len(long_rows)], ref_long, "whole, long")
    close(outs[0][len(long_rows):], ref_short, "whole, short beside it")
    k = len([r for r in long_rows if r < n - 8])
    close(outs[1], ref_long[:k], "prefix")
    tail = torch.cat([outs[s] for s in range(2, 10)])
    close(tail, ref_long[k:], "last 8 one by one")
    # the long request once more, fed in three pieces (several tokens on top of a cache that is not empty)
    cuts = [(0, 60), (60, 130), (130, n)]
    steps = [{"step": i, "entries": [{"id": "l3", "tokens": reqs["long"][a:b],
                                      "want": [r - a for r in long_rows if a <= r < b]}],
              "end": ["l3"] if b == n else []} for i, (a, b) in enumerate(cuts)]
    outs = T.run_in_process(engine, steps)
    close(torch.cat([outs[i] for i in range(3) if i in outs]), ref_long, "in three pieces")
    from dlgo_b200.csrc import kernels
    kernels.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_llama_1b_sizes_against_the_plain_implementation(big, dtype):
    from dlgo_b200.engine.engine import Engine
    d, reqs, refs = big
    eng = Engine(d, dtype=dtype, max_tokens=512, max_seq_len=256)
    eng.cache.poison()
    run(eng, reqs, refs, dtype, "graphs")
    if dtype == "bfloat16":
        eng2 = Engine(d, dtype=dtype, max_tokens=512, max_seq_len=256, cuda_graphs=False)
        eng2.cache.poison()
        run(eng2, reqs, refs, dtype, "no graphs")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_llama_8b_layer_sizes_against_the_plain_implementation(big8, dtype):
    from dlgo_b200.engine.engine import Engine
    d, reqs, refs = big8
    eng = Engine(d, dtype=dtype, max_tokens=512, max_seq_len=256)
    eng.cache.poison()
    run(eng, reqs, refs, dtype, "8B sizes")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_llama_3b_layer_sizes_against_the_plain_implementation(big3, dtype):
    from dlgo_b200.engine.engine import Engine
    d, reqs, refs = big3
    eng = Engine(d, dtype=dtype, max_tokens=512, max_seq_len=256)
    eng.cache.poison()
    run(eng, reqs, refs, dtype, "3B sizes")
