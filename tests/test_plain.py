"""The plain implementation itself, and host-side pieces of the library that can be checked against it
without a GPU (rotary tables, sampling filters)."""
import math

import pytest
import torch

import plain_llama as P
from tiny_configs import TINY, plain_logits, random_tokens


def test_rmsnorm_closed_form():
    # as the reference's own unit test does (ops/norm_test.go:8-52)
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    w = torch.tensor([1.0, 0.5, 2.0, 1.0])
    rms = math.sqrt((1 + 4 + 9 + 16) / 4 + 1e-5)
    assert torch.allclose(P.rmsnorm(x, w, 1e-5), x / rms * w, atol=1e-6)


def test_rope_rotates_pairs_and_keeps_norm():
    freqs = P.rope_frequencies(8, 10000.0, None)
    assert freqs[0] == 1.0 and abs(freqs[1] - 10000.0 ** (-2 / 8)) < 1e-12
    v = torch.arange(1.0, 9.0)
    assert torch.equal(P.rope(v, 0, freqs), v)                 # position 0 is the identity
    r = P.rope(v, 1, freqs)                                   # first pair (0, 4) turns by 1 radian
    assert abs(r[0] - (1 * math.cos(1) - 5 * math.sin(1))) < 1e-5
    assert abs(r[4] - (1 * math.sin(1) + 5 * math.cos(1))) < 1e-5
    assert abs(float(r.norm()) - float(v.norm())) < 1e-4


def test_llama3_scaling_has_three_bands():
    sc = TINY["B"]["cfg"]["rope_scaling"]
    hd, theta = 32, 500000.0
    plain = P.rope_frequencies(hd, theta, None)
    scaled = P.rope_frequencies(hd, theta, sc)
    kept = [i for i in range(16) if scaled[i] == plain[i]]
    divided = [i for i in range(16) if abs(scaled[i] - plain[i] / 4.0) < 1e-15]
    between = [i for i in range(16) if i not in kept and i not in divided]
    assert kept and divided and between                         # all three bands occur at these sizes
    assert max(kept) < min(between) and max(between) < min(divided)
    for i in between:
        assert plain[i] / 4.0 < scaled[i] < plain[i]


def test_library_rotary_tables_match_the_plain_frequencies():
    from dlgo_b200.parts.rope import RotaryEmbedding, rotary_frequencies
    for name in ("A", "B"):
        c = TINY[name]["cfg"]
        f_plain = P.rope_frequencies(c["head_dim"], c["rope_theta"], c["rope_scaling"])
        assert rotary_frequencies(c["head_dim"], c["rope_theta"], c["rope_scaling"]) == f_plain
        pe = RotaryEmbedding(c["head_dim"], c["head_dim"], c["rope_theta"], c["max_position_embeddings"],
                             scaling=c["rope_scaling"])
        cos, sin = pe.tables()
        assert cos.shape == (c["max_position_embeddings"], c["head_dim"] // 2) and cos.dtype == torch.float32
        pos = c["max_position_embeddings"] - 1
        for i in (0, 3, c["head_dim"] // 2 - 1):
            assert abs(float(cos[pos, i]) - math.cos(pos * f_plain[i])) < 1e-6
            assert abs(float(sin[pos, i]) - math.sin(pos * f_plain[i])) < 1e-6
    with pytest.raises(ValueError):
        RotaryEmbedding(16, 18, 1e4, 8)
    with pytest.raises(ValueError):
        RotaryEmbedding(16, 16, 1e4, 8, pairing="other")


def test_attention_single_position_returns_the_value_and_groups_share_kv():
    # layers/gqa_test.go:8-136: one position => output equals V; GQA maps head h to kv head h / (Hq/Hkv)
    q = torch.randn(1, 4 * 8)
    k = torch.randn(1, 2 * 8)
    v = torch.randn(1, 2 * 8)
    o = P.attention(q, k, v, 4, 2, 8)
    assert torch.allclose(o[0, 0:8], v[0, 0:8]) and torch.allclose(o[0, 8:16], v[0, 0:8])
    assert torch.allclose(o[0, 16:24], v[0, 8:16]) and torch.allclose(o[0, 24:32], v[0, 8:16])


def test_attention_is_causal_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 8), torch.randn(6, 8), torch.randn(6, 8)
    full = P.attention(q, k, v, 1, 1, 8)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, 9.0                                    # the future does not reach positions 0..3
    assert torch.allclose(P.attention(q, k2, v2, 1, 1, 8)[:4], full[:4])
    win = P.attention(q, k, v, 1, 1, 8, window=2)
    assert torch.allclose(win[:2], full[:2]) and not torch.allclose(win[5], full[5])
    k3, v3 = k.clone(), v.clone()
    k3[:4], v3[:4] = 5.0, 5.0                                    # position 5 sees keys 4 and 5 only
    assert torch.allclose(P.attention(q, k3, v3, 1, 1, 8, window=2)[5], win[5])


def test_softmax_swiglu_argmax():
    s = P.softmax(torch.tensor([1.0, 2.0, 3.0]))
    assert abs(float(s.sum()) - 1) < 1e-6 and s[2] > s[1] > s[0]
    g, u = torch.tensor([0.0, 1.0, -2.0]), torch.tensor([3.0, 2.0, 1.0])
    want = torch.tensor([0.0, 2.0 / (1 + math.exp(-1.0)), -2.0 / (1 + math.exp(2.0))])
    assert torch.allclose(P.swiglu(g, u), want, atol=1e-6)
    assert P.argmax(torch.tensor([1.0, 5.0, 5.0, 2.0])) == 1     # first maximum wins (ops/ops.go:272-285)


def test_philox_uniform_is_a_counter_function():
    a = P.philox_uniform(7, 3, 2)
    assert a == P.philox_uniform(7, 3, 2) and 0.0 <= a < 1.0
    assert len({P.philox_uniform(7, d, r) for d in range(20) for r in range(5)}) == 100
    assert P.philox_uniform(8, 3, 2) != a
    # known answer of Philox-4x32-10 for an all-zero key and counter (Random123 test vector)
    M = 0xFFFFFFFF
    assert int(P.philox_uniform(0, 0, 0) * 16777216) == (0x6627E8D5 >> 8)


def test_sample_temperature_inverse_cdf():
    logits = torch.log(torch.tensor([0.1, 0.2, 0.3, 0.4]))
    assert P.sample_temperature(logits, 1.0, 0.05) == 0
    assert P.sample_temperature(logits, 1.0, 0.25) == 1
    assert P.sample_temperature(logits, 1.0, 0.95) == 3
    assert P.sample_temperature(torch.tensor([0.0, 100.0, 0.0]), 0.5, 0.5) == 1


def test_whole_model_shapes_and_prefix_property(model_dirs):
    toks = random_tokens(12, 256, 3)
    full = plain_logits(model_dirs["A"], toks)
    assert full.shape == (12, 256) and torch.isfinite(full).all() and float(full.std()) > 0.01
    part = plain_logits(model_dirs["A"], toks[:7])
    assert torch.allclose(full[:7], part, atol=1e-5)            # causal: a prefix does not see what follows
    f64 = plain_logits(model_dirs["A"], toks, "float64")
    assert float((full - f64).abs().max()) < 1e-4 * float(f64.abs().max())


def test_plain_filter_pipeline_in_the_references_order():
    ninf = float("-inf")
    x = torch.log(torch.tensor([0.4, 0.3, 0.15, 0.1, 0.05]))
    assert torch.equal(P.filter_logits(x, [], 1.0, 1.0, 0, 1.0, 0.0), x)
    k = P.filter_logits(x, [], 1.0, 1.0, 3, 1.0, 0.0)
    assert torch.isfinite(k[:3]).all() and torch.isinf(k[3:]).all()
    # after top-k 3 the probabilities are 0.4/0.85, 0.3/0.85, 0.15/0.85: 0.8 is reached with the second
    kp = P.filter_logits(x, [], 1.0, 1.0, 3, 0.8, 0.0)
    assert torch.isfinite(kp[:2]).all() and torch.isinf(kp[2:]).all()
    m = P.filter_logits(x, [], 1.0, 1.0, 0, 1.0, 0.5)           # threshold 0.2
    assert torch.isfinite(m[:2]).all() and torch.isinf(m[2:]).all()
    r = P.filter_logits(torch.tensor([2.0, -2.0, 1.0]), [0, 1, 1, 99, -1], 2.0, 0.5, 0, 1.0, 0.0)
    assert r.tolist() == [2.0, -8.0, 2.0]                       # penalty first, then the temperature
    t = P.filter_logits(torch.tensor([1.0, 4.0, 3.0, 4.0, 2.0]), [], 1.0, 1.0, 3, 1.0, 0.0)
    assert t.tolist() == [ninf, 4.0, 3.0, 4.0, ninf]            # ties at the cutoff stay


def test_plain_primitives_agree_with_the_references_own_c_kernels():
    # tests/golden/primitives.json holds what computerex/dlgo's quant/simd_dot.c computes (made by
    # tests/golden/make_primitives.py); its exp is a 5-digit polynomial, hence 1e-4
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "primitives.json")) as f:
        cases = json.load(f)["cases"]
    assert len(cases) >= 5
    for c in cases:
        x, g, u = (torch.tensor(c[k], dtype=torch.float32) for k in ("x", "gate", "up"))
        torch.testing.assert_close(P.softmax(x), torch.tensor(c["softmax"]), atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(P.swiglu(g, u), torch.tensor(c["swiglu"]), atol=1e-4, rtol=2e-4)
        assert abs(float(g @ u) - c["dot"]) <= 1e-4 * max(1.0, abs(c["dot"]))
        # the weighted sum of values is built from this axpy (models/llm/forward.go:274-277)
        torch.testing.assert_close(x + 0.375 * u, torch.tensor(c["scale_add_0.375"]), atol=1e-6, rtol=1e-6)
