"""The plain implementation against the cases of computerex/dlgo's own unit tests, and against results
that follow from its formulas by hand.

The reference is a Go module and no Go toolchain exists here, so its model code cannot run.  Its unit
tests, read as text, still give inputs with expected outputs (ops/norm_test.go, ops/rope_test.go,
ops/ops_test.go, ops/activation_test.go, ops/sampling_test.go); each case below cites the test it
restates and uses that test's own tolerance.  The second half pins what those small cases do not reach
(the causal bound, which kv head a query head reads, the order of a layer, tying) with inputs for which
the reference's formulas give the answer in closed form.  No GPU.
"""
import math

import pytest
import torch

import plain_llama as P


def close(got, want, tol):
    got = [float(v) for v in (got.tolist() if torch.is_tensor(got) else got)]
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        assert abs(g - w) <= tol, (i, g, w)


# ----------------------------------------------------------------- cases of the reference's unit tests
def test_rmsnorm_cases():
    # ops/norm_test.go:8-22 (TestRMSNorm): x = 1..4, unit weights, eps 1e-5; out = x / sqrt(7.5 + eps), tol 1e-3
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    rms = math.sqrt(7.5 + 1e-5)
    close(P.rmsnorm(x, torch.ones(4), 1e-5)[0], [v / rms for v in (1, 2, 3, 4)], 1e-3)
    # ops/norm_test.go:24-38 (TestRMSNormInPlace): x = 2, 4, 6, weights 0.5
    x = torch.tensor([[2.0, 4.0, 6.0]])
    rms = math.sqrt((4 + 16 + 36) / 3.0)
    close(P.rmsnorm(x, torch.full((3,), 0.5), 1e-5)[0], [0.5 * v / rms for v in (2, 4, 6)], 1e-3)
    # ops/norm_test.go:40-52 (TestRMSNormWithScaledWeights): equal inputs normalise to 1, so out = w, tol 1e-2
    close(P.rmsnorm(torch.ones(1, 4), torch.tensor([2.0, 3.0, 4.0, 5.0]), 1e-5)[0], [2, 3, 4, 5], 1e-2)


def test_rope_cases():
    # ops/rope_test.go:8-21,23-36: position 0 changes nothing, in either pairing
    f4 = P.rope_frequencies(4, 10000.0, None)
    close(P.rope(torch.tensor([1.0, 0.0, 0.0, 0.0]), 0, f4), [1, 0, 0, 0], 1e-5)
    # ops/rope_test.go:38-50 (TestRoPERotation): head of 2, base 1, position 1: (1, 0) -> (cos 1, sin 1).
    # With one pair the two pairings coincide, so the split-half rotation must give the same.
    f2 = P.rope_frequencies(2, 1.0, None)
    assert f2 == [1.0]
    close(P.rope(torch.tensor([1.0, 0.0]), 1, f2), [math.cos(1), math.sin(1)], 1e-5)
    # ops/rope_test.go:52-72 (TestRoPEFrequencyTable): theta_i = base^(-2i/dim) (models/llm/workers.go:163-165)
    close(f4, [1.0, 10000.0 ** -0.5], 1e-12)
    # split-half pairs (i, i + hd/2): ops/rope.go:21-25.  A unit vector in dim 1 at position 3 moves into
    # dims 1 and 3 by the SECOND frequency's angle.
    a = 3 * f4[1]
    close(P.rope(torch.tensor([0.0, 1.0, 0.0, 0.0]), 3, f4), [0, math.cos(a), 0, math.sin(a)], 1e-6)


def test_softmax_argmax_matvec_dot_cases():
    # ops/ops_test.go:121-134 (TestSoftmax): sums to one, keeps the order
    s = P.softmax(torch.tensor([1.0, 2.0, 3.0]))
    assert abs(float(s.sum()) - 1.0) <= 1e-5 and s[0] < s[1] < s[2]
    # ops/ops_test.go:175-183 (TestArgmax)
    assert P.argmax(torch.tensor([1.0, 5.0, 3.0, 2.0])) == 1
    # ops/ops_test.go:193-201 (TestMatVecMul): the identity
    close(P.linear(torch.tensor([[3.0, 7.0]]), torch.tensor([[1.0, 0.0], [0.0, 1.0]]))[0], [3, 7], 0)
    # ops/ops_test.go:153-161 (TestDotProduct)
    a = torch.arange(1.0, 10.0)
    assert abs(float(P.linear(a[None], a.flip(0)[None])[0, 0]) - 165.0) <= 1e-4


def test_swiglu_cases():
    # ops/activation_test.go:16-27 (TestSwiGLU): gate 0, 1, -1, 2, up 1; out = g / (1 + exp(-g)), tol 1e-5
    g = torch.tensor([0.0, 1.0, -1.0, 2.0])
    close(P.swiglu(g, torch.ones(4)), [v / (1 + math.exp(-v)) for v in (0, 1, -1, 2)], 1e-5)
    # ops/activation_test.go:45-52: a zero gate gives zero whatever the up value
    close(P.swiglu(torch.zeros(3), torch.tensor([5.0, -3.0, 9.0])), [0, 0, 0], 0)


def test_sampling_cases():
    ninf = float("-inf")
    # ops/sampling_test.go:9-16 (greedy): temperature 0 picks the maximum
    assert P.argmax(torch.tensor([1.0, 5.0, 2.0, 3.0])) == 1
    # ops/sampling_test.go:18-30: one overwhelming logit is drawn whatever the uniform number
    lg = torch.tensor([100.0, -100.0, -100.0, -100.0])
    assert all(P.sample_temperature(lg, 0.1, u) == 0 for u in (0.0, 0.3, 0.999999))
    # ops/sampling_test.go:32-46 (repetition penalty 2 over tokens 0 and 1)
    r = P.filter_logits(torch.tensor([2.0, -1.0, 3.0, 0.0]), [0, 1], 2.0, 1.0, 0, 1.0, 0.0)
    close(r, [1, -2, 3, 0], 1e-5)
    # ops/sampling_test.go:48-57 (temperature 2 halves the logits)
    close(P.filter_logits(torch.tensor([2.0, 4.0, 6.0]), [], 1.0, 2.0, 0, 1.0, 0.0), [1, 2, 3], 1e-5)
    # ops/sampling_test.go:59-70 (top-k 2 keeps 5 and 4)
    k = P.filter_logits(torch.tensor([1.0, 4.0, 2.0, 5.0, 3.0]), [], 1.0, 1.0, 2, 1.0, 0.0)
    assert k.tolist() == [ninf, 4.0, ninf, 5.0, ninf]
    # ops/sampling_test.go:72-80 (top-p 0.5 keeps the dominant token) and :82-89 (min-p 0.1 keeps the top token)
    assert P.filter_logits(torch.tensor([10.0, 1.0, 1.0, 1.0]), [], 1.0, 1.0, 0, 0.5, 0.0).tolist() == [10.0, ninf, ninf, ninf]
    assert float(P.filter_logits(torch.tensor([10.0, 5.0, 1.0, -5.0]), [], 1.0, 1.0, 0, 1.0, 0.1)[0]) == 10.0


# ------------------------------------------------------------- closed-form consequences of the formulas
def test_zero_queries_average_the_values_up_to_the_position_per_kv_head():
    # models/llm/forward.go:258-278: scores over t in [0, pos] only, kv head = h / (Hq/Hkv).  With q = 0 every
    # score is 0, the softmax is uniform over 0..pos, so head h's output at pos is the running mean of kv head
    # h // 2's values: a key beyond pos, or the other kv head, would change it.
    T, hq, hkv, hd = 6, 4, 2, 4
    torch.manual_seed(0)
    v = torch.randn(T, hkv * hd)
    k = torch.randn(T, hkv * hd)
    out = P.attention(torch.zeros(T, hq * hd), k, v, hq, hkv, hd)
    for p in range(T):
        for h in range(hq):
            g = h // (hq // hkv)
            want = v[:p + 1, g * hd:(g + 1) * hd].mean(0)
            torch.testing.assert_close(out[p, h * hd:(h + 1) * hd], want, atol=1e-6, rtol=1e-6)


def test_a_dominant_key_is_found_and_scaled_by_one_over_sqrt_head_size():
    # scores are (q . k) / sqrt(hd) (models/llm/forward.go:260-266): with q . k_2 = 40 * sqrt(hd) against zeros
    # elsewhere the probabilities are softmax([0, 0, 40, 0]); without the scale they would differ
    hd, T = 16, 4
    q = torch.zeros(T, hd)
    k = torch.zeros(T, hd)
    q[3, 0] = 40.0
    k[2, 0] = math.sqrt(hd)
    v = torch.eye(T, hd)
    out = P.attention(q, k, v, 1, 1, hd)
    pr = P.softmax(torch.tensor([0.0, 0.0, 40.0, 0.0]))
    torch.testing.assert_close(out[3, :T], pr, atol=1e-6, rtol=1e-6)
    # a window of 1 (the query sees only itself) gives its own value back
    torch.testing.assert_close(P.attention(q, k, v, 1, 1, hd, window=1), v, atol=0, rtol=0)


def test_one_layer_by_hand_and_tying():
    # models/llm/forward.go:144-169 with numbers small enough to follow: identity-like weights, one head.
    # r = x + Wo . attn(norm(x)); out = r + Wd . swiglu(Wg . norm(r), Wu . norm(r)).  Logits with a tied head
    # are E . norm(out) (forward.go:189-197).
    d = 2
    cfg = dict(hidden_size=d, num_hidden_layers=1, intermediate_size=d, num_attention_heads=1, num_key_value_heads=1,
               head_dim=d, vocab_size=3, rope_theta=1.0, rope_scaling=None, rms_norm_eps=0.0, tie_word_embeddings=True)
    eye = torch.eye(d)
    E = torch.tensor([[3.0, 4.0], [1.0, 0.0], [0.0, 2.0]])
    w = {"model.embed_tokens.weight": E, "model.norm.weight": torch.ones(d)}
    p = "model.layers.0."
    w.update({p + "input_layernorm.weight": torch.ones(d), p + "post_attention_layernorm.weight": torch.ones(d),
              p + "self_attn.q_proj.weight": torch.zeros(d, d), p + "self_attn.k_proj.weight": eye,
              p + "self_attn.v_proj.weight": eye, p + "self_attn.o_proj.weight": eye,
              p + "mlp.gate_proj.weight": eye, p + "mlp.up_proj.weight": eye, p + "mlp.down_proj.weight": eye})
    got = P.forward(cfg, w, [0])
    # token 0: x = (3, 4); norm(x) = x / sqrt(12.5) (eps 0); one position, so attention returns v = norm(x)
    n = lambda a: [v / math.sqrt(sum(t * t for t in a) / len(a)) for v in a]
    x = [3.0, 4.0]
    r = [a + b for a, b in zip(x, n(x))]
    rn = n(r)
    y = [g / (1 + math.exp(-g)) * g for g in rn]
    out = [a + b for a, b in zip(r, y)]
    on = n(out)
    want = [sum(E[v, j].item() * on[j] for j in range(d)) for v in range(3)]
    close(got[0], want, 1e-5)


def test_llama3_scaling_by_hand():
    # three bands around original_max_position = 64 with factor 4, low 1, high 4 (wavelengths 16 and 64):
    # theta^(-2i/8) for i = 0..3 at theta = 500000 gives wavelengths 6.28 (kept), 167, 4443 and 118k (divided by 4)
    sc = dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=64)
    base = [500000.0 ** (-2 * i / 8) for i in range(4)]
    got = P.rope_frequencies(8, 500000.0, sc)
    assert got[0] == pytest.approx(base[0], rel=1e-12)
    for i in (1, 2, 3):
        assert got[i] == pytest.approx(base[i] / 4.0, rel=1e-12)
    # a wavelength inside the band (between 16 and 64): theta = 100, head of 4 -> i = 1 has wavelength 62.8
    f = 100.0 ** -0.5
    smooth = (64 / (2 * math.pi / f) - 1.0) / (4.0 - 1.0)
    assert P.rope_frequencies(4, 100.0, sc)[1] == pytest.approx((1 - smooth) * f / 4.0 + smooth * f, rel=1e-12)
