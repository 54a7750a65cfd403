"""A plain, slow implementation of the Llama forward pass, written from the
reference's formulas (computerex/dlgo; file:line cited at each function).

Whole sequences, no cache, one function per part, float32 (or float64) on the
CPU.  It shares no code with the ``dlgo_b200`` package: it parses config.json
with ``json``, reads weights with the ``safetensors`` library, and computes with
elementary torch tensor arithmetic only.

The reference's model code is Go and there is no Go toolchain on the build
machine, so it cannot be imported or compiled for a comparison: this
implementation rests on the formulas as read from the source.  What pins it:
  * the C kernels of quant/simd_dot.c do compile here and anchor softmax,
    swiglu, the dot product and the axpy of the weighted sum through
    tests/golden/primitives.json (made by tests/golden/make_primitives.py);
  * the cases of the reference's own unit tests (ops/norm_test.go,
    ops/rope_test.go, ops/ops_test.go, ops/activation_test.go,
    ops/sampling_test.go), read as text, anchor rmsnorm, rope, softmax, argmax,
    linear, swiglu and the sampling filters (tests/test_reference_vectors.py);
  * inputs for which the formulas give the answer in closed form anchor the
    causal bound, the kv head a query head reads, the score scale, a layer's
    order, the tied head and the three bands of the llama3 scaling (same file).
Differences that
follow from the weight layout, not from the formulas: checkpoints in the
safetensors layout pair rotary dims (i, i + hd/2) (the reference's ``neox``
branch, ops/rope.go:21-25), and the llama3 frequency scaling is not in the
reference at all (it has no rope scaling): it is the published Llama 3.1 rule.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


def read_model(model_dir: str, dtype=torch.float32) -> tuple[dict, Dict[str, torch.Tensor]]:
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            weights[k] = f.get_tensor(k).to(dtype)
    return cfg, weights


def embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x = E[token, :], no scaling for llama (models/llm/forward.go:132-135, forward_batch.go:97-104)."""
    return torch.stack([table[int(t)] for t in tokens])


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum x^2; scale = 1/sqrt(ss/n + eps); out = x * scale * w (ops/norm.go:10-32)."""
    out = torch.empty_like(x)
    n = x.shape[-1]
    for r in range(x.shape[0]):
        ss = (x[r] * x[r]).sum()
        scale = 1.0 / torch.sqrt((ss / n + eps).to(torch.float64))
        out[r] = x[r] * scale.to(x.dtype) * w
    return out


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = W . x for W [out, in], one dot product per output row (blas/blas.go:152-196; models/llm/forward.go:224)."""
    return x @ w.t()


def rope_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> List[float]:
    """theta_i = base^(-2i/dim) (models/llm/workers.go:163-165); then the llama3 rescaling, which the
    reference does not have: wavelengths under orig/high are kept, over orig/low divided by factor,
    between them blended."""
    half = head_dim // 2
    freqs = [1.0 / math.pow(theta, (2 * i) / head_dim) for i in range(half)]
    if not scaling:
        return freqs
    factor, low, high = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
    orig = scaling["original_max_position_embeddings"]
    out = []
    for f in freqs:
        wavelen = 2 * math.pi / f
        if wavelen < orig / high:
            out.append(f)
        elif wavelen > orig / low:
            out.append(f / factor)
        else:
            smooth = (orig / wavelen - low) / (high - low)
            out.append((1 - smooth) * f / factor + smooth * f)
    return out


def rope(vec: torch.Tensor, pos: int, freqs: List[float], interleaved: bool = False) -> torch.Tensor:
    """Rotate one head vector at absolute position `pos`: angle = pos * theta_i in float64, cos/sin
    cast to the working precision (models/llm/workers.go:160-169); pairs (i, i + half) -> (x0 c - x1 s,
    x0 s + x1 c) (ops/rope.go:21-25, models/llm/workers.go:196-204), or, `interleaved`, pairs (2i, 2i + 1)
    (ops/rope.go:26-31, models/llm/workers.go:205-214)."""
    half = len(freqs)
    ang = torch.tensor([float(pos) * f for f in freqs], dtype=torch.float64)
    c = torch.cos(ang).to(torch.float32).to(vec.dtype)
    s = torch.sin(ang).to(torch.float32).to(vec.dtype)
    out = vec.clone()
    if interleaved:
        x0, x1 = vec[0:2 * half:2], vec[1:2 * half:2]
        out[0:2 * half:2] = x0 * c - x1 * s
        out[1:2 * half:2] = x0 * s + x1 * c
        return out
    x0, x1 = vec[:half], vec[half:2 * half]
    out[:half] = x0 * c - x1 * s
    out[half:2 * half] = x0 * s + x1 * c
    return out


def softmax(x: torch.Tensor) -> torch.Tensor:
    """Subtract the max, exp, sum, multiply by 1/sum (ops/ops.go:150-170; exact exp as in
    quant/simd_dot_stub.go:54-74)."""
    e = torch.exp(x - x.max())
    return e * (1.0 / e.sum())


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
              window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention for one whole sequence.  For head h, kv head h / (Hq/Hkv);
    scores s_t = (q . k_t) * 1/sqrt(hd) for t in [0, pos] (the causal bound is the loop bound), softmax,
    weighted sum of values (models/llm/forward.go:258-278; prompts: forward_batch.go:188-207)."""
    T = q.shape[0]
    kv_mul = n_heads // n_kv_heads
    scale = 1.0 / math.sqrt(head_dim)
    out = torch.zeros_like(q)
    for p in range(T):
        lo = 0 if window is None else max(0, p - window + 1)
        for h in range(n_heads):
            g = h // kv_mul
            qh = q[p, h * head_dim:(h + 1) * head_dim]
            kh = k[lo:p + 1, g * head_dim:(g + 1) * head_dim]
            vh = v[lo:p + 1, g * head_dim:(g + 1) * head_dim]
            scores = (kh @ qh) * scale
            pr = softmax(scores)
            out[p, h * head_dim:(h + 1) * head_dim] = pr @ vh
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """h = g / (1 + exp(-g)) * u (ops/activation.go:8-38)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def feed_forward(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """gate and up projections, SwiGLU, down projection (models/llm/forward.go:296-298)."""
    return linear(swiglu(linear(x, wg), linear(x, wu)), wd)


def layer(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, freqs: List[float],
          start_pos: int = 0) -> torch.Tensor:
    """One block: pre-norm, attention, residual, pre-norm, feed-forward, residual
    (models/llm/forward.go:144-169)."""
    hq, hkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // hq
    eps = cfg.get("rms_norm_eps", 1e-5)
    xn = rmsnorm(x, w[prefix + "input_layernorm.weight"], eps)
    q = linear(xn, w[prefix + "self_attn.q_proj.weight"])
    k = linear(xn, w[prefix + "self_attn.k_proj.weight"])
    v = linear(xn, w[prefix + "self_attn.v_proj.weight"])
    inter = bool(cfg.get("rope_interleaved", False))
    for p in range(x.shape[0]):
        for h in range(hq):
            q[p, h * hd:(h + 1) * hd] = rope(q[p, h * hd:(h + 1) * hd], start_pos + p, freqs, inter)
        for h in range(hkv):
            k[p, h * hd:(h + 1) * hd] = rope(k[p, h * hd:(h + 1) * hd], start_pos + p, freqs, inter)
    a = attention(q, k, v, hq, hkv, hd)
    r = x + linear(a, w[prefix + "self_attn.o_proj.weight"])
    rn = rmsnorm(r, w[prefix + "post_attention_layernorm.weight"], eps)
    y = feed_forward(rn, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                     w[prefix + "mlp.down_proj.weight"])
    return r + y


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence (models/llm/forward.go:123-204 applied
    to each position; final norm :189; output matrix = embedding when tied :193-197)."""
    hq = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // hq
    scaling = cfg.get("rope_scaling")
    if scaling and scaling.get("rope_type", scaling.get("type")) in (None, "default"):
        scaling = None
    freqs = rope_frequencies(hd, cfg.get("rope_theta", 10000.0), scaling)
    x = embedding(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        x = layer(x, w, f"model.layers.{i}.", cfg, freqs)
    x = rmsnorm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5))
    out_w = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(x, out_w)


# ------------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor) -> int:
    """First index of the maximum, strict '>' (ops/ops.go:272-285)."""
    best, besti = logits[0].item(), 0
    for i in range(1, logits.shape[0]):
        if logits[i].item() > best:
            best, besti = logits[i].item(), i
    return besti


def philox_uniform(seed: int, draw: int, request: int) -> float:
    """Philox-4x32-10 with key = seed and counter = (draw, request, 0, 0); the first output word's top
    24 bits over 2^24.  (The reference draws from Go's math/rand, models/llm/generate.go:92-95; a
    counter-based draw stands in so a request's numbers do not depend on its batch.)"""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    mask = 0xFFFFFFFF
    c = [draw & mask, request & mask, 0, 0]
    k0, k1 = seed & mask, (seed >> 32) & mask
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c[3] ^ k1) & mask, p0 & mask]
        k0, k1 = (k0 + W0) & mask, (k1 + W1) & mask
    return (c[0] >> 8) / 16777216.0


def sample_temperature(logits: torch.Tensor, temperature: float, u: float) -> int:
    """logits / T, softmax, first index whose running sum reaches u, else the last
    (ops/sampling.go:72-80,167-181); sums in float64 here."""
    p = torch.softmax(logits.to(torch.float64) / temperature, dim=0)
    c = torch.cumsum(p, dim=0)
    idx = int(torch.searchsorted(c, torch.tensor(u, dtype=torch.float64)).item())
    return min(idx, logits.shape[0] - 1)


def filter_logits(logits: torch.Tensor, recent: Sequence[int], penalty: float, temperature: float, top_k: int,
                  top_p: float, min_p: float) -> torch.Tensor:
    """One row through the filters in the reference's order (ops/sampling.go:32-48): repetition penalty
    (:53-69), temperature (:72-80), top-k (:83-95), top-p (:99-138), min-p (:143-165).  Returns a copy;
    dropped tokens hold -inf."""
    x = logits.detach().to(torch.float32).clone()
    n = x.numel()
    ninf = float("-inf")
    if penalty > 1.0:
        seen = set()
        for tok in recent:
            tok = int(tok)
            if tok < 0 or tok >= n or tok in seen:
                continue
            seen.add(tok)
            x[tok] = x[tok] / penalty if x[tok] > 0 else x[tok] * penalty
    if temperature > 0 and temperature != 1.0:
        x = x * (1.0 / temperature)
    if 0 < top_k < n:
        cutoff = sorted(x.tolist(), reverse=True)[top_k - 1]
        x[x < cutoff] = ninf
    if top_p < 1.0:
        probs = softmax(x)
        order = sorted(range(n), key=lambda i: -float(probs[i]))
        cum, last = 0.0, n - 1
        for rank, i in enumerate(order):
            cum += float(probs[i])
            if cum >= top_p:
                last = rank
                break
        drop = torch.ones(n, dtype=torch.bool)
        drop[order[:last + 1]] = False
        x[drop] = ninf
    if min_p > 0:
        probs = softmax(x)
        x[probs < min_p * probs.max()] = ninf
    return x


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n: int) -> List[int]:
    """Greedy continuation by re-running the whole sequence each step (no cache)."""
    seq = list(prompt)
    out = []
    for _ in range(n):
        tok = argmax(forward(cfg, w, seq)[-1])
        out.append(tok)
        seq.append(tok)
    return out
