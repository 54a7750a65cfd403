"""Two tiny configurations of the architecture that differ in every size and option, and helpers
that build their model folders and run the engine and the plain implementation on them."""
from __future__ import annotations

import functools
import os
from typing import Dict, List, Sequence

import torch

TINY: Dict[str, dict] = {
    # 2 layers, hidden 64, 4 heads / 2 kv heads of 16, ffn 160, vocab 256, theta 1e4, no scaling, tied
    "A": dict(cfg=dict(hidden_size=64, num_hidden_layers=2, intermediate_size=160, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, vocab_size=256, rope_theta=10000.0, rope_scaling=None,
                       rms_norm_eps=1e-5, max_position_embeddings=128, tie_word_embeddings=True,
                       architectures=["LlamaForCausalLM"]), seed=0),
    # 3 layers, hidden 96, 3 heads / 1 kv head of 32, ffn 256, vocab 384, theta 5e5, llama3 scaling, untied
    "B": dict(cfg=dict(hidden_size=96, num_hidden_layers=3, intermediate_size=256, num_attention_heads=3,
                       num_key_value_heads=1, head_dim=32, vocab_size=384, rope_theta=500000.0,
                       rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                         original_max_position_embeddings=64),
                       rms_norm_eps=1e-6, max_position_embeddings=256, tie_word_embeddings=False,
                       architectures=["LlamaForCausalLM"]), seed=1),
    # sizes that are no power of two anywhere: 5 heads / 5 kv heads of 48, hidden 200, ffn 328, vocab 1000
    "C": dict(cfg=dict(hidden_size=200, num_hidden_layers=2, intermediate_size=328, num_attention_heads=5,
                       num_key_value_heads=5, head_dim=48, vocab_size=1000, rope_theta=25000.0, rope_scaling=None,
                       rms_norm_eps=3e-6, max_position_embeddings=640, tie_word_embeddings=False,
                       architectures=["LlamaForCausalLM"]), seed=2),
}


def write_tiny(name: str, out_dir: str, std: float = 0.02, sharpen: float = 1.0) -> str:
    """The model folder of a tiny configuration.  `sharpen` > 1 scales the query and key projections,
    so that attention is far from uniform and a wrong or missing key changes the logits visibly."""
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.weights import Checkpoint, save_tensors, write_random_model
    cfg = config_from_dict(TINY[name]["cfg"])
    write_random_model(cfg, TINY[name]["seed"], out_dir, std=std)
    if sharpen != 1.0:
        ck = Checkpoint(out_dir)
        tensors = {n: ck.read(n).clone() for n in ck.names()}
        ck.close()
        for n in tensors:
            if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
                tensors[n] = (tensors[n].float() * sharpen).to(tensors[n].dtype)
        save_tensors(os.path.join(out_dir, "model.safetensors"), tensors)
    return out_dir


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


@functools.lru_cache(maxsize=64)
def _plain_cached(model_dir: str, tokens: tuple, dtype_name: str) -> torch.Tensor:
    import plain_llama as P
    dt = torch.float64 if dtype_name == "float64" else torch.float32
    cfg, w = P.read_model(model_dir, dt)
    return P.forward(cfg, w, list(tokens)).to(torch.float32)


def plain_logits(model_dir: str, tokens: Sequence[int], dtype_name: str = "float32") -> torch.Tensor:
    """Logits [T, vocab] of the plain implementation for one whole sequence (cached per test session)."""
    return _plain_cached(model_dir, tuple(int(t) for t in tokens), dtype_name)


def tolerance(dtype: str, ref: torch.Tensor) -> float:
    """Largest absolute difference allowed, relative to the size of the logits compared."""
    scale = float(ref.abs().max())
    return (1e-4 if dtype == "float32" else 3e-2) * scale


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str) -> None:
    got = got.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    diff = (got - ref).abs()
    tol = tolerance(dtype, ref)
    worst = int(diff.max(dim=-1).values.argmax()) if diff.dim() > 1 else 0
    assert float(diff.max()) <= tol, (
        f"{what}: max abs diff {float(diff.max()):.3e} > {tol:.3e} (first row over: "
        f"{int((diff.max(dim=-1).values > tol).nonzero()[0]) if diff.dim() > 1 else 0}, worst row {worst})")
