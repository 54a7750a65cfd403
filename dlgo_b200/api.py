"""The Python entry point, in the manner of the reference's ``dlgo`` package.

Reference: ``LoadLLM(path, maxSeqLen)`` (dlgo.go:37), ``Generate`` (:51),
``GenerateStream`` (:79), ``Benchmark`` (:93), ``ModelInfo`` (:117), and the
options ``WithMaxTokens / WithTemperature / WithTopK / WithTopP / WithSeed /
WithGreedy`` (:213-240) over ``DefaultGenerateConfig`` (models/llm/generate.go:25-31).
Here the options are keyword arguments of the same names and meanings.  Prompts
are token ids (the tokenizer is not part of this library); a call takes one
prompt or a list of prompts, which are generated in batches.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Union

import torch

from .engine.engine import Engine
from .engine.generate import GenerateConfig, GenerateResult, GenerationLoop
from .sampling.sampler import DeviceSampler, SamplerConfig

Prompt = Sequence[int]


@dataclass
class ModelInfo:
    """Counterpart of the reference's ``ModelInfo`` (dlgo.go:170-186)."""

    architecture: str
    layers: int
    dimension: int
    heads: int
    kv_heads: int
    ffn_dim: int
    vocab_size: int
    context_len: int

    def __str__(self) -> str:
        return (f"{self.architecture} ({self.layers} layers, {self.dimension} dim, {self.heads} heads, "
                f"vocab {self.vocab_size}, ctx {self.context_len})")


@dataclass
class BenchmarkResult:
    """Counterpart of the reference's ``BenchmarkResult`` (dlgo.go:188-207)."""

    tokens: List[List[int]]
    tokens_per_sec: float
    prefill_ms: float
    generate_ms: float
    total_ms: float
    prompt_tokens: int
    output_tokens: int
    architecture: str

    def __str__(self) -> str:
        return (f"{self.tokens_per_sec:.1f} tok/s | prefill: {self.prefill_ms:.0f}ms | gen: {self.generate_ms:.0f}ms | "
                f"{self.output_tokens} tokens")


class _EngineBackend:
    """The generation loop's view of the engine: a step followed by sampling on the device."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.max_seq_len = engine.max_seq_len

    def take_slot(self) -> int:
        return self.engine.take_slot()

    def free_slot(self, slot: int) -> None:
        self.engine.free_slot(slot)

    def pages_free(self) -> int:
        return min(g.pool.n_free for g in self.engine.cache.book.groups.values()) \
            if self.engine.cache.book.groups else 1 << 30

    def slots_free(self) -> int:
        return self.engine.cache.book.n_free_slots

    def pages_for(self, n_positions: int) -> int:
        ps = self.engine.cache.page_size
        return (n_positions + ps - 1) // ps

    def greedy_steps(self, slots, tokens, n_steps: int, stop_ids) -> Optional[List[List[int]]]:
        """Several greedy decode steps in one native call (``None``: step one by one)."""
        return self.engine.greedy_run(slots, tokens, n_steps, stop_ids)

    def sampled_steps(self, slots, tokens, n_steps: int, stop_ids, sampler: SamplerConfig, seed: int, requests,
                      draws, recent) -> Optional[List[List[int]]]:
        """Several sampled decode steps in one native call (``None``: step one by one)."""
        return self.engine.sampled_run(slots, tokens, n_steps, stop_ids, sampler, seed, requests, draws, recent)

    def step_and_sample(self, slots, tokens, requests, draws, sampler: SamplerConfig, seed: int, recent) -> List[int]:
        logits = self.engine.step(slots, tokens)
        if sampler.greedy:
            from .csrc import kernels
            return kernels.argmax_to_host(logits)    # kernels, copy and wait in one native call
        ids = DeviceSampler(seed).sample(logits, sampler, requests, draws, recent)   # holds the seed, nothing else
        return ids.cpu().tolist()   # the only device-to-host traffic of a step: one id per sequence


class LLM:
    """A loaded model ready to generate (reference: ``dlgo.LLM``, dlgo.go:31)."""

    def __init__(self, engine: Engine, max_batch: int = 64):
        self.engine = engine
        self.backend = _EngineBackend(engine)
        self.loop = GenerationLoop(self.backend, engine.spec.stop_token_ids, max_batch=max_batch)

    # ---------------------------------------------------------------- generation
    @staticmethod
    def _config(max_tokens: int, temperature: float, top_k: int, top_p: float, min_p: float,
                repetition_penalty: float, seed: int, greedy: bool, stop_token_ids: Sequence[int],
                ignore_eos: bool, include_stop: bool) -> GenerateConfig:
        if greedy:
            temperature = 0.0
        if temperature < 0:
            raise ValueError("temperature must be >= 0")
        return GenerateConfig(
            max_tokens=max_tokens,
            sampler=SamplerConfig(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p,
                                  repetition_penalty=repetition_penalty),
            seed=seed, stop_token_ids=tuple(stop_token_ids), ignore_eos=ignore_eos, include_stop=include_stop)

    def generate_detailed(self, prompts: Union[Prompt, Sequence[Prompt]], *, max_tokens: int = 256,
                          temperature: float = 0.7, top_k: int = 40, top_p: float = 0.9, min_p: float = 0.0,
                          repetition_penalty: float = 1.1, seed: int = -1, greedy: bool = False,
                          stop_token_ids: Sequence[int] = (), ignore_eos: bool = False, include_stop: bool = False,
                          on_token: Optional[Callable[[int, int], None]] = None) -> GenerateResult:
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        batch = [list(prompts)] if single else [list(p) for p in prompts]
        cfg = self._config(max_tokens, temperature, top_k, top_p, min_p, repetition_penalty, seed, greedy,
                           stop_token_ids, ignore_eos, include_stop)
        return self.loop.run(batch, cfg, on_token)

    def generate(self, prompts: Union[Prompt, Sequence[Prompt]], **options) -> Union[List[int], List[List[int]]]:
        """Generated token ids: a list for one prompt, a list of lists for a list of prompts.

        Options: ``max_tokens`` (256), ``temperature`` (0.7; 0 = greedy), ``top_k`` (40),
        ``top_p`` (0.9), ``seed`` (-1 = from the clock), ``greedy``, and beyond the
        reference's: ``min_p``, ``repetition_penalty`` (1.1), ``stop_token_ids``,
        ``ignore_eos``, ``include_stop``.
        """
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        res = self.generate_detailed(prompts, **options)
        return res.tokens[0] if single else res.tokens

    def generate_stream(self, prompts: Union[Prompt, Sequence[Prompt]], on_token: Callable[..., None],
                        **options) -> None:
        """Call ``on_token`` for each token as it is produced: ``on_token(token)`` for one
        prompt, ``on_token(request index, token)`` for a list (reference: ``GenerateStream``, dlgo.go:79)."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        cb = (lambda r, t: on_token(t)) if single else on_token
        self.generate_detailed(prompts, on_token=cb, **options)

    def benchmark(self, prompts: Union[Prompt, Sequence[Prompt]], **options) -> BenchmarkResult:
        import time
        t0 = time.perf_counter()
        res = self.generate_detailed(prompts, **options)
        torch.cuda.synchronize(self.engine.runtime.device)
        total = (time.perf_counter() - t0) * 1e3
        return BenchmarkResult(res.tokens, res.tokens_per_sec, res.prefill_ms, res.generate_ms, total,
                               res.prompt_tokens, res.output_tokens, self.engine.spec.name)

    # ----------------------------------------------------------------- the step
    def step(self, slots, tokens, want=None):
        """The raw step function (see :meth:`Engine.step`)."""
        return self.engine.step(slots, tokens, want)

    def model_info(self) -> ModelInfo:
        c = self.engine.config
        return ModelInfo(
            architecture=self.engine.spec.name, layers=len(self.engine.spec.order),
            dimension=self.engine.spec.hidden_size, heads=getattr(c, "num_attention_heads", 0),
            kv_heads=getattr(c, "num_key_value_heads", 0), ffn_dim=getattr(c, "intermediate_size", 0),
            vocab_size=self.engine.spec.vocab_size, context_len=self.engine.spec.max_positions)


def load_llm(model_path: str, max_seq_len: int = 0, *, dtype: str = "bfloat16", device: str = "cuda:0",
             max_tokens: Optional[int] = None, max_batch: int = 64, cuda_graphs: bool = True) -> LLM:
    """Load a model folder (config.json + model.safetensors) and return a ready LLM.

    ``max_seq_len`` is the longest sequence (0 = the model's context), as in the
    reference's ``LoadLLM(path, maxSeqLen)`` (dlgo.go:37-48).  ``max_tokens`` sizes the
    cache: positions that live sequences may hold together (default: ``max_batch``
    sequences of ``max_seq_len``, within half of the device's free memory).
    """
    engine = Engine(model_path, dtype=dtype, device=device, max_tokens=max_tokens,
                    max_seq_len=max_seq_len if max_seq_len > 0 else None, cuda_graphs=cuda_graphs,
                    default_batch=max_batch)
    return LLM(engine, max_batch=max_batch)
