"""Typed configuration of the Llama architecture, read from its config.json keys.

Counterpart of the reference's ``ModelConfig`` / ``parseConfig``
(models/llm/config.go:11-123), which fills the same numbers from GGUF metadata:
hidden size, layers, feed-forward width, heads, KV heads (default: heads,
config.go:100-102), head size (default: hidden / heads, config.go:103-105),
vocabulary, norm eps (default 1e-5, config.go:61-64), rope base (default 10000,
config.go:77), context (default 2048, config.go:69) and the stop tokens
(config.go:113-120).  The reference has no rope scaling; the llama3 scaling
keys are read here because Llama 3.x checkpoints carry them.

No size stands in code: every number a part is built with comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import ArchitectureSpec, LayerSpec, PartSpec, RunEntry


@dataclass(frozen=True)
class RopeScaling:
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


def _need(d: Mapping[str, Any], key: str, typ: type) -> Any:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing required key {key!r}")
    return _as(d[key], key, typ)


def _as(v: Any, key: str, typ: type) -> Any:
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                return int(v)
            raise ConfigError(f"config.json: {key!r} must be an integer, got {v!r}")
        return v
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {key!r} must be a number, got {v!r}")
        return float(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: {key!r} must be true or false, got {v!r}")
        return v
    raise TypeError(typ)


def _opt(d: Mapping[str, Any], key: str, typ: type, default: Any) -> Any:
    if key not in d or d[key] is None:
        return default
    return _as(d[key], key, typ)


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    max_position_embeddings: int = 2048
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    hidden_act: str = "silu"
    architecture: str = "LlamaForCausalLM"
    # rotation pairs (2i, 2i+1) instead of (i, i + head_dim/2): for weights whose q/k rows were exported in the
    # reference's own order (its llama default, models/llm/arch.go:18, ops/rope.go:26-31).  Checkpoints in the
    # common safetensors layout are split-half: absent or false.
    rope_interleaved: bool = False

    # ------------------------------------------------------------------ derived
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # --------------------------------------------------------------- validation
    def __post_init__(self) -> None:
        pos = {
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
        }
        for k, v in pos.items():
            if v <= 0:
                raise ConfigError(f"config.json: {k!r} must be positive, got {v}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even for rotary pairs")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"config.json: rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(
                f"config.json: hidden_act {self.hidden_act!r} is not supported by this architecture (only 'silu')")
        rs = self.rope_scaling
        if rs is not None:
            if rs.rope_type != "llama3":
                raise ConfigError(
                    f"config.json: rope scaling type {rs.rope_type!r} is not supported (none/'default' or 'llama3')")
            if rs.factor <= 0 or rs.original_max_position_embeddings <= 0:
                raise ConfigError("config.json: rope_scaling factor and original_max_position_embeddings must be > 0")
            if rs.high_freq_factor <= rs.low_freq_factor:
                raise ConfigError("config.json: rope_scaling high_freq_factor must exceed low_freq_factor")

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        hidden = _need(d, "hidden_size", int)
        heads = _need(d, "num_attention_heads", int)
        if heads <= 0:
            raise ConfigError(f"config.json: 'num_attention_heads' must be positive, got {heads}")
        kv_heads = _opt(d, "num_key_value_heads", int, heads)
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _as(d["head_dim"], "head_dim", int)
        else:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size ({hidden}) is not a multiple of num_attention_heads ({heads}) "
                    "and no head_dim is given")
            head_dim = hidden // heads
        for key in ("attention_bias", "mlp_bias"):
            if _opt(d, key, bool, False):
                raise ConfigError(f"config.json: {key}=true is not supported (this architecture has no biases)")

        # rope: either flat keys (rope_theta, rope_scaling) or one rope_parameters object.
        rp = d.get("rope_parameters")
        theta_src: Mapping[str, Any] = d
        scaling_src = d.get("rope_scaling")
        if isinstance(rp, dict):
            if "rope_theta" in rp:
                theta_src = rp
            if scaling_src is None:
                scaling_src = rp
        theta = _opt(theta_src, "rope_theta", float, 10000.0)
        scaling = None
        if scaling_src is not None:
            if not isinstance(scaling_src, dict):
                raise ConfigError("config.json: 'rope_scaling' must be an object or null")
            rtype = scaling_src.get("rope_type", scaling_src.get("type", "default"))
            if rtype not in (None, "default"):
                scaling = RopeScaling(
                    rope_type=str(rtype),
                    factor=_need(scaling_src, "factor", float),
                    low_freq_factor=_opt(scaling_src, "low_freq_factor", float, 1.0),
                    high_freq_factor=_opt(scaling_src, "high_freq_factor", float, 4.0),
                    original_max_position_embeddings=_need(
                        scaling_src, "original_max_position_embeddings", int),
                )

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(_as(e, "eos_token_id", int) for e in eos)
        else:
            eos_ids = (_as(eos, "eos_token_id", int),)

        archs = d.get("architectures") or ["LlamaForCausalLM"]
        if isinstance(archs, str):
            archs = [archs]
        return cls(
            hidden_size=hidden,
            num_hidden_layers=_need(d, "num_hidden_layers", int),
            intermediate_size=_need(d, "intermediate_size", int),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_need(d, "vocab_size", int),
            rms_norm_eps=_opt(d, "rms_norm_eps", float, 1e-5),
            rope_theta=theta,
            rope_scaling=scaling,
            max_position_embeddings=_opt(d, "max_position_embeddings", int, 2048),
            tie_word_embeddings=_opt(d, "tie_word_embeddings", bool, False),
            rope_interleaved=_opt(d, "rope_interleaved", bool, False),
            bos_token_id=_opt(d, "bos_token_id", int, None),
            eos_token_ids=eos_ids,
            hidden_act=str(d.get("hidden_act", "silu")),
            architecture=str(archs[0]),
        )

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else asdict(self.rope_scaling),
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": "bfloat16",
        }
        if self.rope_interleaved:
            d["rope_interleaved"] = True
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d

    # ------------------------------------------------------- architecture as data
    def architecture_spec(self) -> ArchitectureSpec:
        """Llama as a list of parts: every layer is a pre-norm block of grouped-query
        attention (rotary positions) and a SwiGLU feed-forward, run once each in
        index order (models/llm/forward.go:137-183)."""
        rope_params: Dict[str, Any] = {
            "head_dim": self.head_dim,
            "rotary_dim": self.head_dim,
            "theta": self.rope_theta,
            "max_positions": self.max_position_embeddings,
            "pairing": "interleaved" if self.rope_interleaved else "split_half",
        }
        if self.rope_scaling is not None:
            rope_params["scaling"] = asdict(self.rope_scaling)
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        mixer = PartSpec("gqa_attention", {
            "hidden_size": self.hidden_size,
            "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "scale": self.head_dim ** -0.5,
            "window": None,
            "position_encoding": "rope",
            "cache_group": "full",
        })
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        layers: List[LayerSpec] = []
        for i in range(self.num_hidden_layers):
            layers.append(LayerSpec(
                prefix=f"model.layers.{i}.",
                block="prenorm",
                mixer=mixer,
                ffn=ffn,
                norms={"mixer_norm": norm, "ffn_norm": norm},
                names={"mixer": "self_attn.", "ffn": "mlp.",
                       "mixer_norm": "input_layernorm.", "ffn_norm": "post_attention_layernorm."},
            ))
        spec = ArchitectureSpec(
            name=self.architecture,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            embedding_prefix="model.embed_tokens.",
            layers=layers,
            order=[RunEntry(i) for i in range(self.num_hidden_layers)],
            final_norm=norm,
            final_norm_prefix="model.norm.",
            head=PartSpec("linear_head", {
                "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None}),
            head_prefix="lm_head.",
            position_encodings={"rope": PartSpec("rotary", rope_params)},
            bos_token_id=self.bos_token_id,
            stop_token_ids=tuple(self.eos_token_ids),
        )
        spec.validate()
        return spec


register_architecture("LlamaForCausalLM", LlamaConfig)
