"""Configuration and registry (no GPU)."""
import json

import pytest

from dlgo_b200.config import (ConfigError, LlamaConfig, config_from_dict, load_config, register_architecture,
                              registered_architectures)
from dlgo_b200.config.spec import ArchitectureSpec, RunEntry
from tiny_configs import TINY


def test_reads_every_key_of_both_tiny_configs():
    a = config_from_dict(TINY["A"]["cfg"])
    b = config_from_dict(TINY["B"]["cfg"])
    assert (a.hidden_size, a.num_hidden_layers, a.intermediate_size) == (64, 2, 160)
    assert (a.num_attention_heads, a.num_key_value_heads, a.head_dim, a.vocab_size) == (4, 2, 16, 256)
    assert a.rope_scaling is None and a.tie_word_embeddings and a.rms_norm_eps == 1e-5
    assert (b.q_dim, b.kv_dim, b.group_size) == (96, 32, 3)
    assert b.rope_scaling.rope_type == "llama3" and b.rope_scaling.factor == 4.0
    assert b.rope_scaling.original_max_position_embeddings == 64
    assert b.rope_theta == 500000.0 and not b.tie_word_embeddings and b.rms_norm_eps == 1e-6


def test_defaults_follow_the_reference():
    c = LlamaConfig.from_dict(dict(hidden_size=64, num_hidden_layers=1, intermediate_size=8, num_attention_heads=4,
                                   vocab_size=10))
    assert c.num_key_value_heads == 4          # default: heads (models/llm/config.go:100-102)
    assert c.head_dim == 16                    # default: hidden / heads (config.go:103-105)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.max_position_embeddings == 2048
    assert c.eos_token_ids == ()


def test_eos_as_int_or_list_and_rope_parameters_object():
    base = dict(TINY["A"]["cfg"])
    assert config_from_dict({**base, "eos_token_id": 7}).eos_token_ids == (7,)
    assert config_from_dict({**base, "eos_token_id": [7, 9]}).eos_token_ids == (7, 9)
    d = {k: v for k, v in base.items() if k not in ("rope_theta", "rope_scaling")}
    d["rope_parameters"] = dict(rope_type="llama3", rope_theta=123.0, factor=2.0, low_freq_factor=1.0,
                                high_freq_factor=4.0, original_max_position_embeddings=32)
    c = config_from_dict(d)
    assert c.rope_theta == 123.0 and c.rope_scaling.factor == 2.0


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "intermediate_size", "num_attention_heads",
                                 "vocab_size"])
def test_missing_required_key(key):
    d = {k: v for k, v in TINY["A"]["cfg"].items() if k != key}
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("patch,word", [
    (dict(num_key_value_heads=3), "multiple"), (dict(head_dim=15), "even"), (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"), (dict(mlp_bias=True), "mlp_bias"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0, original_max_position_embeddings=8)), "yarn"),
    (dict(vocab_size=0), "positive"), (dict(hidden_size="64"), "integer"), (dict(rms_norm_eps=0.0), "rms_norm_eps"),
])
def test_rejects(patch, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict({**TINY["A"]["cfg"], **patch})


def test_unknown_architecture_lists_the_registered_ones():
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        config_from_dict({**TINY["A"]["cfg"], "architectures": ["NopeForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY["A"]["cfg"].items() if k != "architectures"})
    assert "LlamaForCausalLM" in registered_architectures()


def test_registry_takes_a_new_architecture_and_refuses_a_duplicate():
    class Other:
        @classmethod
        def from_dict(cls, d):
            return cls()
    register_architecture("OtherForCausalLM_test", Other, replace=True)
    assert isinstance(config_from_dict({"architectures": ["OtherForCausalLM_test"]}), Other)
    with pytest.raises(ValueError):
        register_architecture("OtherForCausalLM_test", Other)


def test_round_trip_through_config_json(tmp_path):
    for name in ("A", "B"):
        c = config_from_dict(TINY[name]["cfg"])
        (tmp_path / name).mkdir()
        (tmp_path / name / "config.json").write_text(json.dumps(c.to_dict()))
        assert load_config(str(tmp_path / name)) == c
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path / "missing"))


def test_architecture_spec_carries_every_constant():
    spec = config_from_dict(TINY["B"]["cfg"]).architecture_spec()
    assert isinstance(spec, ArchitectureSpec)
    assert len(spec.layers) == 3 and [e.layer for e in spec.order] == [0, 1, 2]
    m = spec.layers[0].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (3, 1, 32)
    assert abs(m["scale"] - 32 ** -0.5) < 1e-12
    assert spec.layers[0].norms["mixer_norm"].params["eps"] == 1e-6
    assert spec.position_encodings["rope"].params["scaling"]["factor"] == 4.0
    assert spec.head.params["tied_to"] is None
    assert config_from_dict(TINY["A"]["cfg"]).architecture_spec().head.params["tied_to"] == "model.embed_tokens.weight"


def test_run_order_is_validated():
    import dataclasses
    spec = config_from_dict(TINY["A"]["cfg"]).architecture_spec()
    dataclasses.replace(spec, order=[RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_of=1)]).validate()
    with pytest.raises(ValueError, match="layer"):
        dataclasses.replace(spec, order=[RunEntry(5)]).validate()
    with pytest.raises(ValueError, match="before"):
        dataclasses.replace(spec, order=[RunEntry(0, cache_of=1), RunEntry(1)]).validate()
    with pytest.raises(ValueError, match="borrows"):
        dataclasses.replace(spec, order=[RunEntry(0), RunEntry(1, cache_of=0), RunEntry(0, cache_of=1)]).validate()


def test_command_line_writes_and_describes_a_model_folder(tmp_path):
    # the commands that need no GPU: random-model and info (python -m dlgo_b200 ...)
    import json
    from dlgo_b200.__main__ import main
    from tiny_configs import TINY
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY["A"]["cfg"]))
    out = tmp_path / "model"
    assert main(["random-model", "--config", str(cfg_path), "--seed", "3", "--out", str(out)]) == 0
    assert (out / "config.json").exists() and (out / "model.safetensors").exists()
    assert main(["info", str(out)]) == 0
    # generate refuses bad options before it looks for a GPU
    assert main(["generate", str(out), "--max-tokens", "0", "--prompt-ids", "1,2"]) == 2
    assert main(["generate", str(out)]) == 2


def test_rope_pairing_comes_from_the_configuration():
    from dlgo_b200.config import config_from_dict
    from tiny_configs import TINY
    base = dict(TINY["A"]["cfg"])
    assert config_from_dict(base).architecture_spec().position_encodings["rope"].params["pairing"] == "split_half"
    cfg = config_from_dict(dict(base, rope_interleaved=True))
    assert cfg.architecture_spec().position_encodings["rope"].params["pairing"] == "interleaved"
    assert cfg.to_dict()["rope_interleaved"] is True and "rope_interleaved" not in config_from_dict(base).to_dict()
