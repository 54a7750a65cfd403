"""Safetensors reading and writing, weight errors, random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from dlgo_b200.config import config_from_dict
from dlgo_b200.engine.model import CausalLM
from dlgo_b200.weights import (Checkpoint, SafetensorsError, WeightError, WeightSource, check_against, save_tensors,
                               stored_precision, write_random_model)
from tiny_configs import TINY, write_tiny


def test_round_trip_and_agreement_with_the_safetensors_library(tmp_path):
    import safetensors.torch as st
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).view(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    (tmp_path / "m").mkdir()
    p = str(tmp_path / "m" / "model.safetensors")
    save_tensors(p, t)
    ours = Checkpoint(str(tmp_path / "m"))
    theirs = st.load_file(p)
    assert ours.names() == sorted(t)
    for k in t:
        assert torch.equal(ours.read(k), t[k]) and torch.equal(theirs[k], t[k])
    # and the other way round: a file their library wrote
    (tmp_path / "n").mkdir()
    st.save_file(t, str(tmp_path / "n" / "model.safetensors"))
    back = Checkpoint(str(tmp_path / "n"))
    for k in t:
        assert torch.equal(back.read(k), t[k])


def test_sharded_folder_through_its_index(tmp_path):
    save_tensors(str(tmp_path / "s1.safetensors"), {"x": torch.ones(2)})
    save_tensors(str(tmp_path / "s2.safetensors"), {"y": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    ck = Checkpoint(str(tmp_path))
    assert ck.names() == ["x", "y"] and ck.read("y").shape == (3,)


def test_broken_files(tmp_path):
    with pytest.raises(SafetensorsError, match="neither"):
        Checkpoint(str(tmp_path))
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="truncated"):
        Checkpoint(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="JSON"):
        Checkpoint(str(tmp_path))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="truncated"):
        Checkpoint(str(tmp_path))
    hdr = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="dtype"):
        Checkpoint(str(tmp_path))


def test_precision_rule():
    assert stored_precision(torch.zeros(2, dtype=torch.bfloat16)).dtype == torch.bfloat16
    assert stored_precision(torch.zeros(2, dtype=torch.float16)).dtype == torch.bfloat16
    assert stored_precision(torch.zeros(2, dtype=torch.float32)).dtype == torch.float32   # 32-bit stays 32-bit
    assert stored_precision(torch.zeros(2, dtype=torch.int64)).dtype == torch.int32       # integer tables
    assert stored_precision(torch.zeros(2, dtype=torch.uint8)).dtype == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_tiny("A", str(tmp_path / "A"))
    model = CausalLM(config_from_dict(TINY["A"]["cfg"]).architecture_spec())
    expected = {n: ps.shape for n, ps in model.expected_tensors().items()}
    ck = Checkpoint(d)
    tensors = {n: ck.read(n).clone() for n in ck.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["lm_head.weight"] = torch.zeros(256, 64)          # tied model: a head of its own is unexpected
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64)
    bad = tmp_path / "bad"
    bad.mkdir()
    save_tensors(str(bad / "model.safetensors"), tensors)
    src = WeightSource(str(bad), torch.device("cpu"))
    with pytest.raises(WeightError) as ei:
        check_against(expected, src.found())
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (64, 64), (32, 64))]
    msg = str(e)
    for word in ("missing (2)", "unexpected (2)", "wrong shape (1)", "expected [32, 64]", "model.norm.weight"):
        assert word in msg


def test_expected_tensors_of_tied_and_untied_models():
    a = CausalLM(config_from_dict(TINY["A"]["cfg"]).architecture_spec()).expected_tensors()
    b = CausalLM(config_from_dict(TINY["B"]["cfg"]).architecture_spec()).expected_tensors()
    assert "lm_head.weight" not in a and b["lm_head.weight"].shape == (384, 96)
    assert a["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert b["model.layers.2.mlp.down_proj.weight"].shape == (96, 256)
    assert len(a) == 1 + 2 * 9 + 1 and len(b) == 1 + 3 * 9 + 2


def test_random_model_is_a_function_of_config_and_seed(tmp_path):
    d1 = write_tiny("B", str(tmp_path / "b1"))
    d2 = write_tiny("B", str(tmp_path / "b2"))
    cfg = config_from_dict(TINY["B"]["cfg"])
    d3 = write_random_model(cfg, 99, str(tmp_path / "b3"))
    c1, c2, c3 = Checkpoint(d1), Checkpoint(d2), Checkpoint(d3)
    assert c1.names() == c2.names() == c3.names()
    for n in c1.names():
        assert torch.equal(c1.read(n), c2.read(n))
    assert not torch.equal(c1.read("lm_head.weight"), c3.read("lm_head.weight"))
    w = c1.read("model.layers.0.mlp.gate_proj.weight").float()
    nw = c1.read("model.norm.weight").float()
    assert w.dtype == torch.float32 and abs(float(w.std()) - 0.02) < 2e-3 and abs(float(w.mean())) < 2e-3
    assert abs(float(nw.mean()) - 1.0) < 2e-2
    assert json.load(open(os.path.join(d1, "config.json")))["rope_scaling"]["factor"] == 4.0
    d4 = write_random_model(cfg, 1, str(tmp_path / "b4"), dtype=torch.float32)
    assert Checkpoint(d4).info("model.norm.weight").dtype == torch.float32
