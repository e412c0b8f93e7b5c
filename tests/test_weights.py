"""Weights: safetensors round trip, kept precisions, the one error for everything wrong,
file damage, shards, and seeded random weights."""
import json
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B
from oracle_engine_b200 import LlamaConfig, WeightError, write_model_folder
from oracle_engine_b200.config.base import get_architecture
from oracle_engine_b200.engine.runtime import Runtime
from oracle_engine_b200.parts.model import DecoderModel
from oracle_engine_b200.weights.loader import check_tensors, load_weights
from oracle_engine_b200.weights.random_init import RandomSource, normal_tensor
from oracle_engine_b200.weights.safetensors_io import ModelFiles, SafetensorsFile, kept_dtype, write_safetensors


def _model(raw):
    cfg = LlamaConfig.from_dict(raw)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    return cfg, DecoderModel(spec, Runtime(torch.float32, torch.device("cpu")))


def test_round_trip_and_kept_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int64),
         "d": torch.randn(2, 2).to(torch.float16), "e": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", t, metadata={"k": 1})
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert set(f.names()) == set(t) and f.metadata == {"k": "1"}
    for n, want in t.items():
        got = f.read(n)
        assert got.dtype == want.dtype and got.shape == want.shape and torch.equal(got, want)
    assert kept_dtype(torch.bfloat16) == torch.bfloat16 and kept_dtype(torch.float16) == torch.bfloat16
    assert kept_dtype(torch.float32) == torch.float32 and kept_dtype(torch.int64) == torch.int32
    # our own reader against the plain implementation's reader
    import plain_llama
    p = plain_llama.read_safetensors(tmp_path / "x.safetensors")
    assert torch.equal(p["a"], t["a"].double()) and torch.equal(p["c"], t["c"])


def test_one_error_lists_everything(tmp_path):
    cfg, model = _model(TINY_B)
    write_model_folder(tmp_path, cfg, seed=3)
    files = ModelFiles(tmp_path)
    tensors = {n: files.read(n).clone() for n in files.names()}
    files.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 190, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.zeros(2)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)      # ignorable buffer
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_weights(model, ModelFiles(tmp_path))
    msg = str(e.value)
    assert "2 missing" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "1 unexpected" in msg and "model.layers.7.extra.weight" in msg and "inv_freq" not in msg
    assert "1 wrong shape" in msg and "[64, 190]" in msg and "[64, 192]" in msg


def test_tied_and_untied_head(tmp_path):
    cfg, model = _model(TINY_A)                       # tied: no lm_head.weight is read
    names = {d.name for d in model.tensors()}
    assert "lm_head.weight" not in names and "model.embed_tokens.weight" in names
    cfg_b, model_b = _model(TINY_B)
    assert "lm_head.weight" in {d.name for d in model_b.tensors()}
    avail = {d.name: (torch.bfloat16, d.shape) for d in model.tensors()}
    avail["lm_head.weight"] = (torch.bfloat16, (256, 64))
    check_tensors(avail, model.tensors(), model.spec.ignored_tensors)       # tolerated when tied
    avail_b = {d.name: (torch.bfloat16, d.shape) for d in model_b.tensors() if d.name != "lm_head.weight"}
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_tensors(avail_b, model_b.tensors(), model_b.spec.ignored_tensors)


def test_damaged_files(tmp_path):
    cfg, _ = _model(TINY_A)
    write_model_folder(tmp_path, cfg, seed=0)
    raw = (tmp_path / "model.safetensors").read_bytes()
    (tmp_path / "cut.safetensors").write_bytes(raw[:len(raw) - 100])
    with pytest.raises(WeightError, match="outside the file"):
        SafetensorsFile(tmp_path / "cut.safetensors")
    (tmp_path / "short.safetensors").write_bytes(raw[:5])
    with pytest.raises(WeightError, match="truncated"):
        SafetensorsFile(tmp_path / "short.safetensors")
    (tmp_path / "hdr.safetensors").write_bytes(struct.pack("<Q", 10 ** 9) + raw[8:])
    with pytest.raises(WeightError, match="truncated header"):
        SafetensorsFile(tmp_path / "hdr.safetensors")
    (tmp_path / "json.safetensors").write_bytes(struct.pack("<Q", 4) + b"{{{{" + raw[12:])
    with pytest.raises(WeightError, match="JSON"):
        SafetensorsFile(tmp_path / "json.safetensors")
    with pytest.raises(WeightError, match="neither"):
        ModelFiles(tmp_path / "nothing")


def test_shards(tmp_path):
    cfg, model = _model(TINY_A)
    write_model_folder(tmp_path / "one", cfg, seed=0)
    files = ModelFiles(tmp_path / "one")
    names = sorted(files.names())
    d = tmp_path / "two"
    d.mkdir()
    half = len(names) // 2
    write_safetensors(d / "s1.safetensors", {n: files.read(n) for n in names[:half]})
    write_safetensors(d / "s2.safetensors", {n: files.read(n) for n in names[half:]})
    wm = {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    sharded = ModelFiles(d)
    assert sorted(sharded.names()) == names
    assert all(torch.equal(sharded.read(n), files.read(n)) for n in names)
    wm[names[0]] = "s2.safetensors"
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    with pytest.raises(WeightError, match=names[0]):
        ModelFiles(d)


def test_random_weights_are_a_function_of_seed_and_name(tmp_path):
    a = normal_tensor(3, "w", (64, 33), 0.0, 0.02, torch.bfloat16, "cpu")
    b = normal_tensor(3, "w", (64, 33), 0.0, 0.02, torch.bfloat16, "cpu")
    c = normal_tensor(4, "w", (64, 33), 0.0, 0.02, torch.bfloat16, "cpu")
    d = normal_tensor(3, "v", (64, 33), 0.0, 0.02, torch.bfloat16, "cpu")
    assert torch.equal(a, b) and not torch.equal(a, c) and not torch.equal(a, d)
    big = normal_tensor(1, "n", (200000,), 0.0, 1.0, torch.float32, "cpu")
    assert abs(big.mean()) < 0.01 and abs(big.std() - 1) < 0.01
    cfg, model = _model(TINY_B)
    write_model_folder(tmp_path, cfg, seed=9)
    files = ModelFiles(tmp_path)
    src = RandomSource(model.tensors(), 9)
    for n in files.names():
        assert torch.equal(files.read(n), src.read(n))
    norm = files.read("model.norm.weight").float()
    assert abs(norm.mean() - 1) < 0.05 and 0.05 < norm.std() < 0.15
    w = files.read("model.layers.2.mlp.down_proj.weight").float()
    assert abs(w.std() - 0.02) < 0.002
    assert json.loads((tmp_path / "config.json").read_text())["architectures"] == ["LlamaForCausalLM"]
