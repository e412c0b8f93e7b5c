"""Configuration: reading config.json keys, defaults, refusals, and the registry."""
import json

import pytest

from conftest import TINY_A, TINY_B
from oracle_engine_b200 import ConfigError, LlamaConfig, load_config
from oracle_engine_b200.config.base import ARCHITECTURES, get_architecture


def test_reads_every_key():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (384, 192, 512, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.group_size) == (6, 2, 32, 3)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0 and c.max_position_embeddings == 512
    assert c.rope_scaling.factor == 4.0 and c.rope_scaling.original_max_position_embeddings == 64
    assert not c.tie_word_embeddings and c.eos_token_ids == (7, 9) and c.bos_token_id == 5


def test_defaults_are_derived_not_constant():
    raw = dict(TINY_A)
    raw.pop("num_key_value_heads")
    raw.pop("rope_theta")
    c = LlamaConfig.from_dict(raw)
    assert c.num_key_value_heads == c.num_attention_heads == 4
    assert c.head_dim == 64 // 4 and c.rope_theta == 10000.0 and c.rope_scaling is None
    assert c.eos_token_ids == (2,)


def test_round_trip(tmp_path):
    c = LlamaConfig.from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    c2, arch = load_config(tmp_path)
    assert c2 == c and arch.name == "LlamaForCausalLM"


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "rms_norm_eps", "max_position_embeddings"])
def test_missing_required_key(key):
    raw = dict(TINY_A)
    raw.pop(key)
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(raw)


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_size": 66, "num_attention_heads": 4}, "head_dim"),
    ({"head_dim": 15}, "even"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_local_experts": 8}, "experts"),
    ({"sliding_window": 128}, "sliding_window"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"eos_token_id": "x"}, "eos_token_id"),
])
def test_refusals(patch, word):
    raw = dict(TINY_A)
    raw.update(patch)
    if patch.get("hidden_size") == 66:
        raw.pop("head_dim", None)
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(raw)


def test_registry(tmp_path):
    assert "LlamaForCausalLM" in ARCHITECTURES
    with pytest.raises(ConfigError, match="registered: .*LlamaForCausalLM"):
        get_architecture("MambaForCausalLM")
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["Nope"]}))
    with pytest.raises(ConfigError, match="Nope"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(tmp_path)
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(tmp_path / "missing")


def test_spec_is_data():
    """The order of layers is a list; the Llama spec names each layer once, in order."""
    c = LlamaConfig.from_dict(TINY_B)
    spec = get_architecture(c.architecture).build_spec(c)
    assert [e.layer for e in spec.schedule] == [0, 1, 2] and all(e.cache_from is None for e in spec.schedule)
    assert spec.layers[1].mixer.kind == "gqa_attention" and spec.layers[1].feed_forward.kind == "swiglu"
    assert spec.layers[2].mixer.params["head_dim"] == 32 and spec.final_norm.params["eps"] == 1e-6
    capped = get_architecture(c.architecture).build_spec(c, 100)
    assert capped.max_positions == 100
