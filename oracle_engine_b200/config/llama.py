"""LlamaConfig: the Llama dense decoder's sizes and constants, read from config.json.

Counterpart of the reference's `ModelConfig` (core/model.hpp:10-27) and of the key
reading in `Model::load` (core/model.cpp:48-64).  Differences on purpose: the context is
`max_position_embeddings`, not a fixed 512 (core/model.cpp:64); `rms_norm_eps` is always
handed to the norms (the reference reads it and then uses the default of
core/ops.hpp:43); `rope_scaling` of type llama3 is understood (the reference has no
frequency scaling, core/ops.cpp:461-466).
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

from .base import ConfigError, _Reader


@dataclass(frozen=True)
class RopeScaling:
    """llama3 frequency scaling of the rotary angles."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(raw) -> Optional["RopeScaling"]:
        if raw is None:
            return None
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: `rope_scaling` must be an object or null, got {raw!r}")
        kind = raw.get("rope_type", raw.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported "
                              f"(supported: llama3, default)")
        r = _Reader(raw)
        sc = RopeScaling(
            rope_type="llama3",
            factor=r.number("factor"),
            low_freq_factor=r.number("low_freq_factor"),
            high_freq_factor=r.number("high_freq_factor"),
            original_max_position_embeddings=r.integer("original_max_position_embeddings"),
        )
        if not sc.high_freq_factor > sc.low_freq_factor:
            raise ConfigError("config.json: rope_scaling.high_freq_factor must exceed low_freq_factor")
        return sc


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    bos_token_id: Optional[int]
    eos_token_ids: tuple[int, ...]
    torch_dtype: Optional[str]

    @property
    def group_size(self) -> int:
        """Query heads per KV head (`n_gqa`, core/model.hpp:24)."""
        return self.num_attention_heads // self.num_key_value_heads

    @staticmethod
    def from_dict(raw: dict) -> "LlamaConfig":
        r = _Reader(raw)
        archs = raw.get("architectures") or ["LlamaForCausalLM"]
        # Things this decoder does not have: refuse rather than run wrongly
        # (the reference refuses MoE / SSM / VL models the same way, core/model.cpp:32-46).
        for key in ("num_local_experts", "num_experts", "n_routed_experts"):
            if raw.get(key):
                raise ConfigError(f"config.json: `{key}` is set; routed experts are not part of the "
                                  f"Llama dense decoder")
        for key in ("attention_bias", "mlp_bias"):
            if r.boolean(key, False):
                raise ConfigError(f"config.json: `{key}` = true is not supported (Llama has no biases)")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: `hidden_act` must be \"silu\" (SwiGLU), got {act!r}")
        if raw.get("sliding_window"):
            raise ConfigError("config.json: `sliding_window` is set; the Llama decoder attends to all keys")

        hidden = r.integer("hidden_size")
        heads = r.integer("num_attention_heads")
        kv_heads = r.integer("num_key_value_heads", default=heads, required=False)
        head_dim = r.integer("head_dim", default=None, required=False)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"config.json: hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and `head_dim` is not given")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(f"config.json: num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even (rotary pairs)")
        bos = r.id_list("bos_token_id")
        dtype = raw.get("torch_dtype", raw.get("dtype"))
        return LlamaConfig(
            architecture=archs[0],
            vocab_size=r.integer("vocab_size"),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size"),
            num_hidden_layers=r.integer("num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=r.number("rms_norm_eps"),
            rope_theta=r.number("rope_theta", default=10000.0, required=False),
            rope_scaling=RopeScaling.from_dict(raw.get("rope_scaling")),
            max_position_embeddings=r.integer("max_position_embeddings"),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            bos_token_id=bos[0] if bos else None,
            eos_token_ids=r.id_list("eos_token_id"),
            torch_dtype=dtype if isinstance(dtype, str) else None,
        )

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["model_type"] = "llama"
        d["hidden_act"] = "silu"
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = list(eos) if len(eos) != 1 else eos[0]
        if not eos:
            d["eos_token_id"] = None
        d["attention_bias"] = False
        d["mlp_bias"] = False
        return d
