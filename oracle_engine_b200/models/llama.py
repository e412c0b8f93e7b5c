"""The Llama dense decoder ("LlamaForCausalLM") as data: LlamaConfig -> ModelSpec.

Every layer: RMSNorm -> grouped-query attention with rotary positions -> residual;
RMSNorm -> SwiGLU -> residual; then a final RMSNorm and the (tied or separate) head.
Reference: core/model.cpp:361-492.  Tensor names are those of the model's safetensors
file (the reference's GGUF names `blk.N.attn_q.weight` etc., core/model.cpp:99-112,
map to `model.layers.N.self_attn.q_proj.weight` etc.).
"""
from __future__ import annotations

from dataclasses import asdict

from ..config.base import register_architecture
from ..config.llama import LlamaConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def build_spec(cfg: LlamaConfig, max_positions: int | None = None) -> ModelSpec:
    max_pos = cfg.max_position_embeddings if max_positions is None else min(max_positions, cfg.max_position_embeddings)
    scaling = asdict(cfg.rope_scaling) if cfg.rope_scaling is not None else None
    positions = {"rope": PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                             "scaling": scaling, "max_positions": max_pos})}
    layers = []
    for l in range(cfg.num_hidden_layers):
        layers.append(LayerSpec(
            prefix=f"model.layers.{l}.",
            mixer=PartSpec("gqa_attention", {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
                                             "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                                             "position": "rope", "window": 0}),
            feed_forward=PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                                             "intermediate_size": cfg.intermediate_size}),
            mixer_norm=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                             "name": "input_layernorm.weight"}),
            ffn_norm=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                           "name": "post_attention_layernorm.weight"}),
            block="pre_norm"))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=max_pos,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                               "name": "model.embed_tokens.weight"}),
        final_norm=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                         "name": "model.norm.weight"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                  "tied": cfg.tie_word_embeddings, "name": "lm_head.weight"}),
        positions=positions,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(l) for l in range(cfg.num_hidden_layers)),
        stop_ids=tuple(cfg.eos_token_ids),
        bos_id=cfg.bos_token_id,
        # buffers some exporters store; a tied model's file may repeat the table as lm_head.weight
        ignored_tensors=("rotary_emb.inv_freq",) + (("lm_head.weight",) if cfg.tie_word_embeddings else ()),
    )


register_architecture("LlamaForCausalLM", LlamaConfig, build_spec)
