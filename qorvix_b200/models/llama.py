"""The Llama dense decoder as data: LlamaConfig -> ModelSpec.

Layer order, tensor roles and formulas are the reference's CPU model
(runtime/src/text_model.cpp:133-176; tensor roles runtime/src/weights.cpp:27-47); tensor
names are the ones a config.json + safetensors checkpoint of this architecture uses.
Every layer is attention + SwiGLU in the pre-norm arrangement; the head is the embedding
table when tie_word_embeddings is set (reference: weights.hpp:119 falls back the same way).
"""
from __future__ import annotations

import math

from ..config import LlamaConfig, register_architecture
from ..parts.spec import AttentionSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec, SwiGLUSpec


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    rotary = RotarySpec(head_dim=cfg.head_dim, rotary_dim=cfg.head_dim, theta=cfg.rope_theta,
                        scaling=cfg.rope_scaling)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            mixer_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, p + "input_layernorm.weight"),
            mixer=AttentionSpec(
                hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                scale=1.0 / math.sqrt(cfg.head_dim),
                q_proj=p + "self_attn.q_proj.weight", k_proj=p + "self_attn.k_proj.weight",
                v_proj=p + "self_attn.v_proj.weight", o_proj=p + "self_attn.o_proj.weight",
                position=rotary),
            ffn_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, p + "post_attention_layernorm.weight"),
            feed_forward=SwiGLUSpec(cfg.hidden_size, cfg.intermediate_size, p + "mlp.gate_proj.weight",
                                    p + "mlp.up_proj.weight", p + "mlp.down_proj.weight"),
            block="pre_norm"))
    tied = cfg.tie_word_embeddings
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        embedding="model.embed_tokens.weight", layers=layers,
        final_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, "model.norm.weight"),
        lm_head=None if tied else "lm_head.weight",
        optional_tensors=("lm_head.weight",) if tied else (),
        # older checkpoints of this architecture store each layer's rotary frequencies as a buffer
        ignored_tensors=("model.layers.*.self_attn.rotary_emb.inv_freq",),
        max_position=cfg.max_position_embeddings)


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_spec)
