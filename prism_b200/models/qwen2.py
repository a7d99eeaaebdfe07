"""Qwen2 / Qwen2.5 dense decoder as a layer plan.

What andre-fu/prism's executor computes (engine/executor.py:106-130) and
which tensors it reads (engine/weight_pool.py:156-199), written as data:
per layer a pre-norm block of RMSNorm, grouped-query attention with q/k/v
bias and rotary positions, RMSNorm, SwiGLU; then a final RMSNorm and a linear
head that shares the embedding when ``tie_word_embeddings`` is set.
"""

from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..parts.base import PartSpec
from .decoder import ModelSpec


def qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    H = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec("gqa_attention", dict(
            hidden_size=H, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, qkv_bias=cfg.attention_bias, o_bias=False,
            window=cfg.layer_window(i),
            position=PartSpec("rotary", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta))),
            prefix=p + "self_attn.")
        ff = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=cfg.intermediate_size), prefix=p + "mlp.")
        layers.append(PartSpec("prenorm", dict(
            mixer=mixer, feed_forward=ff,
            mixer_norm=PartSpec("rmsnorm", dict(width=H, eps=cfg.rms_norm_eps), prefix=p + "input_layernorm."),
            ff_norm=PartSpec("rmsnorm", dict(width=H, eps=cfg.rms_norm_eps), prefix=p + "post_attention_layernorm."))))
    return ModelSpec(
        architecture="Qwen2ForCausalLM", hidden_size=H, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token", dict(vocab_size=cfg.vocab_size, hidden_size=H), prefix="model."),
        layers=layers,
        final_norm=PartSpec("rmsnorm", dict(width=H, eps=cfg.rms_norm_eps), prefix="model.norm."),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab_size, hidden_size=H,
                                     tied_to="embedding.weight" if cfg.tie_word_embeddings else None),
                      prefix="lm_head."),
        eos_token_id=cfg.eos_token_id)
