"""Qwen3 dense (``Qwen3ForCausalLM``) as a :class:`ModelSpec`.

Every layer is a pre-norm block of grouped-query attention (per-head q/k RMSNorm, rotary
positions, no biases) and a SwiGLU feed-forward; RMSNorm everywhere with one eps; the head
is the embedding table when ``tie_word_embeddings``.  Structure and checkpoint names as in
raun6k/Pylon (src/pylon/model/model.py:18-35, src/pylon/model/layers.py:81-200,
src/pylon/model/weights.py:51-83).
"""
from __future__ import annotations

from typing import Optional

from pylon_b200.config.model_config import Qwen3Config
from pylon_b200.parts.spec import LayerSpec, ModelSpec, PartSpec


def qwen3_spec(config: Qwen3Config, max_positions: Optional[int] = None) -> ModelSpec:
    positions = config.max_position_embeddings if max_positions is None else min(max_positions, config.max_position_embeddings)
    norm = PartSpec("rmsnorm", {"width": config.hidden_size, "eps": config.rms_norm_eps})
    mixer = PartSpec(
        "gqa_attention",
        {
            "width": config.hidden_size,
            "n_heads": config.num_attention_heads,
            "n_kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim,
            "qk_norm_eps": config.rms_norm_eps,
            "position": PartSpec("rope", {"head_dim": config.head_dim, "theta": config.rope_theta, "max_positions": positions}),
        },
    )
    feed_forward = PartSpec("swiglu", {"width": config.hidden_size, "intermediate": config.intermediate_size})
    block = PartSpec("prenorm", {"mixer": mixer, "feed_forward": feed_forward, "mixer_norm": norm, "ffn_norm": norm})
    layers = tuple(LayerSpec(f"model.layers.{i}.", block) for i in range(config.num_hidden_layers))
    return ModelSpec(
        width=config.hidden_size,
        vocab_size=config.vocab_size,
        max_positions=positions,
        embedding_name="model.embed_tokens.weight",
        lm_head_name=None if config.tie_word_embeddings else "lm_head.weight",
        final_norm=norm,
        final_norm_prefix="model.norm.",
        layers=layers,
        order=tuple(range(config.num_hidden_layers)),
        eos_token_ids=config.eos_token_ids,
        ignored_tensors=("lm_head.weight",) if config.tie_word_embeddings else (),
    )
