"""Qwen3 dense as a model specification.

Reference: models/qwen3.py:9-84 (embedding, N decoder layers, final norm, head tied or not),
models/transformer_block.py:7-52 (pre-norm block), models/self_attn.py:81-104 (head norm on),
factory/config.py:107-130 (which config.json keys feed which constant).  Tensor names are the
checkpoint's: ``model.embed_tokens.weight``, ``model.layers.{i}.input_layernorm.weight``,
``...self_attn.{q,k,v,o}_proj.weight``, ``...self_attn.{q,k}_norm.weight``,
``...post_attention_layernorm.weight``, ``...mlp.{gate,up,down}_proj.weight``,
``model.norm.weight``, ``lm_head.weight`` (only when the head is not tied).
"""

from __future__ import annotations

from ..config.model_config import SLIDING_ATTENTION, Qwen3Config
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..registry import register_architecture

_BLOCK_NAMES = {"norm1": "input_layernorm", "mixer": "self_attn",
                "norm2": "post_attention_layernorm", "feed_forward": "mlp"}


@register_architecture("Qwen3ForCausalLM", Qwen3Config)
def qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    norm = PartSpec("rms_norm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    rotary = PartSpec("rotary_neox", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                      "max_positions": cfg.max_position_embeddings})
    feed_forward = PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                                       "intermediate_size": cfg.intermediate_size})
    layers = []
    for i, layer_type in enumerate(cfg.layer_types):
        mixer = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "qk_norm_eps": cfg.rms_norm_eps, "position": rotary,
            "window": cfg.sliding_window if layer_type == SLIDING_ATTENTION else None})
        block = PartSpec("pre_norm", {"norm1": norm, "mixer": mixer, "norm2": norm,
                                      "feed_forward": feed_forward, "names": _BLOCK_NAMES})
        layers.append((f"model.layers.{i}", block))
    embedding_name = "model.embed_tokens"
    head = PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                "tied_to": f"{embedding_name}.weight" if cfg.tie_word_embeddings else None})
    return ModelSpec(
        embedding=(embedding_name, PartSpec("token_embedding", {"vocab_size": cfg.vocab_size,
                                                                "hidden_size": cfg.hidden_size})),
        layers=layers,
        order=[LayerCall(layer=i, cache=i) for i in range(cfg.num_hidden_layers)],
        final_norm=("model.norm", norm),
        head=("lm_head", head),
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        # a tied checkpoint may still carry a copy of the head; it is not read
        ignorable_weights=("lm_head.weight",) if cfg.tie_word_embeddings else (),
        eos_token_id=cfg.eos_token_id,
    )
