"""Llama as data: which parts each layer has, with constants taken from a :class:`LlamaConfig`.

Parity: the reference's decoder is pre-norm RMSNorm, rotary grouped-query attention without
biases, a SwiGLU feed-forward, a final RMSNorm and a tied or untied output matrix
(src/llmserve/model/llama.py:57-153); tensor names are the checkpoint's own
(src/llmserve/model/llama.py:1-5).
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .plan import LayerRun, LayerSpec, ModelPlan


def llama_plan(cfg: LlamaConfig) -> ModelPlan:
    rotary = PartSpec(
        "rotary",
        {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "max_positions": cfg.max_position_embeddings},
    )
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}
        layers.append(
            LayerSpec(
                block=PartSpec("pre_norm"),
                mixer_norm=PartSpec("rms_norm", norm, p + "input_layernorm."),
                mixer=PartSpec(
                    "attention",
                    {
                        "hidden_size": cfg.hidden_size,
                        "num_heads": cfg.num_attention_heads,
                        "num_kv_heads": cfg.num_key_value_heads,
                        "head_dim": cfg.head_dim,
                        "scale": cfg.head_dim**-0.5,
                        "window": None,
                        "position": rotary,
                    },
                    p + "self_attn.",
                ),
                ff_norm=PartSpec("rms_norm", norm, p + "post_attention_layernorm."),
                feed_forward=PartSpec(
                    "gated_mlp",
                    {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size, "activation": "silu"},
                    p + "mlp.",
                ),
            )
        )
    return ModelPlan(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding="model.embed_tokens.weight",
        layers=tuple(layers),
        schedule=tuple(LayerRun(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.norm."),
        head=None if cfg.tie_word_embeddings else "lm_head.weight",
        # a tied checkpoint may still store the output matrix; the reference overrides it with the token table
        # (src/llmserve/weights.py:49-52)
        ignored=("lm_head.weight",) if cfg.tie_word_embeddings else (),
    )


register_architecture("LlamaForCausalLM", LlamaConfig, llama_plan)
