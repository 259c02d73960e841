"""``LlamaForCausalLM``: a decoder of identical pre-norm layers, each grouped-query
attention with rotary positions and a SwiGLU feed-forward, RMS norms, an untied or tied
output head (reference ``models/llama/llama.py:98-172``).

This file is the only place that knows the architecture: it turns a ``LlamaConfig`` into
a ``ModelSpec`` of generic parts and names the checkpoint tensors
(``model.embed_tokens.weight``, ``model.layers.{i}.self_attn.q_proj.weight`` ...,
``model.norm.weight``, ``lm_head.weight``).
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def assemble(cfg: LlamaConfig) -> ModelSpec:
    H = cfg.hidden_size
    scaling = None
    if cfg.rope_scaling is not None:
        s = cfg.rope_scaling
        scaling = {
            "factor": s.factor,
            "low_freq_factor": s.low_freq_factor,
            "high_freq_factor": s.high_freq_factor,
            "original_max_position_embeddings": s.original_max_position_embeddings,
        }
    position = PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": scaling})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(
            LayerSpec(
                mixer=PartSpec(
                    "gqa_attention",
                    {
                        "hidden_size": H,
                        "num_heads": cfg.num_attention_heads,
                        "num_kv_heads": cfg.num_key_value_heads,
                        "head_dim": cfg.head_dim,
                    },
                    prefix=p + "self_attn.",
                ),
                feed_forward=PartSpec(
                    "swiglu",
                    {"hidden_size": H, "intermediate_size": cfg.intermediate_size},
                    prefix=p + "mlp.",
                ),
                mixer_norm=PartSpec("rmsnorm", {"hidden_size": H, "eps": cfg.rms_norm_eps},
                                    prefix=p + "input_layernorm."),
                feed_forward_norm=PartSpec("rmsnorm", {"hidden_size": H, "eps": cfg.rms_norm_eps},
                                           prefix=p + "post_attention_layernorm."),
                position=position,
                arrangement="prenorm",
            )
        )
    return ModelSpec(
        hidden_size=H,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H},
                           prefix="model.embed_tokens."),
        layers=tuple(layers),
        final_norm=PartSpec("rmsnorm", {"hidden_size": H, "eps": cfg.rms_norm_eps}, prefix="model.norm."),
        head=PartSpec("linear_head",
                      {"vocab_size": cfg.vocab_size, "hidden_size": H, "tied": cfg.tie_word_embeddings},
                      prefix="lm_head."),
        max_positions=cfg.max_position_embeddings,
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_json, assemble, replace=True)
