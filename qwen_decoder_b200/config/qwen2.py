"""``Qwen2ForCausalLM``: the Qwen2.5 dense decoder the reference runs, as a ModelSpec.

Structure as in the reference's forward pass (gpu_decoder.cu:311-540,
cpu_decoder.cpp:111-220): embedding; per layer pre-norm -> grouped-query
attention with q/k/v bias and rotary positions -> residual -> pre-norm -> SwiGLU
feed-forward -> residual; final norm; output projection (tied to the embedding
when ``tie_word_embeddings`` is set, which the reference cannot do:
common.cpp:119 requires ``output.weight``).
"""
from __future__ import annotations

from .model_config import Qwen2Config
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def describe_qwen2(cfg: Qwen2Config) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    layers = []
    for i in range(cfg.num_hidden_layers):
        layers.append(LayerSpec(
            prefix=f"model.layers.{i}.",
            block="pre_norm",
            mixer=PartSpec("gq_attention", {
                "hidden_size": cfg.hidden_size,
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "qkv_bias": cfg.attention_bias,
                "out_bias": False,
                "position": "rope",
                "window": None,
                "prefix": "self_attn.",
            }),
            feed_forward=PartSpec("swiglu", {
                "hidden_size": cfg.hidden_size,
                "intermediate_size": cfg.intermediate_size,
                "prefix": "mlp.",
            }),
            norms={
                "input": PartSpec("rmsnorm", dict(norm.params, prefix="input_layernorm.")),
                "post_mixer": PartSpec("rmsnorm", dict(norm.params, prefix="post_attention_layernorm.")),
            },
        ))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding_tensor="model.embed_tokens.weight",
        positions={"rope": PartSpec("rotary", {
            "head_dim": cfg.head_dim,
            "rotary_dim": cfg.head_dim,
            "base": cfg.rope_theta,
            "pairing": cfg.rope_pairing,
        })},
        layers=layers,
        schedule=[ScheduleEntry(layer=i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", dict(norm.params, prefix="")),
        final_norm_prefix="model.norm.",
        lm_head_tensor=None if cfg.tie_word_embeddings else "lm_head.weight",
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, describe_qwen2)
