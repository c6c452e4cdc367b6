"""Qwen3 dense: the architecture entry and its model names.

The decoder as the reference defines it (engine/models/qwen/_archs.py:92-125 with
engine/nn/*): pre-norm blocks of GQA attention with per-head q/k RMSNorm before
rotate-half RoPE, head_dim free of the width, SwiGLU feed-forward, RMSNorm, no biases,
full causal attention (a layer may be given a sliding window through the config), tied
embeddings when the config says so.  Tensor names are the checkpoint's own
(engine/models/qwen/_checkpoint.py:9-24 maps them to the reference's module names).
"""

from __future__ import annotations

from tokensprint_b200.config.model_config import SLIDING_ATTENTION, Qwen3Config
from tokensprint_b200.config.registry import PRESET_DIR, register_architecture, register_preset
from tokensprint_b200.models.spec import ModelSpec
from tokensprint_b200.parts.base import PartSpec

QWEN_ORG = "qwen"


@register_architecture("Qwen3ForCausalLM", model_types=("qwen3",), config_from_dict=Qwen3Config.from_dict)
def build_qwen3_spec(config: Qwen3Config) -> ModelSpec:
    layers = []
    for i, kind in enumerate(config.layer_types):
        p = f"model.layers.{i}."
        position = PartSpec("rotary", {"dim": config.head_dim, "theta": config.rope_theta})
        mixer = PartSpec(
            "attention",
            {
                "hidden_size": config.hidden_size,
                "num_heads": config.num_attention_heads,
                "num_kv_heads": config.num_key_value_heads,
                "head_dim": config.head_dim,
                "qk_norm": True,
                "qk_norm_eps": config.rms_norm_eps,
                "window": config.sliding_window if kind == SLIDING_ATTENTION else 0,
                "position": position,
                "q": p + "self_attn.q_proj.weight",
                "k": p + "self_attn.k_proj.weight",
                "v": p + "self_attn.v_proj.weight",
                "o": p + "self_attn.o_proj.weight",
                "q_norm": p + "self_attn.q_norm.weight",
                "k_norm": p + "self_attn.k_norm.weight",
            },
        )
        feed_forward = PartSpec(
            "swiglu",
            {
                "hidden_size": config.hidden_size,
                "intermediate_size": config.intermediate_size,
                "gate": p + "mlp.gate_proj.weight",
                "up": p + "mlp.up_proj.weight",
                "down": p + "mlp.down_proj.weight",
            },
        )
        norm = {"dim": config.hidden_size, "eps": config.rms_norm_eps}
        layers.append(
            PartSpec(
                "pre_norm",
                {
                    "mixer": mixer,
                    "feed_forward": feed_forward,
                    "mixer_norm": PartSpec("rmsnorm", {**norm, "weight": p + "input_layernorm.weight"}),
                    "ffn_norm": PartSpec("rmsnorm", {**norm, "weight": p + "post_attention_layernorm.weight"}),
                },
            )
        )
    return ModelSpec(
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        embedding="model.embed_tokens.weight",
        layers=layers,
        final_norm=PartSpec("rmsnorm", {"dim": config.hidden_size, "eps": config.rms_norm_eps, "weight": "model.norm.weight"}),
        lm_head=None if config.tie_word_embeddings else "lm_head.weight",
        max_positions=config.max_position_embeddings,
        eos_token_id=config.eos_token_id,
        ignorable_tensors=("lm_head.weight",) if config.tie_word_embeddings else (),
    )


for _path in sorted(PRESET_DIR.glob("qwen3-*.json")):
    register_preset(QWEN_ORG, _path.stem, _path)
