"""Qwen3 dense: its typed configuration, the architecture entry and its model names.

The decoder as the reference defines it (engine/models/qwen/_archs.py:92-125 with
engine/nn/*): pre-norm blocks of GQA attention with per-head q/k RMSNorm before
rotate-half RoPE, head_dim free of the width, SwiGLU feed-forward, RMSNorm, no biases,
full causal attention (a layer may be given a sliding window through the config), tied
embeddings when the config says so.  Tensor names are the checkpoint's own
(engine/models/qwen/_checkpoint.py:9-24 maps them to the reference's module names).

config.json key    <-> reference field (engine/models/qwen/_archs.py:92-125, engine/models/_registry.py:12-40)
vocab_size         ModelConfig.vocab_dim
hidden_size        AttentionConfig.model_dim / FFNConfig.model_dim
num_hidden_layers  ModelConfig.num_layers
num_attention_heads / num_key_value_heads / head_dim   AttentionConfig.*
intermediate_size  FFNConfig.inner_dim
rope_theta, rms_norm_eps, tie_word_embeddings, max_position_embeddings
                   ModelConfig.rope_theta / norm_eps (and qk_norm_eps) / tie_weights / max_seq_len
sliding_window (+ use_sliding_window, max_window_layers, layer_types)
                   ModelConfig.attn_window_len (engine/models/_registry.py:20; unused there)
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

from tokensprint_b200.config.model_config import ConfigError, read_config_json, require, write_config_json
from tokensprint_b200.config.registry import PRESET_DIR, register_architecture, register_preset
from tokensprint_b200.models.spec import ModelSpec
from tokensprint_b200.parts.base import PartSpec

QWEN_ORG = "qwen"
FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config:
    """All sizes and constants of one Qwen3 dense model."""

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float = 1_000_000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 40960
    # One entry per layer: FULL_ATTENTION or SLIDING_ATTENTION.
    layer_types: tuple[str, ...] = ()
    # Number of keys (the query's own included) that a sliding layer sees.
    sliding_window: int | None = None
    eos_token_id: int = -1
    torch_dtype: str = "bfloat16"
    architectures: tuple[str, ...] = ("Qwen3ForCausalLM",)
    model_type: str = "qwen3"
    extra: dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def __post_init__(self) -> None:
        positive = (
            "vocab_size",
            "hidden_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
            "intermediate_size",
            "max_position_embeddings",
        )
        for key in positive:
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                "config.json: 'num_attention_heads' must be a multiple of 'num_key_value_heads', "
                f"got {self.num_attention_heads} and {self.num_key_value_heads}"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: 'head_dim' must be even for rotary pairs, got {self.head_dim}")
        if self.rope_theta <= 0 or self.rms_norm_eps <= 0:
            raise ConfigError("config.json: 'rope_theta' and 'rms_norm_eps' must be positive")
        if not self.layer_types:
            object.__setattr__(self, "layer_types", (FULL_ATTENTION,) * self.num_hidden_layers)
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError(
                f"config.json: 'layer_types' has {len(self.layer_types)} entries for "
                f"{self.num_hidden_layers} layers"
            )
        for kind in self.layer_types:
            if kind not in (FULL_ATTENTION, SLIDING_ATTENTION):
                raise ConfigError(f"config.json: unknown entry {kind!r} in 'layer_types'")
        if SLIDING_ATTENTION in self.layer_types:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("config.json: sliding layers need a positive 'sliding_window'")

    @property
    def kv_group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "Qwen3Config":
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' must be 'silu' for Qwen3, got {act!r}")
        if d.get("attention_bias", False):
            raise ConfigError("config.json: 'attention_bias' must be false for Qwen3 (no biases)")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: 'rope_scaling' is not supported (Qwen3 presets use none)")
        if d.get("attention_dropout", 0.0) not in (0, 0.0):
            raise ConfigError("config.json: 'attention_dropout' must be 0 for inference")

        hidden = require(d, "hidden_size", int)
        heads = require(d, "num_attention_heads", int)
        layers = require(d, "num_hidden_layers", int)
        kv_heads = d.get("num_key_value_heads")
        kv_heads = heads if kv_heads is None else require(d, "num_key_value_heads", int)
        head_dim = d.get("head_dim")
        if head_dim is None:
            # engine/models/_builder.py:37-39: head_dim falls back to model_dim // num_heads
            if hidden % heads != 0:
                raise ConfigError(
                    "config.json: 'head_dim' is absent and 'hidden_size' is no multiple of "
                    "'num_attention_heads'"
                )
            head_dim = hidden // heads
        else:
            head_dim = require(d, "head_dim", int)

        window = d.get("sliding_window")
        layer_types = d.get("layer_types")
        if layer_types is not None:
            layer_types = tuple(str(t) for t in layer_types)
        elif d.get("use_sliding_window", False) and window:
            first_sliding = int(d.get("max_window_layers", layers))
            layer_types = tuple(
                SLIDING_ATTENTION if i >= first_sliding else FULL_ATTENTION for i in range(layers)
            )
        else:
            layer_types = (FULL_ATTENTION,) * layers
        if SLIDING_ATTENTION not in layer_types:
            window = None

        eos = d.get("eos_token_id", -1)
        if isinstance(eos, (list, tuple)):
            eos = eos[0] if eos else -1
        if eos is None:
            eos = -1

        known = {
            "vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "intermediate_size", "rope_theta", "rms_norm_eps",
            "tie_word_embeddings", "max_position_embeddings", "sliding_window", "use_sliding_window",
            "max_window_layers", "layer_types", "eos_token_id", "torch_dtype", "dtype",
            "architectures", "model_type", "hidden_act", "attention_bias", "rope_scaling",
            "attention_dropout",
        }
        extra = {k: v for k, v in d.items() if k not in known}
        return cls(
            vocab_size=require(d, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=require(d, "intermediate_size", int),
            rope_theta=float(d.get("rope_theta", 1_000_000.0)),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=int(d.get("max_position_embeddings", 40960)),
            layer_types=layer_types,
            sliding_window=None if window is None else int(window),
            eos_token_id=int(eos),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            architectures=tuple(d.get("architectures", ("Qwen3ForCausalLM",))),
            model_type=str(d.get("model_type", "qwen3")),
            extra=extra,
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "Qwen3Config":
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        d.pop("extra")
        d["architectures"] = list(self.architectures)
        d["layer_types"] = list(self.layer_types)
        d["use_sliding_window"] = SLIDING_ATTENTION in self.layer_types
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        return d

    def save(self, folder: str | Path) -> None:
        write_config_json(folder, self.to_dict())



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
