"""The tests' own tiny Qwen3 configurations and random weights (no product code here).

The configurations differ in every size and option: head counts and groups, head_dim
against the width, sizes that are no power of two, number of layers, vocabulary, the
norms' eps, rope_theta, tied or untied head, and (TINY_C) sliding-window layers.
Weights are drawn here, by the tests' own generator (plain integer hashing, the same values
under every torch version), under the checkpoint's tensor names
(engine/models/qwen/_checkpoint.py:9-24 of the reference lists them).
"""

from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Optional

import torch

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 128,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "max_position_embeddings": 128,
    "hidden_act": "silu",
    "attention_bias": False,
    "torch_dtype": "float32",
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 6,
    "num_key_value_heads": 3,
    "head_dim": 32,
    "intermediate_size": 224,
    "vocab_size": 512,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 256,
    "hidden_act": "silu",
    "attention_bias": False,
    "torch_dtype": "float32",
}

# Sliding-window layers beside full ones, one KV head for all queries, odd sizes.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 4,
    "hidden_size": 80,
    "num_attention_heads": 5,
    "num_key_value_heads": 1,
    "head_dim": 48,
    "intermediate_size": 136,
    "vocab_size": 301,
    "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False,
    "max_position_embeddings": 512,
    "use_sliding_window": True,
    "sliding_window": 24,
    "layer_types": ["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
    "hidden_act": "silu",
    "attention_bias": False,
    "torch_dtype": "float32",
}

TINY = {"a": TINY_A, "b": TINY_B, "c": TINY_C}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    H, d = cfg["hidden_size"], cfg["head_dim"]
    nq, nkv, I, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    shapes: dict[str, tuple[int, ...]] = {"model.embed_tokens.weight": (V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes[p + "input_layernorm.weight"] = (H,)
        shapes[p + "self_attn.q_proj.weight"] = (nq * d, H)
        shapes[p + "self_attn.k_proj.weight"] = (nkv * d, H)
        shapes[p + "self_attn.v_proj.weight"] = (nkv * d, H)
        shapes[p + "self_attn.o_proj.weight"] = (H, nq * d)
        shapes[p + "self_attn.q_norm.weight"] = (d,)
        shapes[p + "self_attn.k_norm.weight"] = (d,)
        shapes[p + "post_attention_layernorm.weight"] = (H,)
        shapes[p + "mlp.gate_proj.weight"] = (I, H)
        shapes[p + "mlp.up_proj.weight"] = (I, H)
        shapes[p + "mlp.down_proj.weight"] = (H, I)
    shapes["model.norm.weight"] = (H,)
    if not cfg["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (V, H)
    return shapes


def seeded_normal(shape: tuple[int, ...], key: str) -> torch.Tensor:
    """Float32 values of about unit variance that depend on `key` and nothing else: not on the
    torch or numpy version, the platform or the device.  Element i is the sum of twelve uniform
    numbers (21-bit pieces of four splitmix64 hashes of (key, i)) minus six; every step is integer
    arithmetic or exact in float64, so stored results made from these weights stay valid."""
    import numpy as np

    n = 1
    for s in shape:
        n *= int(s)
    base = np.uint64(int.from_bytes(hashlib.sha256(key.encode()).digest()[:8], "little"))
    total = np.zeros(n, dtype=np.uint64)
    index = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        for draw in range(4):
            z = base + (index * np.uint64(4) + np.uint64(draw + 1)) * np.uint64(0x9E3779B97F4A7C15)
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            z = z ^ (z >> np.uint64(31))
            for piece in range(3):
                total += (z >> np.uint64(21 * piece)) & np.uint64((1 << 21) - 1)
    values = (total.astype(np.float64) + 6.0) / float(1 << 21) - 6.0
    return torch.from_numpy(values.astype(np.float32)).reshape(shape)


def tiny_weights(cfg: dict, seed: int, *, std: float = 0.02, norm_std: float = 0.05, sharp: float = 1.0) -> dict[str, torch.Tensor]:
    """Float32 weights: matrices N(0, std), norm weights 1 + N(0, norm_std).

    `sharp` multiplies the q/k norm weights: scores then spread over a wide range, the
    softmax picks few keys, and a fault at any single key (a page's edge, a far key, the
    window's edge) moves the logits far more than rounding does.
    """
    out: dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg).items():
        x = seeded_normal(shape, f"tiny:{seed}:{name}")
        if len(shape) == 1:
            x = 1.0 + norm_std * x
            if name.endswith("q_norm.weight") or name.endswith("k_norm.weight"):
                x = x * sharp
        else:
            x = std * x
        out[name] = x
    return out


def write_model_folder(folder: Path, cfg: dict, weights: dict[str, torch.Tensor], dtype: Optional[torch.dtype] = None) -> Path:
    """config.json + model.safetensors, written with the safetensors package (not the engine's writer)."""
    import json

    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    tensors = {k: (v if dtype is None else v.to(dtype)).contiguous() for k, v in weights.items()}
    save_file(tensors, str(folder / "model.safetensors"))
    return folder
