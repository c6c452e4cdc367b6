"""Plain, slow Qwen3 dense: whole sequences, no cache, one function per part.

Written from the formulas of mirceamironenco/tokensprint (each function cites file:line
of that project); it shares no code with the engine under test.  Weights come as a dict
of tensors under the checkpoint's own names (model.layers.N.self_attn.q_proj.weight, ...).
Everything runs in one dtype (float64 by default) on the CPU.

The attention core (scores, mask, softmax, weighted sum) rests on the formula alone: the
reference hands it to an attention library (engine/nn/sdpa.py:85-102).  Everything else
was compared once with the reference's own modules on the CPU; see tests/golden/.
"""

from __future__ import annotations

import math
from typing import Mapping, Optional, Sequence

import torch


def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """h[t] = E[ids[t]]  (engine/model.py:65)."""
    return table[torch.as_tensor(list(ids), dtype=torch.long, device=table.device)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2, last dim) + eps) * w  (engine/nn/base_layers.py:38-46;
    engine/kernels/triton/rmsnorm.py:19-42)."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def rope_inverse_frequencies(dim: int, theta: float) -> torch.Tensor:
    """inv_freq[j] = 1 / theta^(2j/dim) in float32  (engine/nn/rope.py:28-29)."""
    idx = torch.arange(0, dim, step=2, dtype=torch.float32)
    return 1.0 / (theta ** (idx / dim))


def rope_angles(positions: Sequence[int], dim: int, theta: float) -> torch.Tensor:
    """angle[t, j] = float32(pos[t]) * inv_freq[j], a float32 product as in the reference
    (engine/nn/rope.py:105-108, engine/kernels/triton/rope.py:34)."""
    pos = torch.as_tensor(list(positions), dtype=torch.float32)
    return torch.outer(pos, rope_inverse_frequencies(dim, theta))


def apply_rope(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing (j, j + d/2): x'[j] = x[j] cos - x[j+d/2] sin,
    x'[j+d/2] = x[j+d/2] cos + x[j] sin  (engine/nn/rope.py:111-123;
    engine/kernels/triton/rope.py:53-62).  x: [T, heads, d]; angles: [T, d/2]."""
    half = x.shape[-1] // 2
    cos = angles.to(x.device, x.dtype).cos()[:, None, :]
    sin = angles.to(x.device, x.dtype).sin()[:, None, :]
    re, im = x[..., :half], x[..., half:]
    return torch.cat([re * cos - im * sin, im * cos + re * sin], dim=-1)


def causal_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float, window: Optional[int] = None
) -> torch.Tensor:
    """softmax(q k^T * scale + causal mask) v with grouped heads: query head g reads KV head
    g // (nq / nkv); query t sees keys 0..t (engine/nn/sdpa.py:56,85-102: softmax_scale =
    head_dim^-0.5, causal=True, no softcap).  With `window` = n a query sees only its last
    n keys, itself included (the reference passes window_size=(-1,-1), engine/nn/sdpa.py:97;
    the window is this engine's reading of `attn_window_len`, engine/models/_registry.py:20).
    q: [T, nq, d]; k, v: [T, nkv, d] -> [T, nq, d]."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = torch.empty_like(q)
    t_idx = torch.arange(T, device=q.device)
    visible = t_idx[None, :] <= t_idx[:, None]
    if window is not None and window > 0:
        visible &= t_idx[None, :] > (t_idx[:, None] - window)
    for g in range(nq):
        kh, vh = k[:, g // group], v[:, g // group]
        scores = (q[:, g] @ kh.T) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, g] = torch.softmax(scores, dim=-1) @ vh
    return out


def attention_layer(
    x: torch.Tensor,
    w: Mapping[str, torch.Tensor],
    prefix: str,
    positions: Sequence[int],
    *,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rope_theta: float,
    eps: float,
    window: Optional[int] = None,
    rounding=None,
) -> torch.Tensor:
    """q/k/v projections, reshape to heads, q_norm/k_norm over head_dim (one weight for all
    heads), RoPE on q and k, attention, output projection  (engine/nn/attention.py:164-200)."""
    r = rounding or (lambda t: t)
    T = x.shape[0]
    q = r(x @ w[prefix + "q_proj.weight"].T).view(T, num_heads, head_dim)
    k = r(x @ w[prefix + "k_proj.weight"].T).view(T, num_kv_heads, head_dim)
    v = r(x @ w[prefix + "v_proj.weight"].T).view(T, num_kv_heads, head_dim)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    angles = rope_angles(positions, head_dim, rope_theta)
    q, k = r(apply_rope(q, angles)), r(apply_rope(k, angles))
    o = r(causal_attention(q, k, v, scale=head_dim**-0.5, window=window))
    return r(o.reshape(T, num_heads * head_dim) @ w[prefix + "o_proj.weight"].T)


def swiglu_ffn(x: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, rounding=None) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), silu(z) = z * sigmoid(z)  (engine/nn/layers.py:61-66)."""
    r = rounding or (lambda t: t)
    g = r(x @ w[prefix + "gate_proj.weight"].T)
    u = r(x @ w[prefix + "up_proj.weight"].T)
    return r(r(g * torch.sigmoid(g) * u) @ w[prefix + "down_proj.weight"].T)


def block(
    h: torch.Tensor, w: Mapping[str, torch.Tensor], layer: int, positions: Sequence[int], cfg: Mapping,
    window: Optional[int], rounding=None,
) -> torch.Tensor:
    """Pre-norm: h = h + Attn(RMSNorm(h)); h = h + FFN(RMSNorm(h))  (engine/nn/layers.py:111-121)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    r = rounding or (lambda t: t)
    a = attention_layer(
        r(rms_norm(h, w[p + "input_layernorm.weight"], eps)), w, p + "self_attn.", positions,
        num_heads=cfg["num_attention_heads"], num_kv_heads=cfg["num_key_value_heads"],
        head_dim=cfg["head_dim"], rope_theta=cfg["rope_theta"], eps=eps, window=window, rounding=rounding)
    h = h + a
    f = swiglu_ffn(r(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)), w, p + "mlp.", rounding)
    return h + f


def layer_windows(cfg: Mapping) -> list[Optional[int]]:
    """Per layer: None (full attention) or the window.  `layer_types` wins; else layers from
    `max_window_layers` on slide when `use_sliding_window` is set."""
    n = cfg["num_hidden_layers"]
    types = cfg.get("layer_types")
    if types is None:
        if cfg.get("use_sliding_window") and cfg.get("sliding_window"):
            first = cfg.get("max_window_layers", n)
            types = ["sliding_attention" if i >= first else "full_attention" for i in range(n)]
        else:
            types = ["full_attention"] * n
    return [cfg["sliding_window"] if t == "sliding_attention" else None for t in types]


class _Converted:
    """The weights in the run's dtype and on its device, converted when asked for (and not kept:
    a model of many layers is never held twice)."""

    def __init__(self, weights: Mapping[str, torch.Tensor], dtype: torch.dtype, device, rounding) -> None:
        self.weights, self.dtype, self.device, self.rounding = weights, dtype, device, rounding

    def __getitem__(self, name: str) -> torch.Tensor:
        v = self.weights[name].to(device=self.device, dtype=self.dtype)
        return v if v.dim() == 1 or self.rounding is None else self.rounding(v)


def forward_logits(
    weights: Mapping[str, torch.Tensor], cfg: Mapping, token_ids: Sequence[int], dtype: torch.dtype = torch.float64,
    rounding=None, device=None,
) -> torch.Tensor:
    """Logits [T, V] of one whole sequence: embedding, blocks, final norm, head (tied: the
    embedding table)  (engine/model.py:58-95, engine/nn/layers.py:22-23).

    `rounding` (a function tensor -> tensor) is applied to every matrix weight and to every
    activation that one operation hands to the next, the residual stream excepted.  With
    `round_to_bfloat16` this shows how far 8-bit mantissas alone move the logits of a given
    model and input: the yardstick for a bfloat16 engine's tolerance.

    `device`: where the arithmetic runs (default: the CPU).  The same functions, the same dtype;
    a model of full width is merely done sooner on a GPU."""
    r = rounding or (lambda t: t)
    w = _Converted(weights, dtype, device, rounding)
    positions = list(range(len(token_ids)))
    h = embedding(w["model.embed_tokens.weight"], token_ids)
    for i, window in enumerate(layer_windows(cfg)):
        h = block(h, w, i, positions, cfg, window, rounding)
    h = r(rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return h @ head.T


def round_to_bfloat16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


# ---------------------------------------------------------------------------
# sampling


def _mix64(z: int) -> int:
    m = (1 << 64) - 1
    z = (z + 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


def exponential_noise(key: int, index: int) -> float:
    """Exp(1) noise of (key, index) as the engine's sampler defines it: the entries 2k and 2k + 1
    share one hash of (key, k) (one multiply and two shifts over key ^ k * constant; the key is a
    full hash already); its top 24 bits give u in (0,1) for the even entry,
    the 24 bits below them for the odd one; E = -log(u)."""
    import numpy as np

    m = (1 << 64) - 1
    z = (key & m) ^ (((index >> 1) * 0xD1342543DE82EF95) & m)
    z ^= z >> 32
    z = (z * 0x94D049BB133111EB) & m
    h = z ^ (z >> 29)
    bits = (h >> 40) if index % 2 == 0 else ((h >> 16) & 0xFFFFFF)
    u = np.float32((np.float32(bits) + np.float32(0.5)) * np.float32(1.0 / 16777216.0))
    return float(-np.log(u, dtype=np.float32))


def sample_token(logits: torch.Tensor, temperature: float, key: int) -> int:
    """argmax(softmax(logits / T) / max(E, 1e-10)), E ~ Exp(1) per entry
    (engine/generation/sampler.py:11-16); temperature 0: plain argmax, lowest index on ties."""
    x = logits.to(torch.float64)
    if temperature <= 1e-10:
        return int(torch.argmax(x))
    probs = torch.softmax(x / temperature, dim=-1)
    noise = torch.tensor([max(exponential_noise(key, i), 1e-10) for i in range(x.numel())], dtype=torch.float64)
    return int(torch.argmax(probs / noise))
