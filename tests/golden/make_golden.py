"""Writes tests/golden/qwen3_tiny_{a,b}.json: logits of the reference's own modules on the CPU.

Run once, by hand, where mirceamironenco/tokensprint is checked out:

    python tests/golden/make_golden.py /path/to/tokensprint

It builds the reference's Transformer (engine/models/_builder.py:20-109) for two tiny
Qwen3 configurations in float32 on the CPU with its table RoPE and torch RMSNorm, swaps
the attention core (the reference hard-wires an attention library that needs CUDA,
_builder.py:76; Attention takes any SDPA, engine/nn/attention.py:95-103) for a
ten-line causal softmax, loads this repo's seeded random weights through the reference's
own checkpoint converter (engine/models/qwen/_checkpoint.py:47-62), and stores the
logits of a few token sequences.  So the reference's embedding, RMSNorm, q/k-norm
placement, RoPE, SwiGLU, block wiring, final norm and head anchor the plain
implementation; the softmax-attention core is anchored on the formula only.

The stored file holds the config, the seed, the token ids, a checksum of the weights
and the logits (float32, rounded to 7 significant digits) - no weights.
"""

from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))

from tests.tiny_configs import TINY_A, TINY_B, tiny_weights  # noqa: E402


def weights_checksum(weights: dict[str, torch.Tensor]) -> str:
    h = hashlib.sha256()
    for name in sorted(weights):
        h.update(name.encode())
        h.update(weights[name].to(torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


def reference_logits(reference_root: str, cfg: dict, weights: dict[str, torch.Tensor], sequences: list[list[int]]):
    sys.path.insert(0, reference_root)
    from engine.models._builder import build_model
    from engine.models.qwen._archs import QwenModelConfig
    from engine.models.qwen._checkpoint import convert_qwen_hf_checkpoint_to_mini
    from engine.nn.attention import AttentionConfig
    from engine.nn.layers import FFNConfig
    from engine.nn.sdpa import SDPA
    from engine.utils import reset_non_persistent_buffers

    class TorchSDPA(SDPA):
        def forward(self, query, key, value, *, attn_mask=None, seqinfo=None):
            T, nq, d = query.shape
            group = nq // key.shape[1]
            k = key.repeat_interleave(group, dim=1)
            v = value.repeat_interleave(group, dim=1)
            s = torch.einsum("tgd,sgd->gts", query, k) * d**-0.5
            s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf"))
            return torch.einsum("gts,sgd->tgd", torch.softmax(s, dim=-1), v)

    mc = QwenModelConfig(
        attn_config=AttentionConfig(
            model_dim=cfg["hidden_size"], num_heads=cfg["num_attention_heads"],
            num_kv_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"],
            qk_norm=True, qk_norm_eps=cfg["rms_norm_eps"]),
        ffn_config=FFNConfig(model_dim=cfg["hidden_size"], inner_dim=cfg["intermediate_size"]),
        vocab_dim=cfg["vocab_size"], num_layers=cfg["num_hidden_layers"],
        max_seq_len=cfg["max_position_embeddings"], rope_theta=cfg["rope_theta"], rope_impl="table",
        norm_eps=cfg["rms_norm_eps"], rmsnorm_impl="torch", tie_weights=cfg["tie_word_embeddings"])
    model = build_model(mc, device=torch.device("cpu"), dtype=torch.float32)
    for layer in model.layers:
        layer.attn_layer.sdpa = TorchSDPA()
    state = convert_qwen_hf_checkpoint_to_mini(dict(weights), mc)
    if not cfg["tie_word_embeddings"]:
        # the reference's untied head is nn.Linear with a bias the checkpoint lacks (_builder.py:96)
        state["output_proj.bias"] = torch.zeros(cfg["vocab_size"])
    model.load_state_dict(state, strict=True)
    reset_non_persistent_buffers(model)
    out = []
    with torch.no_grad():
        for ids in sequences:
            t = torch.tensor(ids, dtype=torch.long)
            out.append(model(t, input_pos=torch.arange(len(ids))))
    return out


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/tokensprint")
    reference_root = sys.argv[1]
    for tag, cfg in (("a", TINY_A), ("b", TINY_B)):
        if cfg.get("use_sliding_window"):
            raise SystemExit("golden configs must be full attention (the reference has no window)")
        weights = tiny_weights(cfg, seed=1234)
        g = torch.Generator().manual_seed(99)
        sequences = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (1, 9, 17)]
        logits = reference_logits(reference_root, cfg, weights, sequences)
        record = {
            "config": cfg,
            "seed": 1234,
            "weights_sha256": weights_checksum(weights),
            "sequences": sequences,
            "logits": [[[float(f"{x:.7g}") for x in row] for row in l.tolist()] for l in logits],
        }
        path = Path(__file__).resolve().parent / f"qwen3_tiny_{tag}.json"
        path.write_text(json.dumps(record))
        print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
