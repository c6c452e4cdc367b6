"""Writes tests/golden/flash_attention.json and tests/golden/qwen3_flash_{a,b}.json: outputs of the
reference's own attention path (its FlashSDPA, which calls the flash-attn library) on a GPU.

Run once, by hand, on a machine with a CUDA device, flash-attn and triton, where
mirceamironenco/tokensprint is checked out or installed:

    python tests/golden/make_golden_flash.py /path/to/tokensprint [output folder]

tests/golden/make_golden.py anchors everything but the softmax-attention core on the reference's
modules, on the CPU, where that core had to be swapped out.  This script anchors the core:

* `flash_attention.json`: the reference's FlashSDPA.forward (engine/nn/sdpa.py:40-82, dense path)
  on bfloat16 q, k, v of several shapes with grouped heads; inputs come from the tests' own
  generator (tests/tiny_configs.seeded_normal), so only the outputs are stored.
* `qwen3_flash_{a,b}.json`: logits of the reference's unmodified Transformer (engine/models/
  _builder.py:20-109: FlashSDPA, Triton RoPE and RMSNorm, its serving choices) in bfloat16 for the
  two tiny configurations, weights from tests/tiny_configs.tiny_weights(seed 1234, std 0.05)
  rounded to bfloat16 and loaded through the reference's checkpoint converter.

Nothing of this repository's engine runs here.  Stored values are bfloat16 results widened to
float and written with 5 significant digits.
"""

from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))

from tests.tiny_configs import TINY_A, TINY_B, seeded_normal, tiny_weights  # noqa: E402

# (tokens, query heads, key/value heads, head size): groups of 2, 3, 8 and 5, one KV head, no grouping
ATTENTION_SHAPES = [(40, 4, 2, 16), (33, 6, 2, 32), (21, 8, 1, 64), (19, 5, 1, 128), (130, 4, 4, 32), (1, 6, 3, 64)]
MODEL_SEED, MODEL_STD = 1234, 0.05
SEQUENCE_LENGTHS = (1, 9, 17, 33)


def attention_inputs(shape: tuple[int, int, int, int]) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """bfloat16 q [T, nq, d], k and v [T, nkv, d]; the test derives the same from the shape."""
    T, nq, nkv, d = shape
    name = "x".join(map(str, shape))
    q = seeded_normal((T, nq, d), f"flash:q:{name}").to(torch.bfloat16)
    k = seeded_normal((T, nkv, d), f"flash:k:{name}").to(torch.bfloat16)
    v = seeded_normal((T, nkv, d), f"flash:v:{name}").to(torch.bfloat16)
    return q, k, v


def rounded_weights(cfg: dict) -> dict[str, torch.Tensor]:
    return {k: v.to(torch.bfloat16) for k, v in tiny_weights(cfg, seed=MODEL_SEED, std=MODEL_STD).items()}


def weights_checksum(weights: dict[str, torch.Tensor]) -> str:
    h = hashlib.sha256()
    for name in sorted(weights):
        h.update(name.encode())
        h.update(weights[name].to(torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


def sequences_for(cfg: dict) -> list[list[int]]:
    """Token ids from a hash, so they do not depend on a library's random generator."""
    out = []
    for n in SEQUENCE_LENGTHS:
        digest = hashlib.sha256(f"flash:ids:{cfg['vocab_size']}:{n}".encode()).digest()
        out.append([(i * 7919 + digest[i % 32] * 131 + n) % cfg["vocab_size"] for i in range(n)])
    return out


def as_list(t: torch.Tensor):
    return [[float(f"{x:.5g}") for x in row] for row in t.float().reshape(t.shape[0], -1).tolist()]


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden_flash.py /path/to/tokensprint [output folder]")
    sys.path.insert(0, sys.argv[1])
    out_dir = Path(sys.argv[2]) if len(sys.argv) > 2 else Path(__file__).resolve().parent
    out_dir.mkdir(parents=True, exist_ok=True)
    if not torch.cuda.is_available():
        raise SystemExit("this script needs a CUDA device (flash-attn has no CPU path)")
    device = torch.device("cuda")

    from engine.models._builder import build_model
    from engine.models.qwen._archs import QwenModelConfig
    from engine.models.qwen._checkpoint import convert_qwen_hf_checkpoint_to_mini
    from engine.nn.attention import AttentionConfig
    from engine.nn.layers import FFNConfig
    from engine.nn.sdpa import FlashSDPA
    from engine.utils import reset_non_persistent_buffers

    sdpa = FlashSDPA()
    cases = []
    with torch.no_grad():
        for shape in ATTENTION_SHAPES:
            q, k, v = (t.to(device) for t in attention_inputs(shape))
            out = sdpa(q, k, v)
            cases.append({"shape": list(shape), "out": as_list(out.cpu())})
    path = out_dir / "flash_attention.json"
    path.write_text(json.dumps({"what": "FlashSDPA.forward(q, k, v), dense path, bfloat16", "cases": cases}))
    print("wrote", path, path.stat().st_size, "bytes")

    for tag, cfg in (("a", TINY_A), ("b", TINY_B)):
        weights = rounded_weights(cfg)
        mc = QwenModelConfig(
            attn_config=AttentionConfig(
                model_dim=cfg["hidden_size"], num_heads=cfg["num_attention_heads"],
                num_kv_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"],
                qk_norm=True, qk_norm_eps=cfg["rms_norm_eps"]),
            ffn_config=FFNConfig(model_dim=cfg["hidden_size"], inner_dim=cfg["intermediate_size"]),
            vocab_dim=cfg["vocab_size"], num_layers=cfg["num_hidden_layers"],
            max_seq_len=cfg["max_position_embeddings"], rope_theta=cfg["rope_theta"], rope_impl="triton",
            norm_eps=cfg["rms_norm_eps"], rmsnorm_impl="triton", tie_weights=cfg["tie_word_embeddings"])
        model = build_model(mc, device=device, dtype=torch.bfloat16)
        state = convert_qwen_hf_checkpoint_to_mini({k: v.clone() for k, v in weights.items()}, mc)
        if not cfg["tie_word_embeddings"]:
            # the reference's untied head is nn.Linear with a bias the checkpoint lacks (_builder.py:96)
            state["output_proj.bias"] = torch.zeros(cfg["vocab_size"], dtype=torch.bfloat16)
        model.load_state_dict(state, strict=True)
        reset_non_persistent_buffers(model)
        sequences = sequences_for(cfg)
        logits = []
        with torch.no_grad():
            for ids in sequences:
                t = torch.tensor(ids, dtype=torch.long, device=device)
                logits.append(model(t, input_pos=torch.arange(len(ids), device=device)).float().cpu())
        record = {
            "what": "logits of the reference's Transformer (FlashSDPA, Triton RoPE and RMSNorm), bfloat16",
            "config": cfg, "seed": MODEL_SEED, "std": MODEL_STD, "weights_sha256": weights_checksum(weights),
            "sequences": sequences, "logits": [as_list(l) for l in logits],
        }
        path = out_dir / f"qwen3_flash_{tag}.json"
        path.write_text(json.dumps(record))
        print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
