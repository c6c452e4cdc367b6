"""Single-prompt generation from the command line, in the manner of the reference's run.py.

    python run.py --model-name qwen/qwen3-0.6b --prompt "..." --max-tokens 256 --temperature 0.8

Options of the reference (run.py:25-32) keep their names, defaults and meanings:
--model-name, --cache-dir, --prompt, --max-tokens, --temperature, --enforce-eager;
booleans take an explicit value (`--enforce-eager True`), as with the reference's
FlagConversionOff.  The model folder is `cache_dir/<last part of the repo id>` unless
--model-dir names one.  Added here: --model-dir, --random-weights SEED (writes a model
folder from the registered config and a seed when none is there), --prompt-ids (token ids
instead of text; without tokenizer files in the folder this is the only way),
--dtype, --kvcache-block-size, --num-kvcache-blocks, --max-num-batched-tokens,
--chunked-prefill, --seed, --overlap-steps (launch a step before the host has read the ids
of the step before; default True).
"""

from __future__ import annotations

import argparse
import logging
import sys
from pathlib import Path

logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s: %(message)s", force=True)
log = logging.getLogger("run")


def _bool(v: str) -> bool:
    if v.lower() in ("true", "1", "yes"):
        return True
    if v.lower() in ("false", "0", "no"):
        return False
    raise argparse.ArgumentTypeError(f"expected True or False, got {v!r}")


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model-name", default="qwen/qwen3-0.6b")
    p.add_argument("--cache-dir", type=Path, default=Path("./local_data"))
    p.add_argument("--prompt", default="Tell me a long story about transformers.")
    p.add_argument("--max-tokens", type=int, default=1024)
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--enforce-eager", type=_bool, default=False)
    p.add_argument("--model-dir", type=Path, default=None)
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED")
    p.add_argument("--prompt-ids", type=str, default=None, help="comma-separated token ids")
    p.add_argument("--dtype", default="bfloat16")
    p.add_argument("--kvcache-block-size", type=int, default=16)
    p.add_argument("--num-kvcache-blocks", type=int, default=-1)
    p.add_argument("--max-num-batched-tokens", type=int, default=16384)
    p.add_argument("--chunked-prefill", type=_bool, default=False)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--overlap-steps", type=_bool, default=True)
    return p.parse_args(argv)


def load_tokenizer(model_dir: Path):
    """The folder's own tokenizer through transformers, if its files are there (the
    reference: engine/tokenizer.py:628-657)."""
    if not any((model_dir / f).exists() for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
        return None
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(str(model_dir), use_fast=True)
    if tok.pad_token_id is None and tok.eos_token_id is not None:
        tok.pad_token = tok.eos_token
    return tok


def main(args: argparse.Namespace) -> None:
    import torch

    from tokensprint_b200.config.engine_config import Config, SamplingParams
    from tokensprint_b200.config.registry import get_local_model_dir, get_model_config
    from tokensprint_b200.engine.llm_engine import LLMEngine
    from tokensprint_b200.models.api import load_model
    from tokensprint_b200.weights.loader import write_random_model

    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is required: this engine has no CPU path.")

    model_dir = args.model_dir or get_local_model_dir(args.model_name, cache_dir=args.cache_dir)
    if args.random_weights is not None and not (model_dir / "config.json").exists():
        log.info("Writing random weights (seed %d) for %s to %s.", args.random_weights, args.model_name, model_dir)
        write_random_model(model_dir, get_model_config(args.model_name), args.random_weights, dtype="bfloat16")
    model, model_cfg = load_model(model_dir, device="cuda", dtype=args.dtype)
    tokenizer = load_tokenizer(Path(model_dir))
    eos = tokenizer.eos_token_id if tokenizer is not None and tokenizer.eos_token_id is not None else model_cfg.eos_token_id

    config = Config(
        model=str(model_dir),
        max_model_len=int(model_cfg.max_position_embeddings),
        eos=eos,
        dtype=args.dtype,
        enforce_eager=args.enforce_eager,
        kvcache_block_size=args.kvcache_block_size,
        num_kvcache_blocks=args.num_kvcache_blocks,
        max_num_batched_tokens=args.max_num_batched_tokens,
        chunked_prefill=args.chunked_prefill,
        overlap_steps=args.overlap_steps,
    )
    engine = LLMEngine(model=model, config=config, tokenizer=tokenizer)
    sampling_params = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, seed=args.seed)

    if args.prompt_ids is not None:
        prompt = [int(t) for t in args.prompt_ids.replace(",", " ").split()]
    elif tokenizer is not None:
        prompt = args.prompt
    else:
        raise SystemExit(f"{model_dir} has no tokenizer files: pass --prompt-ids")
    outputs = engine.generate([prompt], sampling_params)
    if tokenizer is not None:
        print(tokenizer.batch_decode(outputs, skip_special_tokens=True)[0])
    else:
        print(" ".join(str(t) for t in outputs[0]))


if __name__ == "__main__":
    main(parse_args())
