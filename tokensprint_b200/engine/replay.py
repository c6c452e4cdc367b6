"""Trace replay: given token ids go through the model step by step, logits come out.

Nothing is sampled.  The replay drives the engine's own model, step function, cache
manager and kernels (the ones generation uses); it has no forward pass, cache or
loader of its own.  One step of a trace is a JSON object

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries`: for each request its next tokens and the places among them whose logits are
wanted; all entries of a step form one batch.  `end`: requests that are finished after
this step; their pages and slot are given back.  For a step in which something is wanted
the logits are written to `<out>/<step>.f32` as little-endian float32 [wanted, vocab].
"""

from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import IO, Any, Optional

import numpy as np
import torch

from tokensprint_b200 import ops
from tokensprint_b200.cache.manager import RequestCache
from tokensprint_b200.engine.runner import ModelRunner, StepEntry
from tokensprint_b200.models.api import load_model

# Defaults of the command line; every one of them is an option.
PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 16
TOKEN_ROUNDING = 64  # --max-tokens counts each live request rounded up to a multiple of this


def pages_for(max_tokens: int, page_size: int, max_live: int) -> int:
    """Pages that hold `max_tokens` tokens of live requests, each request's count rounded up to
    TOKEN_ROUNDING: exactly max_tokens / page_size when pages divide that rounding; larger pages
    round every live request up to a page of their own, so one page more per request."""
    pages = -(-max(max_tokens, 1) // page_size)
    if TOKEN_ROUNDING % page_size:
        pages += max_live
    return pages


class TraceError(ValueError):
    pass


class TraceReplayer:
    def __init__(self, runner: ModelRunner, out_dir: Optional[str | Path] = None) -> None:
        self.runner = runner
        self.out_dir = Path(out_dir) if out_dir is not None else None
        if self.out_dir is not None:
            self.out_dir.mkdir(parents=True, exist_ok=True)
        self.live: dict[str, RequestCache] = {}
        self.lengths: dict[str, int] = {}

    @classmethod
    def from_folder(cls, model_dir: str | Path, dtype: str, max_tokens: int, out_dir: Optional[str | Path] = None,
                    device: str = "cuda", page_size: int = PAGE_SIZE, num_pages: Optional[int] = None,
                    max_live: int = MAX_LIVE_REQUESTS, graphs: bool = False, max_model_len: Optional[int] = None) -> "TraceReplayer":
        """A replayer for a model folder.  The pool holds `num_pages` pages per cache group, or,
        when that is None, what `max_tokens` tokens of live requests need (see pages_for).  With
        `graphs`, steps of single tokens replay CUDA graphs as generation does (bfloat16 models
        whose parts allow it); `max_model_len` bounds the positions such a graph serves."""
        model, config = load_model(model_dir, device=device, dtype=dtype)
        pages = num_pages if num_pages is not None else pages_for(max_tokens, page_size, max_live)
        longest = max_model_len or min(int(getattr(config, "max_position_embeddings", 0) or pages * page_size), pages * page_size)
        runner = ModelRunner(model, page_size=page_size, num_pages=pages, num_slots=max_live,
                             max_num_batched_tokens=max(max_tokens, 1), enforce_eager=not graphs, max_model_len=longest)
        return cls(runner, out_dir)

    def run_step(self, record: dict[str, Any]) -> Optional[np.ndarray]:
        """Runs one step; returns the wanted logits [wanted, vocab] (also written to the
        out folder), or None when nothing was wanted."""
        if "step" not in record or "entries" not in record:
            raise TraceError("a step needs the keys 'step' and 'entries'")
        cm = self.runner.cache_manager
        entries = []
        for e in record["entries"]:
            rid = str(e["id"])
            tokens = [int(t) for t in e["tokens"]]
            if not tokens:
                raise TraceError(f"step {record['step']}: request {rid} brings no tokens")
            rc = self.live.get(rid)
            if rc is None:
                rc = cm.admit(rid)
                self.live[rid] = rc
                self.lengths[rid] = 0
            start = self.lengths[rid]
            cm.extend(rc, start, start + len(tokens))
            entries.append(StepEntry(rc, tokens, start, [int(w) for w in e.get("want", [])]))
        result = None
        if entries:
            logits = self.runner.step(entries)
            for e in entries:
                self.lengths[str(e.cache.request)] += len(e.tokens)
            if logits.shape[0] > 0:
                result = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                if self.out_dir is not None:
                    result.tofile(self.out_dir / f"{record['step']}.f32")
            else:
                torch.cuda.synchronize(self.runner.device)
            ops.check_device_errors()  # the copy back (or the synchronize) has just waited for the step
        for rid in record.get("end", []) or []:
            rid = str(rid)
            rc = self.live.pop(rid, None)
            if rc is None:
                raise TraceError(f"step {record['step']}: request {rid} ends but is not live")
            self.runner.free(rc)
            del self.lengths[rid]
        return result

    def run_stream(self, lines: IO[str], report: IO[str] = sys.stdout) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            try:
                record = json.loads(line)
            except json.JSONDecodeError as e:
                raise TraceError(f"not a JSON object: {line[:80]!r} ({e})") from e
            self.run_step(record)
            print(f"done {record['step']}", file=report, flush=True)


def main(argv: Optional[list[str]] = None) -> int:
    import argparse

    p = argparse.ArgumentParser(prog="trace_run", description="Feed given token ids through a model step by step and write logits.")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help=f"most tokens live requests hold at any time, each request's count rounded up to a multiple of "
                        f"{TOKEN_ROUNDING} (to whole pages where pages are larger); sizes the cache pool")
    p.add_argument("--page-size", type=int, default=PAGE_SIZE, help=f"tokens per cache page (default {PAGE_SIZE})")
    p.add_argument("--num-pages", type=int, default=None, help="pages per cache group (default: what --max-tokens needs)")
    p.add_argument("--max-live", type=int, default=MAX_LIVE_REQUESTS, help=f"most requests live at a time (default {MAX_LIVE_REQUESTS})")
    p.add_argument("--graphs", action="store_true", help="steps of single tokens replay CUDA graphs, as generation does")
    p.add_argument("--max-model-len", type=int, default=None, help="longest request a captured graph serves (default: what the pool holds)")
    args = p.parse_args(argv)
    if args.page_size < 1 or args.max_live < 1 or (args.num_pages is not None and args.num_pages < 1):
        p.error("--page-size, --max-live and --num-pages must be positive")
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; this engine has no CPU path", file=sys.stderr)
        return 1
    replayer = TraceReplayer.from_folder(args.model, args.dtype, args.max_tokens, args.out, page_size=args.page_size,
                                         num_pages=args.num_pages, max_live=args.max_live, graphs=args.graphs,
                                         max_model_len=args.max_model_len)
    replayer.run_stream(sys.stdin)
    return 0
