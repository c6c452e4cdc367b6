"""Helpers of the GPU tests: model folders, traces in several cuttings, comparison with the plain model."""

from __future__ import annotations

import random
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from tests.plain import qwen3_plain as plain
from tests.tiny_configs import tiny_weights, write_model_folder

# Largest allowed |engine - plain| relative to the largest |logit| of the sequence.
# float32: sums of a few hundred float32 products per logit, several layers deep.
# bfloat16: 8 bits of mantissa (2^-9 per rounding) on weights and on each activation
# handed from kernel to kernel, several layers deep, against a float64 model of the
# unrounded weights.
TOLERANCE = {"float32": 1e-4, "bfloat16": 4e-2}


def round64(n: int) -> int:
    return -(-n // 64) * 64


def random_tokens(cfg: dict, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()


class PlainOracle:
    """Plain logits of whole sequences, computed once per sequence."""

    def __init__(self, cfg: dict, weights: dict[str, torch.Tensor]) -> None:
        self.cfg, self.weights = cfg, weights
        self._cache: dict[tuple, torch.Tensor] = {}

    def logits(self, ids: list[int]) -> torch.Tensor:
        key = tuple(ids)
        if key not in self._cache:
            self._cache[key] = plain.forward_logits(self.weights, self.cfg, ids, dtype=torch.float64)
        return self._cache[key]


def make_folder(tmp: Path, cfg: dict, seed: int, sharp: float = 3.0, std: float = 0.05) -> tuple[Path, dict[str, torch.Tensor]]:
    weights = tiny_weights(cfg, seed, std=std, sharp=sharp)
    return write_model_folder(tmp, cfg, weights), weights


# ---------------------------------------------------------------------------
# traces: lists of step records in the trace_run format


def trace_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, every position wanted."""
    steps = []
    for i, (rid, ids) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]})
    return steps


def trace_decode_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps = []
    n = 0
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
        n += 1
        for t in range(head, len(ids)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [ids[t]], "want": [0]}], "end": [rid] if t == len(ids) - 1 else []})
            n += 1
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: dict[str, list[int]], sizes=(7, 2, 13, 2, 64, 3, 2, 31, 5, 2, 16, 17)) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    steps = []
    n = 0
    for rid, ids in requests.items():
        pos, k = 0, 0
        while pos < len(ids):
            size = min(sizes[k % len(sizes)], len(ids) - pos)
            k += 1
            last = pos + size == len(ids)
            steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[pos : pos + size], "want": list(range(size))}], "end": [rid] if last else []})
            n += 1
            pos += size
    return steps


def trace_mixed(requests: dict[str, list[int]], max_tokens: int, seed: int, max_live: int = 4) -> list[dict]:
    """Up to `max_live` live requests: portions of some beside single tokens of others, some
    requests left out of a step; admission keeps sum(round64(final length)) <= max_tokens,
    so with a small max_tokens the pages of finished requests are handed to later ones."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}  # id -> tokens done
    steps = []
    n = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting[0]
            held = sum(round64(len(requests[r])) for r in live)
            if held + round64(len(ids)) > max_tokens:
                break
            waiting.pop(0)
            live[rid] = 0
        if not live:
            raise ValueError("max_tokens is too small for the next request")
        entries, ended = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue  # left out of this step, goes on later
            ids, done = requests[rid], live[rid]
            left = len(ids) - done
            mode = rng.random()
            if mode < 0.4:
                size = 1
            elif mode < 0.6:
                size = 2
            else:
                size = rng.choice([3, 5, 7, 13, 16, 17, 31, 40])
            size = min(size, left)
            entries.append({"id": rid, "tokens": ids[done : done + size], "want": list(range(size))})
            live[rid] = done + size
            if live[rid] == len(ids):
                ended.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": n, "entries": entries, "end": ended})
        n += 1
    return steps


# ---------------------------------------------------------------------------
# running and comparing


def replay_in_process(replayer, steps: list[dict]) -> dict[tuple[str, int], np.ndarray]:
    """Runs the steps; returns logits keyed by (request, position)."""
    done: dict[str, int] = {}
    out: dict[tuple[str, int], np.ndarray] = {}
    for record in steps:
        result = replayer.run_step(record)
        row = 0
        for e in record["entries"]:
            start = done.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], start + w)] = result[row]
                row += 1
            done[e["id"]] = start + len(e["tokens"])
        replayer.runner.cache_manager.check_invariants()
    return out


def worst_error(got: dict[tuple[str, int], np.ndarray], requests: dict[str, list[int]], oracle: PlainOracle) -> tuple[float, Optional[tuple[str, int]]]:
    """Largest relative error over all (request, position), and where it is."""
    worst, where = 0.0, None
    for rid, ids in requests.items():
        want = oracle.logits(ids).numpy()
        scale = float(np.abs(want).max())
        for pos in range(len(ids)):
            if (rid, pos) not in got:
                continue
            g = got[(rid, pos)].astype(np.float64)
            if not np.all(np.isfinite(g)):
                return float("inf"), (rid, pos)
            err = float(np.abs(g - want[pos]).max()) / scale
            if err > worst:
                worst, where = err, (rid, pos)
    return worst, where


def first_bad(got, requests, oracle, tol) -> Optional[tuple[str, int, float]]:
    """The first position (per request order) whose error exceeds tol: where to look for a
    fault of the cache or the batch."""
    for rid, ids in requests.items():
        want = oracle.logits(ids).numpy()
        scale = float(np.abs(want).max())
        for pos in range(len(ids)):
            if (rid, pos) in got:
                g = got[(rid, pos)].astype(np.float64)
                err = float(np.abs(g - want[pos]).max()) / scale if np.all(np.isfinite(g)) else float("inf")
                if err > tol:
                    return rid, pos, err
    return None
