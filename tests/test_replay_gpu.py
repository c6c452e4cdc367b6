"""The engine against the plain model, under every way of cutting and batching the work.

Each request alone and whole; most of it in one step and the last 32 tokens one by one;
in portions of changing size, down to two tokens; and mixed, up to four live requests,
portions of some beside decoded tokens of others, with so few pages that they are used
again.  In float32 and in bfloat16, for three tiny configurations.

The float32 runs use "sharp" weights (q/k norm weights times 3): the softmax picks few
keys, so one wrong key anywhere moves the logits far beyond the tolerance.  The same
weights would make bfloat16 useless as a yardstick: rounding q and k to 8 bits alone then
moves the logits by 10 to 40 % (measured with the plain model's `rounding` hook), so the
bfloat16 runs use the plain q/k norm weights, where that noise is about 1 %; single wrong
keys in bfloat16 are hunted in the kernel tests with inputs made for it.
"""

import pytest
import torch

from tests.replay_helpers import (
    TOLERANCE,
    PlainOracle,
    first_bad,
    make_folder,
    random_tokens,
    replay_in_process,
    trace_decode_tail,
    trace_mixed,
    trace_portions,
    trace_whole,
    worst_error,
)
from tests.tiny_configs import TINY

pytestmark = pytest.mark.gpu

LENGTHS = {"a": [5, 17, 33, 64, 100], "b": [1, 9, 31, 100, 150, 200], "c": [3, 26, 70, 129, 190]}
SEEDS = {"a": 11, "b": 22, "c": 33}
SHARP = {"float32": 3.0, "bfloat16": 1.0}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for tag, cfg in TINY.items():
        requests = {f"r{i}": random_tokens(cfg, n, 1000 * SEEDS[tag] + i) for i, n in enumerate(LENGTHS[tag])}
        for dtype, sharp in SHARP.items():
            folder, weights = make_folder(tmp_path_factory.mktemp(f"tiny_{tag}_{dtype}"), cfg, SEEDS[tag], sharp=sharp)
            out[tag, dtype] = (folder, cfg, requests, PlainOracle(cfg, weights))
    return out


# (configuration, page size): every configuration at the default page of 16; B also at 32, the page
# its workload is stated with, and at 8; A at 8 and at 256 (one page holds any of its requests); C
# (windows give pages back) at 32 and at 256.
CASES = [("a", 16), ("b", 16), ("c", 16), ("b", 32), ("a", 8), ("c", 256), ("a", 256), ("b", 8), ("c", 32)]


def _replayer(folder, dtype, max_tokens, page_size=16):
    from tokensprint_b200.engine.replay import TraceReplayer

    r = TraceReplayer.from_folder(folder, dtype, max_tokens, page_size=page_size, max_live=4)
    r.runner.poison_freed_pages = True
    return r


def _check(got, requests, oracle, dtype, what):
    tol = TOLERANCE[dtype]
    worst, where = worst_error(got, requests, oracle)
    bad = first_bad(got, requests, oracle, tol)
    assert bad is None, f"{what}: first wrong token at request {bad[0]} position {bad[1]} (error {bad[2]:.3g}); worst {worst:.3g} at {where}"
    assert len(got) == sum(len(v) for v in requests.values()), f"{what}: logits are missing"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag, page", CASES)
def test_whole(models, tag, page, dtype):
    folder, cfg, requests, oracle = models[tag, dtype]
    got = replay_in_process(_replayer(folder, dtype, 256, page), trace_whole(requests))
    _check(got, requests, oracle, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag, page", CASES)
def test_decode_tail(models, tag, page, dtype):
    folder, cfg, requests, oracle = models[tag, dtype]
    got = replay_in_process(_replayer(folder, dtype, 256, page), trace_decode_tail(requests))
    _check(got, requests, oracle, dtype, "decode tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag, page", CASES)
def test_portions(models, tag, page, dtype):
    folder, cfg, requests, oracle = models[tag, dtype]
    got = replay_in_process(_replayer(folder, dtype, 256, page), trace_portions(requests))
    _check(got, requests, oracle, dtype, "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag, page", CASES)
def test_mixed_with_page_reuse(models, tag, page, dtype):
    folder, cfg, requests, oracle = models[tag, dtype]
    # twice over the requests under new names, so that later ones get pages earlier ones gave back
    many = dict(requests)
    many.update({k + "x": v for k, v in requests.items()})
    max_tokens = {"a": 192, "b": 448, "c": 384}[tag]
    steps = trace_mixed(many, max_tokens, seed=7)
    replayer = _replayer(folder, dtype, max_tokens, page)
    got = replay_in_process(replayer, steps)
    pool = replayer.runner.cache_manager.pools[0]
    assert sum(-(-len(v) // page) for v in many.values()) > pool.num_pages, "pages were not used again"
    if page <= 64:
        assert sum(len(v) for v in many.values()) > pool.num_pages * page, "pages were not used again"
    assert pool.num_free == pool.num_pages, "pages were lost"
    _check(got, many, oracle, dtype, "mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_agree_with_each_other(models, dtype):
    """The same position through different cuttings: equal beyond rounding."""
    folder, cfg, requests, oracle = models["b", dtype]
    whole = replay_in_process(_replayer(folder, dtype, 256), trace_whole(requests))
    parts = replay_in_process(_replayer(folder, dtype, 256), trace_portions(requests))
    tol = TOLERANCE[dtype]
    for key, row in whole.items():
        scale = float(abs(row).max())
        assert float(abs(row - parts[key]).max()) <= tol * scale, f"cuttings differ at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_that_ends_and_starts_again_under_its_name(models, dtype):
    """What a preemption looks like in a trace: a request is ended in the middle, another one takes
    its pages, then it comes back under the same id and is computed again from its first token."""
    folder, cfg, requests, oracle = models["b", dtype]
    ids, other = requests["r3"], requests["r2"]
    steps = [
        {"step": 0, "entries": [{"id": "p", "tokens": ids[:40], "want": list(range(40))}], "end": []},
        {"step": 1, "entries": [{"id": "p", "tokens": ids[40:41], "want": [0]}, {"id": "q", "tokens": other, "want": list(range(len(other)))}], "end": ["p"]},
        {"step": 2, "entries": [{"id": "q2", "tokens": other[:9], "want": [8]}], "end": ["q", "q2"]},
        {"step": 3, "entries": [{"id": "p", "tokens": ids[:70], "want": list(range(70))}], "end": []},
        {"step": 4, "entries": [{"id": "p", "tokens": ids[70:], "want": list(range(len(ids) - 70))}], "end": ["p"]},
    ]
    replayer = _replayer(folder, dtype, 192, 32)
    first = {}
    got = {}
    for record in steps:
        out = replayer.run_step(record)
        if record["step"] == 0:
            first = {("p", i): out[i] for i in range(40)}
        if record["step"] == 3:
            got.update({("p", i): out[i] for i in range(70)})
        if record["step"] == 4:
            got.update({("p", 70 + i): out[i] for i in range(len(ids) - 70)})
        replayer.runner.cache_manager.check_invariants()
    _check(got, {"p": ids}, oracle, dtype, "second life")
    _check(first, {"p": ids[:40]}, oracle, dtype, "first life")
