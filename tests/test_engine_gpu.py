"""Generation through the entry point, long decoding, the first tokens, preemption, graphs."""

import json

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.replay_helpers import TOLERANCE, PlainOracle, make_folder, random_tokens, replay_in_process, worst_error
from tests.tiny_configs import TINY_A, TINY_B, TINY_C

pytestmark = pytest.mark.gpu


def plain_greedy(weights, cfg, prompt, steps):
    ids = list(prompt)
    for _ in range(steps):
        ids.append(int(torch.argmax(plain.forward_logits(weights, cfg, ids)[-1])))
    return ids[len(prompt):]


def make_engine(folder, dtype, **kw):
    from tokensprint_b200.config.engine_config import Config
    from tokensprint_b200.engine.llm_engine import LLMEngine
    from tokensprint_b200.models.api import load_model

    model, _ = load_model(folder, device="cuda", dtype=dtype)
    defaults = dict(model=str(folder), max_model_len=256, num_kvcache_blocks=64, max_num_batched_tokens=64,
                    max_num_seqs=8, chunked_prefill=True, dtype=dtype, enforce_eager=True)
    defaults.update(kw)
    return LLMEngine(model, Config(**defaults))


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("cfg", [TINY_A, TINY_C], ids=["a", "c"])
def test_greedy_generation_equals_the_plain_model(tmp_path, cfg, eager):
    from tokensprint_b200.config.engine_config import SamplingParams

    folder, weights = make_folder(tmp_path, cfg, 3, sharp=2.0)
    prompts = [random_tokens(cfg, n, 50 + n) for n in (5, 17, 33, 64)]
    want = [plain_greedy(weights, cfg, p, 16) for p in prompts]
    engine = make_engine(folder, "float32", enforce_eager=eager)
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True), use_tqdm=False)
    assert got == want
    if not eager:
        assert engine.model_runner._graphs, "decode steps did not go through a graph"
    engine.model_runner.cache_manager.check_invariants()
    assert engine.model_runner.cache_manager.pages_in_use() == 0


def test_the_largest_batch_has_a_graph_whatever_the_number_of_slots(tmp_path):
    """Five slots: the buckets are 1, 2, 4 and 8, and a decode step of five sequences replays the
    last one (it used to be launched kernel by kernel); the tokens are the eager run's."""
    from tokensprint_b200.config.engine_config import SamplingParams

    folder, _ = make_folder(tmp_path, TINY_A, 3, sharp=2.0)
    prompts = [random_tokens(TINY_A, n, 20 + n) for n in (4, 9, 13, 21, 30)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    want = make_engine(folder, "float32", max_num_seqs=5).generate(prompts, sp, use_tqdm=False)
    engine = make_engine(folder, "float32", max_num_seqs=5, enforce_eager=False)
    runner = engine.model_runner
    assert runner.graph_buckets == [1, 2, 4, 8]
    replayed = runner.graph_launches
    assert engine.generate(prompts, sp, use_tqdm=False) == want
    # every decode step was a replay: nine steps of five sequences went through the graph of 8
    assert 8 in runner._graphs and runner.graph_launches - replayed >= 9 * runner._graphs[8].kernels


def test_timers_per_kernel_class_for_eager_steps(tmp_path):
    """`collect_stats(kernels=True)`: every launching function of the engine is bracketed by CUDA
    events while the run lasts, the tokens are what they are without timers, and afterwards the
    functions are the plain ones again."""
    from tokensprint_b200 import ops
    from tokensprint_b200.config.engine_config import SamplingParams

    folder, _ = make_folder(tmp_path, TINY_A, 3, sharp=2.0)
    prompts = [random_tokens(TINY_A, n, 50 + n) for n in (5, 17, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    want = make_engine(folder, "bfloat16").generate(prompts, sp, use_tqdm=False)
    plain_embed = ops.embed_gather
    engine = make_engine(folder, "bfloat16")
    stats = engine.collect_stats(kernels=True)
    assert ops.embed_gather is not plain_embed
    assert engine.generate(prompts, sp, use_tqdm=False) == want
    summary = stats.summary()
    assert ops.embed_gather is plain_embed and not ops._plain_functions
    kernels = summary["kernels"]
    steps = sum(summary[kind]["steps"] for kind in ("decode", "prefill", "mixed"))
    assert kernels["embed_gather"]["calls"] == steps and kernels["sample"]["calls"] == steps
    assert sum(row["calls"] for name, row in kernels.items() if name.startswith("attention")) == steps * TINY_A["num_hidden_layers"]
    assert all(row["ms"] > 0 for row in kernels.values())
    assert sum(row["ms"] for row in kernels.values()) <= sum(summary[kind]["device_ms"] for kind in ("decode", "prefill", "mixed")) * 1.05


def test_generation_is_the_same_however_it_is_cut_and_batched(tmp_path):
    """Whole prompts, small chunks, one request at a time, eager or graphs: same tokens
    (float32 greedy, and temperature sampling under a fixed seed)."""
    from tokensprint_b200.config.engine_config import SamplingParams

    folder, _ = make_folder(tmp_path, TINY_B, 4, sharp=2.0)
    prompts = [random_tokens(TINY_B, n, 70 + n) for n in (1, 9, 31, 100, 150)]
    for sp in (SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True),
               SamplingParams(temperature=0.8, max_tokens=12, ignore_eos=True, seed=5)):
        runs = []
        for kw in (dict(chunked_prefill=False, max_num_batched_tokens=512), dict(max_num_batched_tokens=7),
                   dict(max_num_seqs=1), dict(enforce_eager=False, max_num_batched_tokens=40)):
            runs.append(make_engine(folder, "float32", **kw).generate(prompts, sp, use_tqdm=False))
        assert all(r == runs[0] for r in runs[1:])
        assert all(len(c) == 12 for c in runs[0])
    other = make_engine(folder, "float32").generate(prompts, SamplingParams(temperature=0.8, max_tokens=12, ignore_eos=True, seed=6), use_tqdm=False)
    assert other != runs[0]


def test_preemption_and_recompute_do_not_change_the_tokens(tmp_path):
    """A cache so small that requests are preempted and recomputed: same tokens as with room for all."""
    from tokensprint_b200.config.engine_config import SamplingParams

    folder, _ = make_folder(tmp_path, TINY_B, 6, sharp=2.0)
    prompts = [random_tokens(TINY_B, n, 90 + n) for n in (1, 9, 31, 100, 150, 200)]
    sp = SamplingParams(temperature=0.8, max_tokens=24, ignore_eos=True, seed=11)
    roomy = make_engine(folder, "float32", kvcache_block_size=32, num_kvcache_blocks=64, max_num_batched_tokens=64)
    want = roomy.generate(prompts, sp, use_tqdm=False)
    assert roomy.scheduler.num_preemptions == 0
    tight = make_engine(folder, "float32", kvcache_block_size=32, num_kvcache_blocks=12, max_num_batched_tokens=64)
    got = tight.generate(prompts, sp, use_tqdm=False)
    assert tight.scheduler.num_preemptions >= 1
    assert got == want
    assert tight.model_runner.cache_manager.pages_in_use() == 0


@pytest.mark.parametrize("eager", [True, False])
def test_overlapping_steps_change_no_token(tmp_path, eager):
    """Steps launched before the host has read the ids of the step before (their tokens are fed on
    the device), against steps one by one: the same completions, with an end-of-sequence token that
    random weights do sample (so ends are seen one step late and the extra token is dropped) and
    with so few pages that requests are preempted while a step of theirs is in flight."""
    from tokensprint_b200.config.engine_config import SamplingParams

    folder, _ = make_folder(tmp_path, TINY_B, 6, sharp=2.0)
    prompts = [random_tokens(TINY_B, n, 40 + n) for n in (1, 9, 31, 100, 150, 200, 3, 60)]
    sps = [SamplingParams(temperature=0.9, max_tokens=40 - 3 * i, ignore_eos=(i % 3 == 0), seed=21) for i in range(len(prompts))]
    # the end-of-sequence token: one that the requests which heed it do sample, a few tokens in
    free = make_engine(folder, "float32", kvcache_block_size=32, num_kvcache_blocks=64, max_num_batched_tokens=64,
                       overlap_steps=False).generate(prompts, sps, use_tqdm=False)
    seen = [t for c, sp in zip(free, sps) if not sp.ignore_eos for t in c[3:]]
    eos = max(set(seen), key=seen.count)
    runs = {}
    for overlap in (False, True):
        kw = dict(kvcache_block_size=32, num_kvcache_blocks=14, max_num_batched_tokens=64, eos=eos, enforce_eager=eager,
                  overlap_steps=overlap)
        engine = make_engine(folder, "float32", **kw)
        assert engine.overlap == overlap
        runs[overlap] = engine.generate(prompts, sps, use_tqdm=False)
        assert engine.scheduler.num_preemptions >= 1
        assert engine.model_runner.cache_manager.pages_in_use() == 0
        engine.model_runner.cache_manager.check_invariants()
    assert runs[True] == runs[False]
    ended_early = [c for c, sp in zip(runs[True], sps) if len(c) < sp.max_tokens]
    assert ended_early and all(c[-1] == eos for c in ended_early), "no request ended with the end-of-sequence token"


@pytest.mark.parametrize("graphs", [False, True])
def test_a_step_takes_tokens_that_only_the_device_knows(tmp_path, graphs):
    """`StepEntry.feed`: a decoded token that lies in a device tensor (what the step before sampled)
    gives the same logits as the same token given by the host, beside entries of both kinds."""
    from tokensprint_b200.engine.runner import ModelRunner, StepEntry
    from tokensprint_b200.models.api import load_model

    cfg = TINY_A
    folder, _ = make_folder(tmp_path, cfg, 9, sharp=2.0)
    model, _ = load_model(folder, device="cuda", dtype="float32")
    results = []
    for fed in (False, True):
        runner = ModelRunner(model, page_size=16, num_pages=32, num_slots=4, enforce_eager=not graphs, max_model_len=128)
        cm = runner.cache_manager
        prompts = [random_tokens(cfg, n, 60 + n) for n in (5, 17, 9)]
        caches = []
        for i, p in enumerate(prompts):
            rc = cm.admit(i)
            cm.extend(rc, 0, len(p))
            caches.append(rc)
        runner.step([StepEntry(rc, p, 0, []) for rc, p in zip(caches, prompts)])
        nxt = [11, 22, 33]
        device_ids = torch.tensor([99, nxt[2], 99, nxt[0]], dtype=torch.int32, device="cuda")  # rows 1 and 3 are used
        entries = []
        for i, (rc, p) in enumerate(zip(caches, prompts)):
            cm.extend(rc, len(p), len(p) + 1)
            feed = {0: 3, 2: 1}.get(i, -1) if fed else -1
            entries.append(StepEntry(rc, [0 if feed >= 0 else nxt[i]], len(p), [0], feed))
        results.append(runner.step(entries, device_ids).clone())
        assert bool(runner._graphs) == graphs
    assert torch.equal(results[0], results[1])
    with pytest.raises(ValueError, match="given none"):
        runner.step([StepEntry(caches[0], [0], len(prompts[0]), [0], 0)])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(tmp_path, dtype):
    """Several hundred single-token steps across many pages, in graphs, against the plain model."""
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.engine.runner import ModelRunner
    from tokensprint_b200.models.api import load_model

    cfg = TINY_C
    folder, weights = make_folder(tmp_path, cfg, 8, sharp=3.0 if dtype == "float32" else 1.0)
    ids = random_tokens(cfg, 400, 123)
    other = random_tokens(cfg, 300, 124)
    model, _ = load_model(folder, device="cuda", dtype=dtype)
    runner = ModelRunner(model, page_size=16, num_pages=64, num_slots=4, enforce_eager=False, max_model_len=512)
    replayer = TraceReplayer(runner)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": ids[:8], "want": list(range(8))},
                                     {"id": "y", "tokens": other[:3], "want": [0, 1, 2]}], "end": []}]
    for t in range(8, 400):
        entries = [{"id": "x", "tokens": [ids[t]], "want": [0]}]
        if t - 5 < 300:
            entries.append({"id": "y", "tokens": [other[t - 5]], "want": [0]})
        steps.append({"step": t, "entries": entries, "end": []})
    got = replay_in_process(replayer, steps)
    assert runner._graphs, "decode steps did not go through a graph"
    worst, where = worst_error(got, {"x": ids, "y": other}, PlainOracle(cfg, weights))
    assert worst < TOLERANCE[dtype], f"worst error {worst} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(tmp_path, dtype):
    """Positions 0, 1, 2 alone and together: one key, no page boundary, nothing to mask."""
    from tokensprint_b200.engine.replay import TraceReplayer

    cfg = TINY_B
    folder, weights = make_folder(tmp_path, cfg, 9, sharp=3.0 if dtype == "float32" else 1.0)
    oracle = PlainOracle(cfg, weights)
    reqs = {"one": random_tokens(cfg, 1, 1), "two": random_tokens(cfg, 2, 2), "three": random_tokens(cfg, 3, 3)}
    steps = [
        {"step": 0, "entries": [{"id": "one", "tokens": reqs["one"], "want": [0]},
                                {"id": "two", "tokens": reqs["two"][:1], "want": [0]},
                                {"id": "three", "tokens": reqs["three"], "want": [0, 1, 2]}], "end": ["one", "three"]},
        {"step": 1, "entries": [{"id": "two", "tokens": reqs["two"][1:], "want": [0]}], "end": ["two"]},
    ]
    got = replay_in_process(TraceReplayer.from_folder(folder, dtype, 256), steps)
    worst, where = worst_error(got, reqs, oracle)
    assert len(got) == 6 and worst < TOLERANCE[dtype], f"worst error {worst} at {where}"


def test_run_py_generates_from_token_ids(tmp_path, capsys):
    import run

    folder, weights = make_folder(tmp_path / "m", TINY_A, 2, sharp=2.0)
    prompt = random_tokens(TINY_A, 9, 5)
    args = run.parse_args(["--model-dir", str(folder), "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6",
                           "--temperature", "0", "--dtype", "float32", "--num-kvcache-blocks", "16", "--enforce-eager", "True"])
    run.main(args)
    out = capsys.readouterr().out.strip().splitlines()[-1]
    got = [int(t) for t in out.split()]
    want = plain_greedy(weights, TINY_A, prompt, 6)
    eos = -1
    assert got == want or (eos in want and got == want[: want.index(eos) + 1])


def test_trace_run_as_a_program(tmp_path):
    """bin/trace_run over stdin/stdout, files in --out, `done <step>` after every step."""
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    cfg = TINY_A
    folder, weights = make_folder(tmp_path / "m", cfg, 12, sharp=3.0)
    ids = random_tokens(cfg, 70, 77)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": ids[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": ids[40:42], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": ids[42:], "want": [27]}], "end": ["a"]},
    ]
    root = Path(__file__).resolve().parents[1]
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "2.f32"]
    want = PlainOracle(cfg, weights).logits(ids).numpy()
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, cfg["vocab_size"])
    b = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, cfg["vocab_size"])
    scale = np.abs(want).max()
    assert np.abs(a[0] - want[0]).max() < 1e-4 * scale and np.abs(a[1] - want[39]).max() < 1e-4 * scale
    assert np.abs(b[0] - want[69]).max() < 1e-4 * scale
