"""Qwen3 layer sizes as served (two layers, so it is quick): the bfloat16 kernels at the widths that
serving uses (head size 128; two, four, five and eight query heads per KV head; widths 1024 to
5120; vocabulary 151936) under several cuttings, every position against the plain model (which
runs its float64 arithmetic on the GPU here, the same functions as on the CPU) and, as a second
line, against the engine's own float32 path."""

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.replay_helpers import random_tokens, replay_in_process, trace_decode_tail, trace_mixed, trace_portions, trace_whole

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["qwen3-8b", "qwen3-14b", "qwen3-32b", "qwen3-0.6b"])
def folder(request, tmp_path_factory):
    """8B: four query heads per KV head; 14B: five (no divisor of 128), width 5120, intermediate
    17408; 32B: eight, intermediate 25600; 0.6B: two, width 1024 with heads of 128 (heads * head
    size is twice the width) and a tied head."""
    from tokensprint_b200.models.qwen3 import Qwen3Config
    from tokensprint_b200.config.registry import get_preset_dict
    from tokensprint_b200.weights.loader import write_random_model

    d = get_preset_dict(request.param)
    d["num_hidden_layers"] = 2
    cfg = Qwen3Config.from_dict(d)
    path = write_random_model(tmp_path_factory.mktemp("wide") / "m", cfg, seed=3, dtype="bfloat16", std=0.02)
    return path, d


def _logits(folder, dtype, steps, graphs=False):
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.engine.runner import ModelRunner
    from tokensprint_b200.models.api import load_model

    model, _ = load_model(folder, device="cuda", dtype=dtype)
    runner = ModelRunner(model, page_size=16, num_pages=64, num_slots=8, enforce_eager=not graphs, max_model_len=512)
    got = replay_in_process(TraceReplayer(runner), steps)
    assert not graphs or runner._graphs
    return got


def test_full_width_cuttings(folder, monkeypatch):
    path, cfg = folder
    requests = {"a": random_tokens(cfg, 150, 1), "b": random_tokens(cfg, 70, 2), "c": random_tokens(cfg, 33, 3)}
    ref = _logits(path, "float32", trace_whole(requests))

    # the plain model for every request and position (float64, its arithmetic on the GPU: the head is 151936 wide)
    from tokensprint_b200.weights.safetensors_io import SafetensorsFolder

    files = SafetensorsFolder(path)
    weights = {n: files.tensor(n) for n in files.keys()}
    want = {}
    for rid, ids in requests.items():
        logits = plain.forward_logits(weights, cfg, ids, dtype=torch.float64, device="cuda").cpu().numpy()
        want.update({(rid, pos): logits[pos] for pos in range(len(ids))})
    del weights
    torch.cuda.empty_cache()
    plain_scale = max(float(abs(v).max()) for v in want.values())

    def against_plain(got, tolerance, what):
        assert len(got) == len(want), f"{what}: logits are missing"
        for key in sorted(want):
            err = float(abs(got[key].astype("float64") - want[key]).max())
            assert err < tolerance * plain_scale, f"{what}: request {key[0]} position {key[1]} strays {err / plain_scale:.3g} from the plain model"

    against_plain(ref, 1e-4, "float32 engine")

    # bfloat16 in every cutting, eager and in graphs, against the plain model and against float32
    scale = max(float(abs(v).max()) for v in ref.values())
    for name, steps, graphs in (
        ("whole", trace_whole(requests), False),
        ("tail", trace_decode_tail(requests), False),
        ("tail in graphs", trace_decode_tail(requests), True),
        ("portions", trace_portions(requests), False),
        ("mixed", trace_mixed(requests, 512, seed=1), False),
        ("mixed with graphs", trace_mixed(requests, 512, seed=2), True),
    ):
        got = _logits(path, "bfloat16", steps, graphs)
        assert len(got) == len(ref)
        against_plain(got, 4e-2, f"bfloat16, {name}")
        worst = max(float(abs(got[k] - ref[k]).max()) for k in ref)
        assert worst < 4e-2 * scale, f"{name}: bfloat16 strays {worst / scale:.3g} from float32"

    # decode steps through the kernel that gives every CTA an even share of all key blocks (the
    # engine takes it for batches whose (sequence, KV head) pairs do not all run at once)
    from tokensprint_b200 import ops

    calls = []
    flat = ops.attention_decode_flat
    monkeypatch.setattr(ops, "attention_decode_prefers_flat", lambda *a: True)
    monkeypatch.setattr(ops, "attention_decode_flat", lambda *a, **k: (calls.append(1), flat(*a, **k))[1])
    for name, steps, graphs in (
        ("tail, even shares", trace_decode_tail(requests), False),
        ("tail in graphs, even shares", trace_decode_tail(requests), True),
        ("mixed with graphs, even shares", trace_mixed(requests, 512, seed=2), True),
    ):
        calls.clear()
        got = _logits(path, "bfloat16", steps, graphs)
        assert calls, f"{name}: the even-share kernel did not run"
        against_plain(got, 4e-2, f"bfloat16, {name}")
        worst = max(float(abs(got[k] - ref[k]).max()) for k in ref)
        assert worst < 4e-2 * scale, f"{name}: bfloat16 strays {worst / scale:.3g} from float32"
    ops.check_device_errors()


def test_many_sequences_decode_through_the_even_share_kernel(tmp_path):
    """Sixty sequences of different lengths decoding together at Qwen3-0.6B layer sizes (8 KV heads
    of 128): more (sequence, KV head) pairs than CTAs run at once, so the engine itself picks the
    even-share decode kernel, in a graph whose batch bucket has lanes without a sequence.  bfloat16
    against the float32 path, the same trace."""
    from tokensprint_b200 import ops
    from tokensprint_b200.models.qwen3 import Qwen3Config
    from tokensprint_b200.config.registry import get_preset_dict
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.engine.runner import ModelRunner
    from tokensprint_b200.models.api import load_model
    from tokensprint_b200.weights.loader import write_random_model

    d = get_preset_dict("qwen3-0.6b")
    d["num_hidden_layers"] = 2
    cfg = Qwen3Config.from_dict(d)
    path = write_random_model(tmp_path / "m", cfg, seed=5, dtype="bfloat16", std=0.02)
    lengths = [3 + (37 * i) % 150 for i in range(60)]
    requests = {f"r{i}": random_tokens(d, n + 6, 100 + i) for i, n in enumerate(lengths)}
    steps = []
    for i, (rid, ids) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": ids[:-6], "want": [len(ids) - 7]}], "end": []})
    for k in range(6):
        steps.append({"step": 60 + k, "entries": [{"id": rid, "tokens": [ids[len(ids) - 6 + k]], "want": [0]} for rid, ids in requests.items()],
                      "end": list(requests) if k == 5 else []})

    calls = []
    flat = ops.attention_decode_flat
    got = {}
    for dtype, graphs in (("float32", False), ("bfloat16", False), ("bfloat16", True)):
        model, _ = load_model(path, device="cuda", dtype=dtype)
        runner = ModelRunner(model, page_size=16, num_pages=60 * 11, num_slots=64, enforce_eager=not graphs, max_model_len=256)
        calls.clear()
        ops.attention_decode_flat = lambda *a, **k: (calls.append(1), flat(*a, **k))[1]
        try:
            got[dtype, graphs] = replay_in_process(TraceReplayer(runner), steps)
        finally:
            ops.attention_decode_flat = flat
        assert bool(calls) == (dtype == "bfloat16"), "the even-share kernel is the bfloat16 path's, for batches like this one"
        assert not graphs or runner._graphs
    ref = got["float32", False]
    scale = max(float(abs(v).max()) for v in ref.values())
    for key in (("bfloat16", False), ("bfloat16", True)):
        assert len(got[key]) == len(ref) == 60 * 7
        worst = max(float(abs(got[key][k] - ref[k]).max()) for k in ref)
        assert worst < 4e-2 * scale, f"{key}: bfloat16 strays {worst / scale:.3g} from float32"
    ops.check_device_errors()


def _engine(path, model, **kw):
    from tokensprint_b200.config.engine_config import Config
    from tokensprint_b200.engine.llm_engine import LLMEngine

    defaults = dict(model=str(path), max_model_len=256, kvcache_block_size=16, num_kvcache_blocks=64, max_num_batched_tokens=128,
                    max_num_seqs=8, chunked_prefill=True, dtype="bfloat16")
    defaults.update(kw)
    return LLMEngine(model, Config(**defaults))


def test_bfloat16_generation_is_the_same_with_graphs_and_with_overlapping_steps(tmp_path, monkeypatch):
    """bfloat16 through the entry point at Qwen3-0.6B widths (heads of 128: the fused epilogues, the
    decode graphs, tokens fed on the device): {steps overlap, one by one} x {graphs, eager} give the
    same tokens, once with so few pages that a request is preempted and recomputed (requests end by
    count, so all four runs make the same schedule) and once with an end-of-sequence token that is
    really sampled (ends are then seen one step late when steps overlap, and the extra token is
    dropped).  The key splits of the decode attention are pinned: a graph plans them for the longest
    context it may serve, an eager step for the one it has, and a different grouping of partial
    sums rounds differently."""
    from tokensprint_b200.config.engine_config import SamplingParams
    from tokensprint_b200.config.registry import get_preset_dict
    from tokensprint_b200.models.api import load_model
    from tokensprint_b200.models.qwen3 import Qwen3Config
    from tokensprint_b200.weights.loader import write_random_model

    monkeypatch.setenv("TS_DECODE_SPLITS", "2")
    d = get_preset_dict("qwen3-0.6b")
    d["num_hidden_layers"] = 2
    path = write_random_model(tmp_path / "m", Qwen3Config.from_dict(d), seed=9, dtype="bfloat16", std=0.02)
    model, _ = load_model(path, device="cuda", dtype="bfloat16")
    prompts = [random_tokens(d, n, 300 + n) for n in (40, 70, 100, 25)]
    variants = [(overlap, eager) for overlap in (False, True) for eager in (True, False)]

    # 1. a pool of 24 pages: the four requests need 29 at their longest, so one is preempted and recomputed
    sp = SamplingParams(temperature=0.7, max_tokens=48, ignore_eos=True, seed=3)
    runs = {}
    for overlap, eager in variants:
        engine = _engine(path, model, num_kvcache_blocks=24, overlap_steps=overlap, enforce_eager=eager)
        runs[overlap, eager] = engine.generate(prompts, sp, use_tqdm=False)
        assert engine.scheduler.num_preemptions >= 1, "no request was preempted"
        assert eager or engine.model_runner._graphs, "decode steps did not go through a graph"
        assert engine.model_runner.cache_manager.pages_in_use() == 0
    first = runs[False, True]
    assert all(len(c) == 48 for c in first)
    for key, got in runs.items():
        assert got == first, f"overlap={key[0]}, eager={key[1]}: other tokens than steps one by one without graphs"

    # 2. an end-of-sequence token that the second request samples as its tenth token
    roomy = _engine(path, model, overlap_steps=False, enforce_eager=True)
    free_run = roomy.generate(prompts, sp, use_tqdm=False)
    eos = free_run[1][9]
    runs = {}
    for overlap, eager in variants:
        engine = _engine(path, model, eos=eos, overlap_steps=overlap, enforce_eager=eager)
        sps = [SamplingParams(temperature=0.7, max_tokens=48, ignore_eos=(i == 0), seed=3) for i in range(len(prompts))]
        runs[overlap, eager] = engine.generate(prompts, sps, use_tqdm=False)
        assert engine.model_runner.cache_manager.pages_in_use() == 0
    first = runs[False, True]
    assert first[1][-1] == eos and len(first[1]) <= 10, "the request did not end at the end-of-sequence token"
    assert len(first[0]) == 48  # it ignores the token
    for key, got in runs.items():
        assert got == first, f"overlap={key[0]}, eager={key[1]}: other tokens with an end-of-sequence token"
    ops_module = __import__("tokensprint_b200.ops", fromlist=["ops"])
    ops_module.check_device_errors()


def test_full_depth_bfloat16_against_float32_and_the_plain_model():
    """All 36 layers of Qwen3-8B with random weights, one 256-token request: bfloat16 whole and with
    its last 32 tokens decoded one by one (eager and in graphs), against the engine's float32 path
    and against the plain model.  Errors of bfloat16 grow with depth: at 36 layers 8-bit mantissas
    alone (the plain model with every matrix and every handed-on activation rounded) move these
    logits by 4e-2 of the largest, which is the whole bound of the two-layer tests.  So the
    yardstick is measured here, on the same model and input: the engine may stray from the exact
    logits 1.5 times as far as that rounded plain model does at its worst entry, and 1.25 times as
    far on average (the engine rounds in fewer places; a wrong key, page or row shows as a
    multiple).  The weights are drawn here, on the device (a folder
    of 16 GB would take the test's time), and handed to the engine and to the plain model alike."""
    from tokensprint_b200.config.registry import get_model_config
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.engine.runner import ModelRunner
    from tokensprint_b200.models.api import build_model
    from tokensprint_b200.weights.loader import WeightSource

    cfg = get_model_config("qwen3-8b")
    d = cfg.to_dict()
    gen = torch.Generator(device="cuda").manual_seed(12)
    weights = {}
    for spec in build_model(cfg, device="cuda", dtype="bfloat16").tensor_specs():
        x = torch.randn(spec.shape, generator=gen, device="cuda", dtype=torch.float32)
        weights[spec.name] = (1.0 + 0.05 * x if len(spec.shape) == 1 else 0.02 * x).to(torch.bfloat16)

    class FromDict(WeightSource):
        where = "weights drawn by the test"

        def shapes(self):
            return {n: tuple(t.shape) for n, t in weights.items()}

        def fetch(self, spec, device, compute_dtype):
            return weights[spec.name].to(device=device, dtype=torch.float32 if spec.role == "vector" else compute_dtype).contiguous()

    ids = random_tokens(d, 256, 77)
    requests = {"a": ids}
    want = plain.forward_logits(weights, d, ids, dtype=torch.float32, device="cuda").double().cpu().numpy()
    scale = float(abs(want).max())
    # How far 8-bit mantissas alone move these logits at this depth: the plain model with every
    # matrix and every activation between two operations rounded to bfloat16 (its `rounding` hook).
    rounded = plain.forward_logits(weights, d, ids, dtype=torch.float32, device="cuda", rounding=plain.round_to_bfloat16).double().cpu().numpy()
    noise = float(abs(rounded - want).max()) / scale
    mean_noise = float(abs(rounded - want).mean()) / scale
    assert 1e-3 < noise < 0.1, f"the yardstick itself is off: rounding alone moves the logits by {noise:.3g}"

    def run(dtype, steps, graphs=False):
        model = build_model(cfg, device="cuda", dtype=dtype)
        model.load(FromDict())
        runner = ModelRunner(model, page_size=16, num_pages=32, num_slots=4, enforce_eager=not graphs, max_model_len=512)
        got = replay_in_process(TraceReplayer(runner), steps)
        assert not graphs or runner._graphs
        del runner, model
        torch.cuda.empty_cache()
        return got

    def worst(got):
        return max(float(abs(got[("a", pos)].astype("float64") - want[pos]).max()) for pos in range(len(ids))) / scale

    exact = run("float32", trace_whole(requests))
    assert worst(exact) < 2e-4, f"float32 engine strays {worst(exact):.3g} from the plain model (float32 arithmetic on both sides)"
    for name, steps, graphs in (("whole", trace_whole(requests), False), ("tail", trace_decode_tail(requests), False),
                                ("tail in graphs", trace_decode_tail(requests), True)):
        got = run("bfloat16", steps, graphs)
        assert len(got) == len(ids)
        assert worst(got) < 1.5 * noise, f"{name}: bfloat16 strays {worst(got):.3g} from the plain model at full depth (rounding alone: {noise:.3g})"
        mean = sum(float(abs(got[("a", pos)].astype("float64") - want[pos]).mean()) for pos in range(len(ids))) / len(ids) / scale
        assert mean < 1.25 * mean_noise, f"{name}: bfloat16 strays {mean:.3g} on average (rounding alone: {mean_noise:.3g})"
        err = max(float(abs(got[k] - exact[k]).max()) for k in exact) / scale
        assert err < 1.5 * noise, f"{name}: bfloat16 strays {err:.3g} from float32 at full depth"


def test_many_requests_through_a_tight_pool_all_finish_and_every_page_comes_back(tmp_path):
    """A serving loop in small: 48 requests of mixed lengths at Qwen3-0.6B widths through `generate`,
    bfloat16, graphs and overlapping steps on, chunked prefill under a small token budget, and a pool
    that holds a third of what they need at their longest, so requests are preempted and recomputed
    all the time.  Every request gets exactly the tokens it asked for, the same ones as with room for
    all wherever no preemption touched it, and no page or slot is lost."""
    import random

    from tokensprint_b200 import ops
    from tokensprint_b200.config.engine_config import SamplingParams
    from tokensprint_b200.config.registry import get_preset_dict
    from tokensprint_b200.models.api import load_model
    from tokensprint_b200.models.qwen3 import Qwen3Config
    from tokensprint_b200.weights.loader import write_random_model

    d = get_preset_dict("qwen3-0.6b")
    d["num_hidden_layers"] = 2
    path = write_random_model(tmp_path / "m", Qwen3Config.from_dict(d), seed=21, dtype="bfloat16", std=0.02)
    model, _ = load_model(path, device="cuda", dtype="bfloat16")
    rng = random.Random(5)
    prompts = [random_tokens(d, rng.randint(10, 300), 900 + i) for i in range(48)]
    sps = [SamplingParams(temperature=0.8, max_tokens=rng.randint(5, 60), ignore_eos=True, seed=9) for _ in prompts]
    longest = sum(-(-(len(p) + sp.max_tokens) // 16) for p, sp in zip(prompts, sps))

    roomy = _engine(path, model, num_kvcache_blocks=longest + 8, max_num_seqs=48, max_num_batched_tokens=256, max_model_len=512)
    want = roomy.generate(prompts, sps, use_tqdm=False)
    assert roomy.scheduler.num_preemptions == 0

    tight = _engine(path, model, num_kvcache_blocks=longest // 3, max_num_seqs=48, max_num_batched_tokens=256, max_model_len=512)
    got = tight.generate(prompts, sps, use_tqdm=False)
    assert tight.scheduler.num_preemptions >= 5, "the pool was not tight enough to preempt"
    assert [len(c) for c in got] == [sp.max_tokens for sp in sps]
    cm = tight.model_runner.cache_manager
    cm.check_invariants()
    assert cm.pages_in_use() == 0 and len(cm.free_slots) == cm.num_slots
    # a recomputed request runs its tokens through the prompt kernels instead of the decode kernels:
    # other rounding, so its continuation may differ; most requests keep every token all the same
    same = sum(a == b for a, b in zip(got, want))
    assert same >= len(prompts) // 2, f"only {same} of {len(prompts)} requests kept their tokens under preemption"
    # the first token depends on the prompt alone (and on how it was cut into portions: rounding)
    first_tokens = sum(a[0] == b[0] for a, b in zip(got, want))
    assert first_tokens >= len(prompts) - 4, f"{len(prompts) - first_tokens} first tokens changed under preemption"
    ops.check_device_errors()


def test_a_long_request_in_portions_and_decoded_against_the_plain_model(tmp_path):
    """5,000 tokens at Qwen3-0.6B widths: the prompt in portions of 2,048 (the later portions attend
    over thousands of cached keys), then 24 tokens one by one (key splits over a long context), eager
    and in graphs.  bfloat16 against the plain model on the device at every wanted position: the last
    rows of every portion and all decoded tokens."""
    from tokensprint_b200.config.registry import get_preset_dict
    from tokensprint_b200.models.qwen3 import Qwen3Config
    from tokensprint_b200.weights.loader import write_random_model
    from tokensprint_b200.weights.safetensors_io import SafetensorsFolder

    d = get_preset_dict("qwen3-0.6b")
    d["num_hidden_layers"] = 2
    path = write_random_model(tmp_path / "m", Qwen3Config.from_dict(d), seed=31, dtype="bfloat16", std=0.02)
    ids = random_tokens(d, 5000, 41)
    files = SafetensorsFolder(path)
    weights = {n: files.tensor(n) for n in files.keys()}
    want = plain.forward_logits(weights, d, ids, dtype=torch.float64, device="cuda").cpu().numpy()
    del weights
    torch.cuda.empty_cache()
    scale = float(abs(want).max())

    steps, pos = [], 0
    for size in (2048, 2048, 880):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": ids[pos : pos + size], "want": list(range(size - 8, size))}], "end": []})
        pos += size
    for t in range(pos, len(ids)):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [ids[t]], "want": [0]}], "end": ["a"] if t == len(ids) - 1 else []})
    wanted = [p for base, size in ((0, 2048), (2048, 2048), (4096, 880)) for p in range(base + size - 8, base + size)] + list(range(4976, 5000))

    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.engine.runner import ModelRunner
    from tokensprint_b200.models.api import load_model

    for graphs in (False, True):
        model, _ = load_model(path, device="cuda", dtype="bfloat16")
        runner = ModelRunner(model, page_size=16, num_pages=320, num_slots=4, enforce_eager=not graphs, max_model_len=5120,
                             max_num_batched_tokens=2048)
        got = replay_in_process(TraceReplayer(runner), steps)
        assert sorted(p for _, p in got) == wanted
        assert not graphs or runner._graphs
        for p in wanted:
            err = float(abs(got[("a", p)].astype("float64") - want[p]).max()) / scale
            assert err < 4e-2, f"graphs={graphs}: position {p} strays {err:.3g} from the plain model"


def test_decoded_tokens_beside_portions_go_to_their_own_kernels(folder, monkeypatch):
    """One step with portions of two prompts and single decoded tokens of two other requests, given
    in turns: the runner puts the single tokens' requests first, the attention sends them to the
    decode kernel and the portions to the prompt kernel (two sequences each), and every wanted row
    comes back in the order of the entries, equal to the plain model's."""
    from tokensprint_b200 import ops
    from tokensprint_b200.weights.safetensors_io import SafetensorsFolder

    path, cfg = folder
    requests = {"a": random_tokens(cfg, 41, 11), "b": random_tokens(cfg, 50, 12), "c": random_tokens(cfg, 71, 13), "d": random_tokens(cfg, 33, 14)}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": requests["a"][:40], "want": []}, {"id": "c", "tokens": requests["c"][:70], "want": [69]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": requests["b"], "want": [10, 49]}, {"id": "a", "tokens": requests["a"][40:], "want": [0]},
                                {"id": "d", "tokens": requests["d"], "want": [0, 32]}, {"id": "c", "tokens": requests["c"][70:], "want": [0]}],
         "end": ["a", "b", "c", "d"]},
    ]
    calls = []
    prompt_kernel = ops.attention_prefill_tcgen05

    def spy(q, k, v, out, cu, lens, table, page, num_seqs, max_q, *rest):
        calls.append((int(num_seqs), int(max_q), q.shape[0]))
        return prompt_kernel(q, k, v, out, cu, lens, table, page, num_seqs, max_q, *rest)

    monkeypatch.setattr(ops, "attention_prefill_tcgen05", spy)
    got = _logits(path, "bfloat16", steps)
    layers = cfg["num_hidden_layers"]
    assert calls[:layers] == [(2, 70, 110)] * layers  # step 0: two portions
    assert calls[layers:] == [(2, 50, 85)] * layers    # step 1: the two portions of the four requests; q holds all 85 tokens

    files = SafetensorsFolder(path)
    weights = {n: files.tensor(n) for n in files.keys()}
    wanted = {("c", 69), ("b", 10), ("b", 49), ("a", 40), ("d", 0), ("d", 32), ("c", 70)}
    assert set(got) == wanted
    for rid in requests:
        logits = plain.forward_logits(weights, cfg, requests[rid], dtype=torch.float64, device="cuda").cpu().numpy()
        scale = float(abs(logits).max())
        for r, pos in wanted:
            if r == rid:
                err = float(abs(got[(r, pos)].astype("float64") - logits[pos]).max()) / scale
                assert err < 4e-2, f"request {r} position {pos} strays {err:.3g} from the plain model"
