"""Qwen3-8B layer sizes (two layers, so it is quick): the bfloat16 kernels at the widths that
serving uses — head size 128, four query heads per KV head, width 4096, vocabulary 151936 —
under several cuttings, against the float32 path, and the float32 path against the plain model."""

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.replay_helpers import random_tokens, replay_in_process, trace_decode_tail, trace_mixed, trace_portions, trace_whole

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["qwen3-8b", "qwen3-32b", "qwen3-0.6b"])
def folder(request, tmp_path_factory):
    """8B: four query heads per KV head; 32B: eight, width 5120, intermediate 25600; 0.6B: two,
    width 1024 with heads of 128 (heads * head size is twice the width) and a tied head."""
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

    # float32 engine against the plain model on the CPU (a short request: the head is 151936 wide)
    from tokensprint_b200.weights.safetensors_io import SafetensorsFolder

    files = SafetensorsFolder(path)
    weights = {n: files.tensor(n) for n in files.keys()}
    want = plain.forward_logits(weights, cfg, requests["c"], dtype=torch.float64).numpy()
    for pos in range(len(requests["c"])):
        assert abs(ref[("c", pos)] - want[pos]).max() < 1e-4 * abs(want).max()

    # bfloat16 in every cutting, eager and in graphs, against float32
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
