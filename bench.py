"""Decode and prefill throughput of the engine on one B200: Qwen3-8B sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload cb14b|long32b [--impl ours|reference]

Prints ONE JSON line.  A "step" is one decode step of a batch of 8 requests (1,024-token
random prompts, context limit 4,096, cache pages of 16 tokens).  `value` is decoded tokens
a second, timed on the device with CUDA events around K steps after W warm-up steps;
`e2e` is the same through `LLMEngine.add_request/step` with host token ids in and sampled
ids out every step, timed with the wall clock in blocks of K steps until at least a second
has been timed (the median block is printed).  `prefill` is one 2,048-token prompt through
`LLMEngine.generate(max_tokens=1)`: `ms` with CUDA events around the call, `e2e_ms` with the
wall clock, in both arms the same way.  `roofline` compares the decode step's bytes (every
weight once, the cache of the live requests) with the HBM peak; `points` adds decode at batch
1 and 64 and, for all three batch sizes, steps that end at a context of 1,536 tokens.  The
weights (16 GB) are far larger than the L2, so no flush is needed between steps.  More than
one GPU is not supported.

`--workload` measures serving loops through `LLMEngine.generate` instead (one JSON line each):
`cb14b`: Qwen3-14B sizes, 256 requests with prompts of U[64, 2048] and outputs of U[64, 1024]
tokens, continuous batching with chunked prefill under a budget of 8,192 tokens a step;
`long32b`: Qwen3-32B sizes, 16 prompts of 16,384 tokens and 256 decoded tokens each.  The cache
pool takes what is free on the device.  The line gives generated tokens a second over the whole
run, and per kind of step (decode / mixed / prefill) the count, the host's time to schedule and
launch it and the device's time.
"""

from __future__ import annotations

import argparse
import json
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
MODEL_NAME = "qwen/qwen3-8b"
PROMPT_LEN = 1024
PREFILL_TOKENS = 2048
CONTEXT_LEN = 4096
PAGE_SIZE = 16
LAST_CONTEXT = 1536  # 1,024-token prompts with 512 generated tokens end here
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            d = json.loads(path.read_text())
            out = {"source": "measured"}
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if key in d:
                    out[key] = float(d[key])
            if "hbm_gbs" in out and "bf16_tflops" in out:
                return out
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while a timed region runs."""

    REASONS = {
        0x8: "hw_slowdown",
        0x40: "hw_thermal_slowdown",
        0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int = 0, period: float = 0.01) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self.period = period
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                self.samples.append(int(self._nvml.nvmlDeviceGetClockInfo(self._handle, self._nvml.NVML_CLOCK_SM)))
                mask = int(self._nvml.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nvml is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def summary(self) -> dict:
        s = sorted(self.samples)
        return {
            "sm_mhz": s[len(s) // 2] if s else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(s),
        }


def prefill_flops(cfg, T: int) -> float:
    """GEMM flops of T tokens through every layer, causal attention over T keys, head for one row."""
    H, I, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nq, nkv, L = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.num_hidden_layers
    per_token = 2 * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    attention = 4 * nq * d * (T * (T + 1) / 2)
    return L * (per_token * T + attention) + 2 * H * cfg.vocab_size


def random_ids(n: int, vocab: int, seed: int) -> list[int]:
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def measure_decode(runner, cfg, batch: int, steps: int, warmup: int, clocks=None, prompt_len: int = PROMPT_LEN):
    """Device-timed decode: `batch` requests prefilled with `prompt_len` tokens, then
    warmup + steps single-token steps with sampling.  Returns (ms per step, mean context, launches)."""
    import torch

    from tokensprint_b200 import ops
    from tokensprint_b200.engine.runner import StepEntry

    cm = runner.cache_manager
    vocab = cfg.vocab_size
    reqs = []
    for b in range(batch):
        rc = cm.admit(("bench", batch, b))
        reqs.append(rc)
    per_step = max(1, 8192 // prompt_len)
    for i in range(0, batch, per_step):
        entries = []
        for b in range(i, min(batch, i + per_step)):
            cm.extend(reqs[b], 0, prompt_len)
            entries.append(StepEntry(reqs[b], random_ids(prompt_len, vocab, 100 + b), 0, []))
        runner.step(entries)
    temps = torch.full((batch,), 0.6, dtype=torch.float32, device=runner.device)
    keys = torch.arange(batch, dtype=torch.int64, device=runner.device)
    sampled = torch.empty(batch, dtype=torch.int32, device=runner.device)
    next_tokens = [random_ids(warmup + steps, vocab, 500 + b) for b in range(batch)]

    def one_step(i: int) -> None:
        pos = prompt_len + i
        entries = []
        for b in range(batch):
            cm.extend(reqs[b], pos, pos + 1)
            entries.append(StepEntry(reqs[b], [next_tokens[b][i]], pos, [0]))
        logits = runner.step(entries)
        ops.sample(logits, temps, keys, sampled)

    for i in range(warmup):
        one_step(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ops.launch_count + getattr(runner, "graph_launches", 0)
    if clocks is not None:
        clocks.__enter__()
    start.record()
    for i in range(warmup, warmup + steps):
        one_step(i)
    end.record()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.__exit__()
    launches = ops.launch_count + getattr(runner, "graph_launches", 0) - launches0
    ms = start.elapsed_time(end) / steps
    mean_ctx = prompt_len + warmup + (steps - 1) / 2 + 1
    for rc in reqs:
        runner.free(rc)
    return ms, mean_ctx, launches


def measure_prefill_step(runner, cfg, reps: int = 5):
    """One 2,048-token prompt as one call of the step function, CUDA events around it."""
    import torch

    from tokensprint_b200.engine.runner import StepEntry

    cm = runner.cache_manager
    times = []
    for r in range(reps + 2):
        rc = cm.admit(("prefill", r))
        cm.extend(rc, 0, PREFILL_TOKENS)
        entry = StepEntry(rc, random_ids(PREFILL_TOKENS, cfg.vocab_size, 900 + r), 0, [PREFILL_TOKENS - 1])
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([entry])
        end.record()
        torch.cuda.synchronize()
        if r >= 2:
            times.append(start.elapsed_time(end))
        runner.free(rc)
    times.sort()
    return times[len(times) // 2]


def time_generate_one_token(generate, vocab: int, reps: int = 5):
    """A 2,048-token prompt and one generated token through an engine's `generate`: the median of
    the device's time (CUDA events around the call) and of the wall clock's, the same for both arms."""
    import torch

    device_ms, wall_ms = [], []
    for r in range(reps + 2):
        ids = random_ids(PREFILL_TOKENS, vocab, 900 + r)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        generate(ids)
        end.record()
        torch.cuda.synchronize()
        if r >= 2:
            wall_ms.append((time.perf_counter() - t0) * 1e3)
            device_ms.append(start.elapsed_time(end))
    device_ms.sort()
    wall_ms.sort()
    return device_ms[len(device_ms) // 2], wall_ms[len(wall_ms) // 2]


E2E_MIN_SECONDS = 1.0


def measure_e2e(model, cfg, batch: int, steps: int, warmup: int, eager: bool = False, ms_hint: float = 4.0):
    """Decode through the public entry point: LLMEngine.add_request + step(), token ids from
    host lists, sampled ids back on the host every step.  Blocks of `steps` steps are timed with
    the wall clock until at least E2E_MIN_SECONDS have been timed; the median block counts.  Also
    the 2,048-token prompt through generate(max_tokens=1)."""
    import torch

    from tokensprint_b200.config.engine_config import Config, SamplingParams
    from tokensprint_b200.engine.llm_engine import LLMEngine

    blocks = max(3, int(E2E_MIN_SECONDS / (steps * ms_hint * 1e-3)) + 2)
    blocks = min(blocks, max(3, (CONTEXT_LEN - PROMPT_LEN - warmup - 32) // steps))
    total = warmup + blocks * steps
    pages = batch * (-(-(PROMPT_LEN + total + 8) // PAGE_SIZE)) + PREFILL_TOKENS // PAGE_SIZE + 64
    config = Config(model=str(ROOT), max_model_len=CONTEXT_LEN, max_num_seqs=max(batch, 8), max_num_batched_tokens=8192,
                    kvcache_block_size=PAGE_SIZE, num_kvcache_blocks=pages, chunked_prefill=True, dtype="bfloat16",
                    enforce_eager=eager)
    engine = LLMEngine(model, config)
    one = SamplingParams(temperature=0.6, max_tokens=1, ignore_eos=True, seed=1)
    pf_ms, pf_wall_ms = time_generate_one_token(lambda ids: engine.generate([ids], one, use_tqdm=False), cfg.vocab_size)

    sp = SamplingParams(temperature=0.6, max_tokens=total + 4, ignore_eos=True, seed=1)
    for b in range(batch):
        engine.add_request(random_ids(PROMPT_LEN, cfg.vocab_size, 300 + b), sp)
    while any(s.num_cached_tokens < s.num_prompt_tokens for s in list(engine.scheduler.running) + list(engine.scheduler.waiting)) or engine.scheduler.waiting:
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    runner = engine.model_runner
    h2d0 = runner.h2d_bytes
    times = []
    for _ in range(blocks):
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    h2d = (runner.h2d_bytes - h2d0) / (blocks * steps) + batch * 12  # + temperatures (4 B) and keys (8 B) per row
    for seq in list(engine.scheduler.running):
        engine.scheduler.abort(seq)
    del engine
    times.sort()
    median = times[len(times) // 2]
    return {"value": batch * steps / median, "h2d": int(h2d), "d2h": batch * 4, "blocks": blocks, "timed_s": sum(times),
            "prefill_ms": pf_ms, "prefill_wall_ms": pf_wall_ms}


def run_ours(args) -> dict:
    import torch

    from tokensprint_b200.config.registry import get_model_config, get_preset_dict
    from tokensprint_b200.models.qwen3 import Qwen3Config
    from tokensprint_b200.engine.runner import ModelRunner
    from tokensprint_b200.models.api import random_model

    torch.cuda.set_device(0)
    peaks = load_peaks()
    full_cfg = get_model_config(MODEL_NAME)
    cfg = full_cfg
    if args.layers and args.layers < full_cfg.num_hidden_layers:
        d = get_preset_dict(MODEL_NAME)
        d["num_hidden_layers"] = args.layers
        cfg = Qwen3Config.from_dict(d)
    model = random_model(cfg, seed=0, dtype="bfloat16", generate_on_device=True)
    torch.cuda.synchronize()

    max_batch = 64 if not args.skip_points else args.batch
    tokens_per_req = max(PROMPT_LEN + args.warmup + max(args.steps, 32), LAST_CONTEXT) + 16
    pages = max_batch * (-(-tokens_per_req // PAGE_SIZE)) + PREFILL_TOKENS // PAGE_SIZE + 64
    runner = ModelRunner(model, page_size=PAGE_SIZE, num_pages=pages, num_slots=max_batch + 8,
                         max_num_batched_tokens=8192, enforce_eager=args.eager, max_model_len=CONTEXT_LEN)

    clocks = ClockSampler()
    ms, mean_ctx, launches = measure_decode(runner, cfg, args.batch, args.steps, args.warmup, clocks)
    value = args.batch * 1000.0 / ms

    kv_bytes_per_token = sum(runner.page_bytes) / PAGE_SIZE
    step_bytes = model.weight_bytes() + args.batch * mean_ctx * kv_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    points = {}
    if not args.skip_points:
        short = (min(args.steps, 32), min(args.warmup, 4))
        for b in (1, 64):
            pms, _, _ = measure_decode(runner, cfg, b, *short)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
        # the workload's last steps: 1,024-token prompts with 512 generated tokens end at a context of 1,536
        for b in (1, 8, 64):
            pms, _, _ = measure_decode(runner, cfg, b, *short, prompt_len=LAST_CONTEXT - sum(short))
            points[f"decode_b{b}_ctx{LAST_CONTEXT}"] = round(b * 1000.0 / pms, 1)

    pf_step_ms = measure_prefill_step(runner, cfg)
    pf_flops = prefill_flops(cfg, PREFILL_TOKENS)

    del runner
    torch.cuda.empty_cache()
    e2e = measure_e2e(model, cfg, args.batch, args.steps, args.warmup, args.eager, ms_hint=ms)
    pf_ms = e2e["prefill_ms"]
    pf_frac = pf_flops / (pf_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)

    return {
        "metric": "decode tokens/s, Qwen3-8B sizes, batch 8, 1 B200",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), uniform-random token ids",
        "impl": "ours",
        "config": {
            "model": "qwen3-8b",
            "layers": cfg.num_hidden_layers,
            "layers_full": full_cfg.num_hidden_layers,
            "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size,
            "vocab": cfg.vocab_size,
            "global_batch": args.batch,
            "prompt_len": PROMPT_LEN,
            "seq_len": CONTEXT_LEN,
            "kv_block": PAGE_SIZE,
            "parallelism": "single GPU",
            "l2": "inputs larger than L2 (16 GB of weights per step)",
            "peaks": peaks["source"],
        },
        "clocks": clocks.summary(),
        "e2e": {"value": round(e2e["value"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                "blocks": e2e["blocks"], "timed_s": round(e2e["timed_s"], 3)},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3), "frac": round(pf_frac, 4),
                    "e2e_ms": round(e2e["prefill_wall_ms"], 3), "step_ms": round(pf_step_ms, 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
    }


def run_probe(args) -> int:
    """A few steps between cudaProfilerStart/Stop, for `ncu --profile-from-start off`: the
    8B layer sizes with `--layers` layers (small enough for a full-metric capture), decode at
    `--batch` requests of 1,024 cached tokens, or one 2,048-token prefill.  Prints `ok`."""
    import torch

    from tokensprint_b200 import ops
    from tokensprint_b200.models.qwen3 import Qwen3Config
    from tokensprint_b200.config.registry import get_preset_dict
    from tokensprint_b200.engine.runner import ModelRunner, StepEntry
    from tokensprint_b200.models.api import random_model

    d = get_preset_dict(MODEL_NAME)
    d["num_hidden_layers"] = args.layers or 4
    cfg = Qwen3Config.from_dict(d)
    model = random_model(cfg, seed=0, dtype="bfloat16", generate_on_device=True)
    batch = args.batch
    runner = ModelRunner(model, page_size=PAGE_SIZE, num_pages=batch * 80 + 400, num_slots=batch + 2,
                         enforce_eager=True, max_model_len=CONTEXT_LEN)
    cm = runner.cache_manager
    if args.probe == "decode":
        reqs = [cm.admit(b) for b in range(batch)]
        for b in range(batch):
            cm.extend(reqs[b], 0, PROMPT_LEN)
            runner.step([StepEntry(reqs[b], random_ids(PROMPT_LEN, cfg.vocab_size, b), 0, [])])
        temps = torch.full((batch,), 0.6, device="cuda")
        keys = torch.arange(batch, dtype=torch.int64, device="cuda")
        out = torch.empty(batch, dtype=torch.int32, device="cuda")

        def step(i: int) -> None:
            entries = []
            for b in range(batch):
                cm.extend(reqs[b], PROMPT_LEN + i, PROMPT_LEN + i + 1)
                entries.append(StepEntry(reqs[b], [7 + b], PROMPT_LEN + i, [0]))
            ops.sample(runner.step(entries), temps, keys, out)

        for i in range(3):
            step(i)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for i in range(3, 5):
            step(i)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    else:
        def prefill(r: int) -> None:
            rc = cm.admit(("p", r))
            cm.extend(rc, 0, PREFILL_TOKENS)
            runner.step([StepEntry(rc, random_ids(PREFILL_TOKENS, cfg.vocab_size, r), 0, [PREFILL_TOKENS - 1])])
            runner.free(rc)

        prefill(0)
        prefill(1)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        prefill(2)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    print("ok")
    return 0


def run_reference(args) -> dict:
    """The unmodified reference (installed under baseline/_ref) through its own public API:
    build_model for the same sizes, random weights, LLMEngine.add_request/step/generate.  The
    reference cannot load a checkpoint here (its loader downloads from a hub and there is no
    network), so the model object comes from its own builder and is filled with random values."""
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "engine").is_dir():
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref"}
    try:
        sys.path.insert(0, str(ref_root))
        return _reference_workload(args) if args.workload else _reference_decode(args)
    except Exception as e:  # an import or launch error of the reference's stack on this box
        reason = f"{type(e).__name__}: {e}".replace("\n", " ")[:300]
        return {"impl": "reference", "unavailable": f"the reference failed to run on this box: {reason}"}


def reference_model(cfg, max_seq_len: int):
    """The reference's own model object for a typed config of this repo, with random parameters."""
    import torch
    from engine.models import build_model
    from engine.models.qwen._archs import QwenModelConfig
    from engine.nn.attention import AttentionConfig
    from engine.nn.layers import FFNConfig
    from engine.utils import reset_non_persistent_buffers

    device = torch.device("cuda")
    ref_cfg = QwenModelConfig(
        attn_config=AttentionConfig(model_dim=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                                    num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, qk_norm=True,
                                    qk_norm_eps=cfg.rms_norm_eps),
        ffn_config=FFNConfig(model_dim=cfg.hidden_size, inner_dim=cfg.intermediate_size),
        vocab_dim=cfg.vocab_size, num_layers=cfg.num_hidden_layers, max_seq_len=max_seq_len, rope_theta=cfg.rope_theta,
        rope_impl="triton", norm_eps=cfg.rms_norm_eps, rmsnorm_impl="triton", tie_weights=cfg.tie_word_embeddings)
    with torch.inference_mode():
        model = build_model(ref_cfg, device=device, dtype=torch.bfloat16)
        g = torch.Generator(device=device).manual_seed(0)
        for name, p in model.named_parameters():
            if p.dim() == 1:
                p.fill_(0.0 if name.endswith("bias") else 1.0)
            else:
                p.normal_(0.0, 0.02, generator=g)
        reset_non_persistent_buffers(model)
    return model


def _reference_decode(args) -> dict:
    import tempfile

    import torch
    from engine.generation.config import Config as RefConfig
    from engine.generation.config import SamplingParams as RefSamplingParams
    from engine.generation.llm_engine import LLMEngine as RefEngine

    from tokensprint_b200.config.registry import get_model_config

    cfg = get_model_config(MODEL_NAME)
    peaks = load_peaks()
    model = reference_model(cfg, CONTEXT_LEN)
    batch, steps, warmup = args.batch, args.steps, args.warmup
    blocks = max(3, int(E2E_MIN_SECONDS / (steps * 7.5e-3)) + 2)
    blocks = min(blocks, max(3, (CONTEXT_LEN - PROMPT_LEN - warmup - 32) // steps - 1))
    with torch.inference_mode(), tempfile.TemporaryDirectory() as model_dir:
        # its paged attention wants cache blocks of 256 tokens (engine/generation/config.py:38-42)
        config = RefConfig(model=model_dir, max_model_len=CONTEXT_LEN, max_num_seqs=max(batch, 8), max_num_batched_tokens=8192,
                           kvcache_block_size=256, chunked_prefill=True, eos=-1, dtype=torch.bfloat16, gpu_memory_utilization=0.5)
        engine = RefEngine(model=model, config=config, tokenizer=None)
        sp = RefSamplingParams(temperature=0.6, max_tokens=warmup + (blocks + 1) * steps + 4, ignore_eos=True)
        for b in range(batch):
            engine.add_request(random_ids(PROMPT_LEN, cfg.vocab_size, 300 + b), sp)
        sched = engine.scheduler
        while sched.waiting or any(s.num_cached_tokens < s.num_prompt_tokens for s in sched.running):
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        clocks = ClockSampler()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with clocks:  # the device-timed K steps
            start.record()
            for _ in range(steps):
                engine.step()
            end.record()
            torch.cuda.synchronize()
        ms = start.elapsed_time(end) / steps
        walls = []  # the same loop by the wall clock, in blocks, until a second has been timed
        for _ in range(blocks):
            t0 = time.perf_counter()
            for _ in range(steps):
                engine.step()
            torch.cuda.synchronize()
            walls.append(time.perf_counter() - t0)
        walls.sort()
        wall = walls[len(walls) // 2]
        while not engine.is_finished():
            engine.step()
        # prefill: one 2,048-token prompt, one generated token, timed as in the other arm
        one = RefSamplingParams(temperature=0.6, max_tokens=1, ignore_eos=True)
        pf_ms, pf_wall_ms = time_generate_one_token(lambda ids: engine.generate([ids], one, use_tqdm=False), cfg.vocab_size)
    # what its stock step copies for B single tokens (engine/generation/model_runner.py:101-201): ids and
    # positions as int64, slot mapping, context lengths, two cu_seqlens, the rows that want logits (int64),
    # temperatures, and block tables of ceil(context / 256) entries; back come ids and rows as int64
    blocks_per_seq = -(-(PROMPT_LEN + warmup + steps) // 256)
    h2d = batch * (8 + 8 + 4 + 4 + 8 + 4) + 2 * (batch + 1) * 4 + batch * blocks_per_seq * 4
    value = batch * 1000.0 / ms
    return {
        "metric": "decode tokens/s, Qwen3-8B sizes, batch 8, 1 B200",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02) in the reference's own model object, uniform-random token ids",
        "impl": "reference",
        "config": {"model": "qwen3-8b", "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size, "global_batch": batch,
                   "prompt_len": PROMPT_LEN, "seq_len": CONTEXT_LEN, "kv_block": 256, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (16 GB of weights per step)", "peaks": peaks["source"]},
        "clocks": clocks.summary(),
        "e2e": {"value": round(batch * steps / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": batch * 16,
                "blocks": blocks, "timed_s": round(sum(walls), 3)},
        "gpu_launches": 0,
        "prefill": {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
                    "frac": round(prefill_flops(cfg, PREFILL_TOKENS) / (pf_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
                    "e2e_ms": round(pf_wall_ms, 3)},
    }


# ---------------------------------------------------------------------------
# serving loops through generate()

WORKLOADS = {
    # 256 requests under continuous batching with chunked prefill (the reference's own harness is such a
    # workload: benchmark.py:23-40,54-63,99-152 of the reference)
    "cb14b": {"model": "qwen/qwen3-14b", "requests": 256, "prompt": (64, 2048), "output": (64, 1024), "budget": 8192,
              "max_seqs": 256, "max_model_len": 4096, "what": "continuous batching, chunked prefill"},
    # long prompts: the cache pool is what the weights leave of the device's memory
    "long32b": {"model": "qwen/qwen3-32b", "requests": 16, "prompt": (16384, 16384), "output": (256, 256), "budget": 8192,
                "max_seqs": 16, "max_model_len": 16384 + 256 + 16, "what": "long context, chunked prefill"},
}


def workload_requests(w: dict, vocab: int, seed: int = 0):
    """Prompts (uniform-random ids) and output lengths of a workload, the same in both arms."""
    import random

    rng = random.Random(seed)
    prompts, outputs = [], []
    for i in range(w["requests"]):
        n = rng.randint(*w["prompt"])
        prompts.append(random_ids(n, vocab, 7000 + i))
        outputs.append(rng.randint(*w["output"]))
    return prompts, outputs


def workload_record(args, w: dict, cfg, impl: str, prompts, outputs, wall: float, generated: int, extra: dict) -> dict:
    record = {
        "workload": args.workload, "impl": impl,
        "metric": f"generated tokens/s, {w['model'].split('/')[-1]} sizes, {w['requests']} requests, {w['what']}, 1 B200",
        "value": round(generated / wall, 1), "unit": "tokens/s", "higher_is_better": True, "n_gpus": 1, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform-random token ids",
        "requests": len(prompts), "prompt_tokens": sum(len(p) for p in prompts), "output_tokens": generated,
        "wall_s": round(wall, 3), "all_tokens_per_s": round((sum(len(p) for p in prompts) + generated) / wall, 1),
        "config": {"model": w["model"].split("/")[-1], "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "max_num_batched_tokens": w["budget"],
                   "max_num_seqs": w["max_seqs"], "max_model_len": w["max_model_len"],
                   "prompt_len": f"U[{w['prompt'][0]},{w['prompt'][1]}]", "output_len": f"U[{w['output'][0]},{w['output'][1]}]"},
    }
    assert generated == sum(outputs), f"{generated} tokens came back, {sum(outputs)} were asked for"
    record.update(extra)
    return record


def run_workload(args) -> dict:
    """A serving loop through this engine's `LLMEngine.generate`, the cache pool sized from free memory."""
    import torch

    from tokensprint_b200.config.engine_config import Config, SamplingParams
    from tokensprint_b200.config.registry import get_model_config, get_preset_dict
    from tokensprint_b200.engine.llm_engine import LLMEngine
    from tokensprint_b200.models.api import random_model
    from tokensprint_b200.models.qwen3 import Qwen3Config

    torch.cuda.set_device(0)
    w = WORKLOADS[args.workload]
    cfg = full_cfg = get_model_config(w["model"])
    if args.layers and args.layers < full_cfg.num_hidden_layers:
        d = get_preset_dict(w["model"])
        d["num_hidden_layers"] = args.layers
        cfg = Qwen3Config.from_dict(d)
    model = random_model(cfg, seed=0, dtype="bfloat16", generate_on_device=True)
    config = Config(model=str(ROOT), max_model_len=w["max_model_len"], max_num_seqs=w["max_seqs"], max_num_batched_tokens=w["budget"],
                    kvcache_block_size=PAGE_SIZE, num_kvcache_blocks=-1, gpu_memory_utilization=0.9, chunked_prefill=True,
                    dtype="bfloat16", enforce_eager=args.eager)
    engine = LLMEngine(model, config)
    prompts, outputs = workload_requests(w, cfg.vocab_size)
    sps = [SamplingParams(temperature=0.6, max_tokens=n, ignore_eos=True, seed=1) for n in outputs]
    # one short request first, as the reference's harness does (benchmark.py:129-131)
    engine.generate([random_ids(32, cfg.vocab_size, 1)], SamplingParams(temperature=0.6, max_tokens=8, ignore_eos=True), use_tqdm=False)
    torch.cuda.synchronize()
    stats = engine.collect_stats(kernels=args.kernel_classes)
    clocks = ClockSampler(period=0.05)
    launches0 = _launches(engine)
    with clocks:
        t0 = time.perf_counter()
        completions = engine.generate(prompts, sps, use_tqdm=False)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
    kinds = stats.summary()
    kernel_classes = kinds.pop("kernels", None)  # --kernel-classes: device time per launching function, eager steps only
    runner = engine.model_runner
    extra = {
        "steps": {k: v["steps"] for k, v in kinds.items()},
        "step_tokens": {k: v["tokens"] for k, v in kinds.items()},
        "host_ms": {k: v["host_ms"] for k, v in kinds.items()},
        "device_ms": {k: v["device_ms"] for k, v in kinds.items()},
        "host_ms_per_step": {k: round(v["host_ms"] / max(v["steps"], 1), 3) for k, v in kinds.items()},
        "device_ms_per_step": {k: round(v["device_ms"] / max(v["steps"], 1), 3) for k, v in kinds.items()},
        "preemptions": engine.scheduler.num_preemptions,
        "cache": {"pages": runner.num_pages[0], "page_size": PAGE_SIZE, "tokens": runner.num_pages[0] * PAGE_SIZE,
                  "gb": round(runner.num_pages[0] * sum(runner.page_bytes) / 1e9, 2), "sizing": runner.sizing},
        "gpu_launches": _launches(engine) - launches0,
        "clocks": clocks.summary(),
    }
    record = workload_record(args, w, cfg, "ours", prompts, outputs, wall, sum(len(c) for c in completions), extra)
    record["config"]["layers_full"] = full_cfg.num_hidden_layers
    record["config"]["kv_block"] = PAGE_SIZE
    if kernel_classes is not None:
        record["kernel_classes_ms"] = {name: row["ms"] for name, row in sorted(kernel_classes.items(), key=lambda kv: -kv[1]["ms"])}
    return record


def _launches(engine) -> int:
    from tokensprint_b200 import ops

    return ops.launch_count + engine.model_runner.graph_launches


def _reference_workload(args) -> dict:
    import tempfile

    import torch
    from engine.generation.config import Config as RefConfig
    from engine.generation.config import SamplingParams as RefSamplingParams
    from engine.generation.llm_engine import LLMEngine as RefEngine

    from tokensprint_b200.config.registry import get_model_config

    w = WORKLOADS[args.workload]
    cfg = get_model_config(w["model"])
    model = reference_model(cfg, w["max_model_len"])
    prompts, outputs = workload_requests(w, cfg.vocab_size)
    with torch.inference_mode(), tempfile.TemporaryDirectory() as model_dir:
        config = RefConfig(model=model_dir, max_model_len=w["max_model_len"], max_num_seqs=w["max_seqs"], max_num_batched_tokens=w["budget"],
                           kvcache_block_size=256, chunked_prefill=True, eos=-1, dtype=torch.bfloat16, gpu_memory_utilization=0.9)
        engine = RefEngine(model=model, config=config, tokenizer=None)
        engine.generate([random_ids(32, cfg.vocab_size, 1)], RefSamplingParams(temperature=0.6, max_tokens=8, ignore_eos=True), use_tqdm=False)
        sps = [RefSamplingParams(temperature=0.6, max_tokens=n, ignore_eos=True) for n in outputs]
        torch.cuda.synchronize()
        clocks = ClockSampler(period=0.05)
        with clocks:
            t0 = time.perf_counter()
            completions = engine.generate(prompts, sps, use_tqdm=False)
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
        extra = {"cache": {"pages": int(config.num_kvcache_blocks), "page_size": 256, "tokens": int(config.num_kvcache_blocks) * 256},
                 "clocks": clocks.summary()}
    record = workload_record(args, w, cfg, "reference", prompts, outputs, wall, sum(len(c) for c in completions), extra)
    record["config"]["kv_block"] = 256
    return record


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=64)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in the record)")
    p.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64")
    p.add_argument("--eager", action="store_true", help="no CUDA graphs for decode steps")
    p.add_argument("--kernel-classes", action="store_true",
                   help="with --workload: device time per launching function of the engine, for the steps that do not replay a graph "
                        "(the events cost host time: take the throughput from a run without this option)")
    p.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                   help="a serving loop through generate() instead of the decode benchmark (one JSON line)")
    p.add_argument("--probe", choices=["decode", "prefill"], default=None,
                   help="run a few steps inside cudaProfilerStart/Stop for ncu and exit (see profiles/)")
    args = p.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.probe:
        return run_probe(args)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        result = run_reference(args)
    else:
        result = run_workload(args) if args.workload else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
