"""The programming entry point: prompts in, completions out.

`LLMEngine(model, config, tokenizer=None)` with `add_request`, `step`, `generate` and
`is_finished`, as in the reference (engine/generation/llm_engine.py:18-114).  The runner
is built first because it decides how many cache pages there are; the scheduler then
works on the runner's cache manager (the reference passes that number through the
config, llm_engine.py:25-26).
"""

from __future__ import annotations

import logging
import time
from typing import Any, Optional, Sequence as Seq

import torch

from tokensprint_b200 import ops
from tokensprint_b200.config.engine_config import Config, SamplingParams
from tokensprint_b200.engine.runner import ModelRunner, StepEntry
from tokensprint_b200.engine.scheduler import Scheduler
from tokensprint_b200.engine.sequence import UNKNOWN_TOKEN, Sequence
from tokensprint_b200.models.model import Model
from tokensprint_b200.sampling.sampler import Sampler, sample_key

log = logging.getLogger(__name__)

STEP_KINDS = ("decode", "mixed", "prefill")


class StepStats:
    """Where the time of a run goes, step by step (switched on with `LLMEngine.collect_stats()`).

    Every step is of one kind: "decode" (every request brings one decoded token), "prefill" (none
    does: portions of prompts only) or "mixed".  Per step the host's time to schedule it, build
    its inputs and launch its kernels is taken with the wall clock, and the device's time with a
    pair of CUDA events on the launching stream (resolved at `summary()`, after a synchronize)."""

    def __init__(self, kernels: bool = False) -> None:
        self.records: list[tuple[str, int, float, "torch.cuda.Event", "torch.cuda.Event"]] = []
        self.kernels = kernels
        if kernels:
            from tokensprint_b200 import ops

            ops.kernel_times()  # forget what was recorded before
            ops.time_kernels(True)

    def begin(self):
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        return time.perf_counter(), start

    def end(self, begun, kind: str, tokens: int) -> None:
        t0, start = begun
        host_ms = (time.perf_counter() - t0) * 1e3
        stop = torch.cuda.Event(enable_timing=True)
        stop.record()
        self.records.append((kind, tokens, host_ms, start, stop))

    def summary(self) -> dict:
        """Per kind: steps, tokens, host ms and device ms (totals), after waiting for the device."""
        torch.cuda.synchronize()
        out = {kind: {"steps": 0, "tokens": 0, "host_ms": 0.0, "device_ms": 0.0} for kind in STEP_KINDS}
        for kind, tokens, host_ms, start, stop in self.records:
            row = out[kind]
            row["steps"] += 1
            row["tokens"] += tokens
            row["host_ms"] += host_ms
            row["device_ms"] += start.elapsed_time(stop)
        for row in out.values():
            row["host_ms"] = round(row["host_ms"], 2)
            row["device_ms"] = round(row["device_ms"], 2)
        if self.kernels:
            from tokensprint_b200 import ops

            out["kernels"] = ops.kernel_times()
            ops.time_kernels(False)
        return out


class LLMEngine:
    def __init__(self, model: Model, config: Config, tokenizer: Optional[Any] = None) -> None:
        self.config = config
        self.model_runner = ModelRunner(
            model,
            page_size=config.kvcache_block_size,
            num_pages=config.num_kvcache_blocks if config.num_kvcache_blocks > 0 else None,
            num_slots=config.max_num_seqs,
            max_num_batched_tokens=config.max_num_batched_tokens,
            gpu_memory_utilization=config.gpu_memory_utilization,
            enforce_eager=config.enforce_eager,
            max_model_len=config.max_model_len,
        )
        config.num_kvcache_blocks = self.model_runner.num_pages[0]
        self.model_runner.capture_graphs(config.max_num_seqs)  # nothing, if decode steps are not captured
        self.scheduler = Scheduler(config, self.model_runner.cache_manager)
        self.sampler = Sampler(model.device)
        self.tokenizer = tokenizer
        self._next_stream = 0
        # Steps overlap (config.overlap_steps): a step is launched before the host has read what
        # the step before sampled; its decoded tokens are fed on the device.  What is in flight:
        # (sequences, which of them are sampled for, the positions of their tokens, the ids' ticket).
        self.overlap = bool(getattr(config, "overlap_steps", True))
        self._inflight = None
        self.stats: Optional[StepStats] = None

    def collect_stats(self, kernels: bool = False) -> StepStats:
        """From now on every step's kind, tokens, host time and device time are recorded.  With
        `kernels`, eager steps also time every class of kernel (`ops.time_kernels`; `summary()` then
        has a "kernels" entry); steps that replay a graph have no calls to time."""
        self.stats = StepStats(kernels=kernels)
        return self.stats

    def _token_ids(self, prompt: str | list[int]) -> list[int]:
        """Token ids of a request: a list is taken as it is, text goes through the tokenizer."""
        if not isinstance(prompt, str):
            return list(prompt)
        if self.tokenizer is None:
            raise ValueError("a text prompt needs a tokenizer; pass token ids instead")
        ids = self.tokenizer.encode(prompt, add_special_tokens=True)
        if not isinstance(ids, list):
            raise TypeError(f"the tokenizer's encode() must return a list of ids, got {type(ids).__name__}")
        return ids

    def is_finished(self) -> bool:
        return self.scheduler.is_finished() and self._inflight is None

    def add_request(self, prompt: str | list[int], sampling_params: SamplingParams) -> Sequence:
        prompt = self._token_ids(prompt)
        vocab = self.model_runner.vocab_size
        if any((t < 0 or t >= vocab) for t in prompt):
            raise ValueError(f"prompt holds a token id outside 0..{vocab - 1}")
        sequence = Sequence(token_ids=list(prompt), sampling_params=sampling_params)
        sequence.sample_stream = self._next_stream
        self._next_stream += 1
        self.scheduler.add_sequence(sequence)
        return sequence

    def _launch(self):
        """Schedules and launches one step; returns what `_inflight` holds."""
        begun = self.stats.begin() if self.stats is not None else None
        seqs = self.scheduler.schedule()
        entries, need, temps, keys = [], [], [], []
        for i, seq in enumerate(seqs):
            start, n = seq.num_cached_tokens, seq.num_new_tokens
            reaches_end = start + n == len(seq)
            tokens = seq.token_ids[start : start + n]
            feed = -1
            if tokens[-1] == UNKNOWN_TOKEN:
                # sampled by the step before and not read yet: the device has it
                if n != 1 or seq.sample_row < 0:
                    raise RuntimeError(f"Sequence {seq.seq_id} is scheduled with a token that is not known yet.")
                feed = seq.sample_row
            entries.append(StepEntry(seq.cache, tokens, start, [n - 1] if reaches_end else [], feed))
            if reaches_end:
                need.append(i)
                temps.append(seq.temperature)
                keys.append(sample_key(seq.seed, seq.sample_stream, len(seq)))
        logits = self.model_runner.step(entries, self.sampler.device_ids)
        if begun is not None:
            single = sum(1 for seq in seqs if seq.num_new_tokens == 1 and seq.num_cached_tokens >= seq.num_prompt_tokens)
            kind = "decode" if single == len(seqs) else ("prefill" if single == 0 else "mixed")
            self._step_begun = (begun, kind, sum(seq.num_new_tokens for seq in seqs))
        return seqs, need, logits, temps, keys

    def _step_launched(self) -> None:
        """Closes the step's record once its sampling has been launched too."""
        if self.stats is not None and getattr(self, "_step_begun", None) is not None:
            begun, kind, tokens = self._step_begun
            self.stats.end(begun, kind, tokens)
            self._step_begun = None

    def step(self) -> tuple[list[tuple[int, list[int]]], int]:
        """One step.  Returns the requests that finished, as (id, completion token ids), and the
        number of their tokens.  With overlapping steps a call launches the next step and then
        reads the ids of the step before, so a request's end is reported one call later."""
        if not self.overlap:
            seqs, need, logits, temps, keys = self._launch()
            ticket = self.sampler.sample_async(logits, temps, keys)
            self._step_launched()
            token_ids = ticket.result()
            ops.check_device_errors()  # the copy of the sampled ids has just synchronised
            self.scheduler.postprocess(seqs, token_ids, need)
            finished = [seq for seq in seqs if seq.is_finished]
        else:
            launched = None
            if not self.scheduler.is_finished():
                seqs, need, logits, temps, keys = self._launch()
                ticket = self.sampler.sample_async(logits, temps, keys)
                self._step_launched()
                positions = self.scheduler.advance(seqs, need)
                launched = (seqs, need, positions, ticket)
            finished = []
            if self._inflight is not None:
                seqs, need, positions, ticket = self._inflight
                token_ids = ticket.result()
                ops.check_device_errors()  # the copy of the sampled ids has just synchronised
                finished = self.scheduler.resolve(seqs, need, positions, token_ids)
            self._inflight = launched
        outputs = [(seq.seq_id, seq.completion_token_ids) for seq in finished]
        num_total_tokens = sum(len(seq) for seq in finished)
        return outputs, num_total_tokens

    def finished_requests(self):
        """Runs steps until nothing is left; yields (request id, completion token ids) as requests end."""
        while not self.is_finished():
            outputs, _ = self.step()
            yield from outputs

    def generate(
        self,
        prompts: Seq[str] | Seq[list[int]],
        sampling_params: SamplingParams | list[SamplingParams],
        use_tqdm: bool = True,
    ) -> list[list[int]]:
        """Completions (token ids) in the order of the prompts (engine/generation/llm_engine.py:67-114
        of the reference: same arguments, same result)."""
        per_prompt = sampling_params if isinstance(sampling_params, list) else [sampling_params] * len(prompts)
        if len(per_prompt) != len(prompts):
            raise ValueError(f"{len(prompts)} prompts but {len(per_prompt)} sampling_params: one per prompt, or one for all.")
        order = [self.add_request(prompt, sp).seq_id for prompt, sp in zip(prompts, per_prompt)]
        progress = _Progress(len(order)) if use_tqdm else None
        completions: dict[int, list[int]] = {}
        for seq_id, token_ids in self.finished_requests():
            completions[seq_id] = token_ids
            if progress is not None:
                progress.request_done(len(token_ids))
        if progress is not None:
            progress.close()
        return [completions[seq_id] for seq_id in order]


class _Progress:
    """A tqdm bar over finished requests with the throughput of generated tokens so far."""

    def __init__(self, total: int) -> None:
        from tqdm.auto import tqdm

        self.bar = tqdm(total=total, desc="Generating", dynamic_ncols=True)
        self.started = time.perf_counter()
        self.tokens = 0

    def request_done(self, completion_tokens: int) -> None:
        self.tokens += completion_tokens
        rate = self.tokens / max(time.perf_counter() - self.started, 1e-9)
        self.bar.set_postfix({"generated": f"{int(rate)}tok/s"})
        self.bar.update(1)

    def close(self) -> None:
        self.bar.close()
