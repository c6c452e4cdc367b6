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
from tokensprint_b200.engine.sequence import Sequence
from tokensprint_b200.models.model import Model
from tokensprint_b200.sampling.sampler import Sampler, sample_key

log = logging.getLogger(__name__)


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
        self.scheduler = Scheduler(config, self.model_runner.cache_manager)
        self.sampler = Sampler(model.device)
        self.tokenizer = tokenizer
        self._next_stream = 0

    def _tokenize_prompt(self, prompt: str) -> list[int]:
        if self.tokenizer is None:
            raise ValueError("a text prompt needs a tokenizer; pass token ids instead")
        token_ids = self.tokenizer.encode(prompt, add_special_tokens=True)
        if not isinstance(token_ids, list):
            raise TypeError("Expected tokenizer.encode(...) to return list[int].")
        return token_ids

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    def add_request(self, prompt: str | list[int], sampling_params: SamplingParams) -> Sequence:
        if isinstance(prompt, str):
            prompt = self._tokenize_prompt(prompt)
        vocab = self.model_runner.vocab_size
        if any((t < 0 or t >= vocab) for t in prompt):
            raise ValueError(f"prompt holds a token id outside 0..{vocab - 1}")
        sequence = Sequence(token_ids=list(prompt), sampling_params=sampling_params)
        sequence.sample_stream = self._next_stream
        self._next_stream += 1
        self.scheduler.add_sequence(sequence)
        return sequence

    def step(self) -> tuple[list[tuple[int, list[int]]], int]:
        seqs = self.scheduler.schedule()
        entries, need, temps, keys = [], [], [], []
        for i, seq in enumerate(seqs):
            start, n = seq.num_cached_tokens, seq.num_new_tokens
            reaches_end = start + n == len(seq)
            entries.append(StepEntry(seq.cache, seq.token_ids[start : start + n], start, [n - 1] if reaches_end else []))
            if reaches_end:
                need.append(i)
                temps.append(seq.temperature)
                keys.append(sample_key(seq.seed, seq.sample_stream, len(seq)))
        logits = self.model_runner.step(entries)
        token_ids = self.sampler.sample(logits, temps, keys)
        ops.check_device_errors()  # the copy of the sampled ids has just synchronised
        self.scheduler.postprocess(seqs, token_ids, need)
        outputs = [(seq.seq_id, seq.completion_token_ids) for seq in seqs if seq.is_finished]
        num_total_tokens = sum(len(seq) for seq in seqs if seq.is_finished)
        return outputs, num_total_tokens

    def generate(
        self,
        prompts: Seq[str] | Seq[list[int]],
        sampling_params: SamplingParams | list[SamplingParams],
        use_tqdm: bool = True,
    ) -> list[list[int]]:
        """Completions (token ids) in the order of the prompts."""
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError(
                f"sampling_params length must match prompts length, got {len(sampling_params)} and {len(prompts)}.")
        pbar = None
        if use_tqdm:
            from tqdm.auto import tqdm

            pbar = tqdm(total=len(prompts), desc="Generating", dynamic_ncols=True)
        for prompt, sp in zip(prompts, sampling_params):
            self.add_request(prompt, sp)
        outputs: dict[int, list[int]] = {}
        num_total_tokens = 0
        t = time.perf_counter()
        while not self.is_finished():
            output, num_step_tokens = self.step()
            num_total_tokens += num_step_tokens
            if pbar is not None:
                throughput = num_total_tokens / max(time.perf_counter() - t, 1e-9)
                pbar.set_postfix({"total_throughput": f"{int(throughput)}tok/s"})
            for seq_id, token_ids in output:
                outputs[seq_id] = token_ids
                if pbar is not None:
                    pbar.update(1)
        if pbar is not None:
            pbar.close()
        return [outputs[seq_id] for seq_id in sorted(outputs)]
