"""Continuous batching on the host: who runs in the next step, and with how many tokens.

The policy is the reference's (engine/generation/scheduler.py:55-214):

* Running requests first, in order, while the step's token budget lasts; then, only if
  nobody was preempted in this step, waiting requests first-come-first-served while
  budget, sequence slots and pages allow.
* A request wants all tokens it has not cached: its whole prompt (or what is left of it),
  its prompt plus completion after a preemption, or the one token it sampled last.  With
  `chunked_prefill` that wish is cut to the remaining budget; without it a waiting
  request that does not fit the budget stops admission for this step.
* When pages run out for a running request, the *last* running request is preempted:
  its pages and slot go back, it returns to the front of the waiting queue and is
  recomputed from its first token when it is admitted again.  A request may preempt
  itself.  If nothing at all can run the scheduler raises: alone, the request needs more
  pages than the cache holds.
* A request finishes on EOS (unless ignored), at `max_tokens`, or at `max_model_len`.

Beyond the reference: a request that could never run is refused when it is added (a
prompt longer than the budget without chunked prefill, or one that needs more pages
than the whole pool), instead of failing later with the generic empty-schedule error.
"""

from __future__ import annotations

import logging
from collections import deque

from tokensprint_b200.cache.manager import CacheManager, OutOfSlots
from tokensprint_b200.config.engine_config import Config
from tokensprint_b200.engine.sequence import UNKNOWN_TOKEN, Sequence, SequenceStatus

log = logging.getLogger(__name__)


class Scheduler:
    def __init__(self, config: Config, cache_manager: CacheManager) -> None:
        self.enable_chunked = config.chunked_prefill
        self.max_model_len = config.max_model_len
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = config.eos
        self.cache_manager = cache_manager
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0
        self.num_steps = 0

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add_sequence(self, seq: Sequence) -> None:
        if len(seq) > self.max_model_len - 1:
            raise ValueError(
                f"Sequence length exceeds max_model_len: got {len(seq)}, max allowed is {self.max_model_len - 1}.")
        if not self.enable_chunked and len(seq) > self.max_num_batched_tokens:
            raise ValueError(
                f"Prompt of {len(seq)} tokens exceeds max_num_batched_tokens={self.max_num_batched_tokens} "
                "and chunked_prefill is off: it could never be scheduled.")
        page = self.cache_manager.page_size
        need = -(-(len(seq) + 1) // page)
        for g, pool in enumerate(self.cache_manager.pools):
            if self.cache_manager.groups[g].kind == "full" and need > pool.num_pages:
                raise ValueError(
                    f"Prompt of {len(seq)} tokens needs {need} cache pages, the pool holds {pool.num_pages}: "
                    "it could never be scheduled.")
        self.waiting.append(seq)

    # -- one step ---------------------------------------------------------------------

    def schedule(self) -> list[Sequence]:
        scheduled_running: list[Sequence] = []
        scheduled_new: list[Sequence] = []
        preempted: list[Sequence] = []
        token_budget = self.max_num_batched_tokens
        cm = self.cache_manager

        index = 0
        while index < len(self.running) and token_budget > 0:
            seq = self.running[index]
            num_new = len(seq) - seq.num_cached_tokens
            if self.enable_chunked:
                num_new = min(num_new, token_budget)
            num_new = min(num_new, self.max_model_len - 1 - seq.num_cached_tokens)
            if num_new <= 0:
                raise RuntimeError(
                    f"Expected a positive num_new_tokens for running sequence {seq.seq_id}, but got {num_new}.")
            while True:
                start = seq.num_cached_tokens
                if cm.can_extend(seq.cache, start, start + num_new):
                    seq.num_new_tokens = num_new
                    cm.extend(seq.cache, start, start + num_new)
                    break
                victim = self.running.pop()
                self.preempt(victim)
                preempted.append(victim)
                if len(self.running) == index:
                    break
            if len(self.running) == index:
                break
            scheduled_running.append(seq)
            token_budget -= seq.num_new_tokens
            index += 1

        if not preempted:
            while self.waiting and token_budget > 0 and len(self.running) < self.max_num_seqs:
                seq = self.waiting[0]
                if seq.cache is not None:
                    raise RuntimeError(f"Waiting sequence {seq.seq_id} still holds cache pages.")
                num_new = len(seq)
                if self.enable_chunked:
                    num_new = min(num_new, token_budget)
                num_new = min(num_new, self.max_model_len - 1)
                if num_new > token_budget:
                    break
                try:
                    rc = cm.admit(seq.seq_id)
                except OutOfSlots:
                    break
                if not cm.can_extend(rc, 0, num_new):
                    cm.free(rc)
                    break
                cm.extend(rc, 0, num_new)
                seq.cache = rc
                seq.num_cached_tokens = 0
                seq.num_new_tokens = num_new
                token_budget -= num_new
                seq.status = SequenceStatus.RUNNING
                self.waiting.popleft()
                self.running.append(seq)
                scheduled_new.append(seq)

        scheduled = scheduled_running + scheduled_new
        if not scheduled:
            raise RuntimeError(
                "Scheduler.schedule produced an empty schedule: the next request alone needs more "
                "cache pages (or a larger token budget) than the engine has.")
        self.num_steps += 1
        return scheduled

    def preempt(self, seq: Sequence) -> None:
        """Back to the front of the waiting queue; everything it cached is dropped."""
        seq.status = SequenceStatus.WAITING
        self._release(seq)
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(seq)

    def _release(self, seq: Sequence) -> None:
        if seq.cache is not None:
            self.cache_manager.free(seq.cache)
            seq.cache = None
        seq.num_cached_tokens = 0
        seq.num_new_tokens = 0

    def postprocess(self, seqs: list[Sequence], token_ids: list[int], seq_need_compute_logits: list[int]) -> None:
        if len(token_ids) != len(seq_need_compute_logits):
            raise ValueError(
                "token_ids and seq_need_compute_logits must have equal length, "
                f"got {len(token_ids)} and {len(seq_need_compute_logits)}.")
        for seq_index, token_id in zip(seq_need_compute_logits, token_ids):
            seq = seqs[seq_index]
            seq.append_token(token_id)
            if (
                (not seq.ignore_eos and token_id == self.eos)
                or seq.num_completion_tokens == seq.max_tokens
                or len(seq) >= self.max_model_len
            ):
                if len(seq) >= self.max_model_len:
                    log.info("Sequence %s reached max_model_len %s.", seq.seq_id, self.max_model_len)
                seq.status = SequenceStatus.FINISHED
                self._release(seq)
                self.running.remove(seq)
        for seq in seqs:
            if seq.status != SequenceStatus.FINISHED:
                seq.num_cached_tokens += seq.num_new_tokens
                seq.num_new_tokens = 0

    # -- steps that overlap ------------------------------------------------------------------
    #
    # A step can be launched before the host has read what the step before sampled: the new
    # token of every sequence is then on the device only.  `advance` does, right after the
    # launch, what `postprocess` does without looking at the tokens: the sequences grow by a
    # token that is not known yet, and the ends that only depend on counts (max_tokens, the
    # model's length) are decided.  `resolve` fills the tokens in when they have arrived, one
    # step later, and ends a sequence whose token was the end-of-sequence token; what the step
    # in flight has meanwhile computed for that sequence is dropped.

    def advance(self, seqs: list[Sequence], seq_need_compute_logits: list[int]) -> list[int]:
        """Returns, for every sequence that the step samples for, the position its token will have."""
        positions = []
        for row, seq_index in enumerate(seq_need_compute_logits):
            seq = seqs[seq_index]
            positions.append(len(seq))
            seq.append_token(UNKNOWN_TOKEN)
            seq.unresolved += 1
            seq.sample_row = row
            if seq.num_completion_tokens == seq.max_tokens or len(seq) >= self.max_model_len:
                if len(seq) >= self.max_model_len:
                    log.info("Sequence %s reached max_model_len %s.", seq.seq_id, self.max_model_len)
                seq.status = SequenceStatus.FINISHED
                self._release(seq)
                self.running.remove(seq)
        for seq in seqs:
            if seq.status != SequenceStatus.FINISHED:
                seq.num_cached_tokens += seq.num_new_tokens
                seq.num_new_tokens = 0
        return positions

    def resolve(self, seqs: list[Sequence], seq_need_compute_logits: list[int], positions: list[int],
                token_ids: list[int]) -> list[Sequence]:
        """Fills in the tokens of a step that `advance` has accounted for.  Returns the sequences
        that are finished and complete (each once)."""
        if not (len(token_ids) == len(seq_need_compute_logits) == len(positions)):
            raise ValueError(
                "token_ids, seq_need_compute_logits and positions must have equal length, "
                f"got {len(token_ids)}, {len(seq_need_compute_logits)} and {len(positions)}.")
        done = []
        for seq_index, position, token_id in zip(seq_need_compute_logits, positions, token_ids):
            seq = seqs[seq_index]
            if 0 <= seq.ended_at < position:
                continue  # sampled after the sequence's end: dropped with the sequence's tail
            seq.set_token(position, token_id)
            seq.unresolved -= 1
            if not seq.ignore_eos and token_id == self.eos:
                seq.ended_at = position
                seq.truncate(position + 1)
                seq.unresolved = 0
                if seq.status == SequenceStatus.RUNNING:
                    self.running.remove(seq)
                elif seq.status == SequenceStatus.WAITING:  # preempted in the meantime
                    self.waiting.remove(seq)
                seq.status = SequenceStatus.FINISHED
                self._release(seq)
            if seq.status == SequenceStatus.FINISHED and seq.unresolved == 0 and not seq.reported:
                seq.reported = True
                done.append(seq)
        return done

    def abort(self, seq: Sequence) -> None:
        """Drops a request wherever it is."""
        if seq in self.running:
            self.running.remove(seq)
        elif seq in self.waiting:
            self.waiting.remove(seq)
        self._release(seq)
        seq.status = SequenceStatus.FINISHED
