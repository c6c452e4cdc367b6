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
        cm = self.cache_manager
        # The most pages the request holds at once: all of them in a group that keeps every key;
        # in a window group all of them too when the prompt comes in one portion (pages are given
        # back between steps only), else the window plus the largest portion.
        for g, pool in enumerate(cm.pools):
            spec = cm.groups[g]
            tokens = len(seq) + 1
            if spec.kind == "window" and self.enable_chunked:
                tokens = min(tokens, spec.window + self.max_num_batched_tokens + cm.page_size)
            need = -(-tokens // cm.page_size)
            if need > pool.num_pages:
                raise ValueError(
                    f"Prompt of {len(seq)} tokens needs {need} cache pages of group {g} ({spec.kind}), the pool holds "
                    f"{pool.num_pages}: it could never be scheduled.")
        self.waiting.append(seq)

    # -- one step ---------------------------------------------------------------------

    def _share(self, seq: Sequence, budget: int) -> int:
        """How many of the tokens it has not cached yet `seq` runs in a step with `budget` left:
        all of them, cut to the budget where portions are allowed, and never past the model's length."""
        share = len(seq) - seq.num_cached_tokens
        if self.enable_chunked:
            share = min(share, budget)
        return min(share, self.max_model_len - 1 - seq.num_cached_tokens)

    def _reserve(self, seq: Sequence, share: int) -> bool:
        """Pages for the next `share` tokens of a sequence that has a cache; False: not now."""
        first = seq.num_cached_tokens
        if not self.cache_manager.can_extend(seq.cache, first, first + share):
            return False
        self.cache_manager.extend(seq.cache, first, first + share)
        seq.num_new_tokens = share
        return True

    def _continue_running(self, budget: int, step: list[Sequence]) -> tuple[int, bool]:
        """Running requests in their order while the budget lasts.  One that finds no pages takes
        them from the tail of the running list, request by request, itself last.  Returns the
        budget left and whether anybody lost its place."""
        evicted = False
        place = 0
        while place < len(self.running) and budget > 0:
            seq = self.running[place]
            share = self._share(seq, budget)
            if share < 1:
                raise RuntimeError(f"Running sequence {seq.seq_id} has nothing to compute (share {share}).")
            while seq.status == SequenceStatus.RUNNING and not self._reserve(seq, share):
                self.preempt(self.running[-1])
                evicted = True
            if seq.status != SequenceStatus.RUNNING:
                break  # it gave up its own place; it was the last one
            step.append(seq)
            budget -= share
            place += 1
        return budget, evicted

    def _admit_waiting(self, budget: int, step: list[Sequence]) -> None:
        """Waiting requests, first come first served, while budget, slots and pages allow."""
        cm = self.cache_manager
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            if seq.cache is not None:
                raise RuntimeError(f"Waiting sequence {seq.seq_id} still holds cache pages.")
            share = self._share(seq, budget)
            if share > budget:
                return  # a whole prompt that does not fit what is left of this step
            try:
                seq.cache = cm.admit(seq.seq_id)
            except OutOfSlots:
                return
            seq.num_cached_tokens = 0
            if not self._reserve(seq, share):
                cm.free(seq.cache)
                seq.cache = None
                return
            self.waiting.popleft()
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            step.append(seq)
            budget -= share

    def schedule(self) -> list[Sequence]:
        """The sequences of the next step, each with `num_new_tokens` set and pages reserved."""
        step: list[Sequence] = []
        budget, evicted = self._continue_running(self.max_num_batched_tokens, step)
        if not evicted:  # a step that took somebody's pages admits nobody
            self._admit_waiting(budget, step)
        if not step:
            raise RuntimeError(
                "empty schedule: the next request alone needs more cache pages (or a larger token "
                "budget) than the engine has.")
        self.num_steps += 1
        return step

    def preempt(self, seq: Sequence) -> None:
        """Out of the running list and back to the front of the waiting queue; everything it
        cached is dropped."""
        if seq in self.running:
            self.running.remove(seq)
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

    def _ends_by_count(self, seq: Sequence) -> bool:
        """Ends that depend on lengths alone: the request's max_tokens, the model's length."""
        if len(seq) >= self.max_model_len:
            log.info("Sequence %s reached max_model_len %s.", seq.seq_id, self.max_model_len)
            return True
        return seq.num_completion_tokens == seq.max_tokens

    def _finish(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.FINISHED
        self._release(seq)
        if seq in self.running:
            self.running.remove(seq)

    def _commit(self, seqs: list[Sequence]) -> None:
        """What the step ran is cached now."""
        for seq in seqs:
            if seq.status != SequenceStatus.FINISHED:
                seq.num_cached_tokens += seq.num_new_tokens
                seq.num_new_tokens = 0

    def postprocess(self, seqs: list[Sequence], token_ids: list[int], seq_need_compute_logits: list[int]) -> None:
        """After a step: `token_ids[r]` was sampled for `seqs[seq_need_compute_logits[r]]`."""
        if len(token_ids) != len(seq_need_compute_logits):
            raise ValueError(
                f"{len(token_ids)} sampled tokens for {len(seq_need_compute_logits)} sequences that asked for one.")
        for row, which in enumerate(seq_need_compute_logits):
            seq, token = seqs[which], token_ids[row]
            seq.append_token(token)
            if (token == self.eos and not seq.ignore_eos) or self._ends_by_count(seq):
                self._finish(seq)
        self._commit(seqs)

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
            if self._ends_by_count(seq):
                self._finish(seq)
        self._commit(seqs)
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
        # nothing of it is reported any more: tokens still in flight for it are dropped
        seq.ended_at = min(seq.ended_at, len(seq) - 1) if seq.ended_at >= 0 else seq.num_prompt_tokens - 1
        seq.unresolved = 0
        seq.reported = True
