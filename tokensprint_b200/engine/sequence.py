"""One request's state on the host (engine/sequence.py:31-251 of the reference)."""

from __future__ import annotations

from copy import copy
from enum import Enum, auto
from itertools import count
from typing import ClassVar, Iterator, Optional

from tokensprint_b200.cache.manager import RequestCache
from tokensprint_b200.config.engine_config import SamplingParams


UNKNOWN_TOKEN = -1  # stands in a sequence for a token that has been sampled but not yet read by the host


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


class Sequence:
    """Prompt plus completion, how much of it the cache holds, and what the next step runs.

    The reference keeps the block table on the sequence and the block size as a class
    constant (engine/sequence.py:33,80); here the pages belong to `cache` (one table per
    cache group, handed out by the cache manager), so a sequence knows no page size.
    """

    counter: ClassVar[Iterator[int]] = count()

    def __init__(self, token_ids: list[int], sampling_params: Optional[SamplingParams] = None) -> None:
        if not token_ids:
            raise ValueError("token_ids must be non-empty.")
        sp = sampling_params if sampling_params is not None else SamplingParams()
        self.seq_id = next(Sequence.counter)
        self.status = SequenceStatus.WAITING
        self.token_ids = copy(list(token_ids))
        self.last_token = self.token_ids[-1]
        self.num_tokens = len(self.token_ids)
        self.num_prompt_tokens = len(self.token_ids)
        self.num_cached_tokens = 0  # tokens whose keys and values are in the cache
        self.num_new_tokens = 0  # tokens the current step runs
        self.temperature = sp.temperature
        self.max_tokens = sp.max_tokens
        self.ignore_eos = sp.ignore_eos
        self.seed = sp.seed
        self.sample_stream = 0  # which noise stream this request draws from (set by the engine)
        self.cache: Optional[RequestCache] = None
        self.num_preemptions = 0
        # Steps that overlap: tokens appended as UNKNOWN_TOKEN and not yet filled in; the row that
        # holds this sequence's newest id among the ids the last step sampled; the position of an
        # end-of-sequence token once one was seen (what later steps sampled for it is dropped).
        self.unresolved = 0
        self.sample_row = -1
        self.ended_at = -1
        self.reported = False

    def __len__(self) -> int:
        return self.num_tokens

    def __getitem__(self, key):
        return self.token_ids[key]

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(token_id)
        self.last_token = token_id
        self.num_tokens += 1

    def set_token(self, position: int, token_id: int) -> None:
        """Fills in a token that was appended before the host knew it."""
        self.token_ids[position] = token_id
        if position == self.num_tokens - 1:
            self.last_token = token_id

    def truncate(self, num_tokens: int) -> None:
        del self.token_ids[num_tokens:]
        self.num_tokens = len(self.token_ids)
        self.last_token = self.token_ids[-1]

    @property
    def is_finished(self) -> bool:
        return self.status == SequenceStatus.FINISHED

    @property
    def num_completion_tokens(self) -> int:
        return self.num_tokens - self.num_prompt_tokens

    @property
    def num_context_tokens(self) -> int:
        return self.num_cached_tokens + self.num_new_tokens

    @property
    def prompt_token_ids(self) -> list[int]:
        return self.token_ids[: self.num_prompt_tokens]

    @property
    def completion_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens :]
