"""Greedy and temperature sampling on the device.

The reference samples with an exponential race over the softmax (engine/generation/
sampler.py:11-16) from torch's global random stream; greedy is refused there
(engine/generation/config.py:13-15).  Here temperature 0 is greedy, and the race's noise
is a pure function of (seed, request's stream, position of the new token, vocabulary
index), so a request draws the same tokens whatever it is batched with and however often
it is preempted and recomputed.
"""

from __future__ import annotations

from typing import Sequence

import torch

from tokensprint_b200 import ops

_MASK = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def sample_key(seed: int, stream: int, position: int) -> int:
    """The 64-bit key of one draw, as a signed integer (it travels in an int64 tensor)."""
    k = _mix64(_mix64(seed & _MASK) ^ (stream & _MASK))
    k = _mix64(k ^ (position & _MASK))
    return k - (1 << 64) if k >= (1 << 63) else k


class SampleTicket:
    """The ids of one sampling call, on their way to the host."""

    def __init__(self, host: torch.Tensor, rows: int, event) -> None:
        self._host, self._rows, self._event = host, rows, event

    def result(self) -> list[int]:
        """Waits for the copy and returns one token id per row."""
        if self._rows == 0:
            return []
        if self._event is not None:
            self._event.synchronize()
        return self._host[: self._rows].tolist()


class Sampler:
    """Temperatures and keys go to the device through pinned staging buffers (two small
    asynchronous copies); the sampled ids stay on the device (`device_ids`, for a step that
    is launched before the host has seen them) and come back in one asynchronous copy.  Two
    sets of staging buffers alternate, so that a call may be made while the copies of the
    call before are still waiting for their turn on the device."""

    SETS = 2

    def __init__(self, device: torch.device | str, max_rows: int = 1024) -> None:
        self.device = torch.device(device)
        self._alloc(max_rows)

    def _alloc(self, rows: int) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)  # nothing in flight still reads the old buffers
        self._rows = rows
        pin = self.device.type == "cuda"
        self._temps_host = [torch.empty(rows, dtype=torch.float32, pin_memory=pin) for _ in range(self.SETS)]
        self._keys_host = [torch.empty(rows, dtype=torch.int64, pin_memory=pin) for _ in range(self.SETS)]
        self._ids_host = [torch.empty(rows, dtype=torch.int32, pin_memory=pin) for _ in range(self.SETS)]
        self._events = [None] * self.SETS
        self._next = 0
        self._temps = torch.empty(rows, dtype=torch.float32, device=self.device)
        self._keys = torch.empty(rows, dtype=torch.int64, device=self.device)
        self._out = torch.empty(rows, dtype=torch.int32, device=self.device)

    @property
    def device_ids(self) -> torch.Tensor:
        """The ids of the last call, row by row, on the device."""
        return self._out

    @torch.inference_mode()
    def sample_async(self, logits: torch.Tensor, temperatures: Sequence[float], keys: Sequence[int]) -> SampleTicket:
        """Launches the sampling of one token id per row of float32 logits [R, V] and the copy of
        the ids to the host; `result()` of the ticket waits for them."""
        R = logits.shape[0]
        if len(temperatures) != R or len(keys) != R:
            raise ValueError(f"{R} rows of logits, {len(temperatures)} temperatures, {len(keys)} keys")
        if R == 0:
            return SampleTicket(self._ids_host[0], 0, None)
        if R > self._rows:
            self._alloc(max(R, 2 * self._rows))
        k = self._next
        self._next = (k + 1) % self.SETS
        if self._events[k] is not None:
            self._events[k].synchronize()  # the call that used this set last is through with it
        self._temps_host[k][:R] = torch.tensor(temperatures, dtype=torch.float32)
        self._keys_host[k][:R] = torch.tensor(keys, dtype=torch.int64)
        self._temps[:R].copy_(self._temps_host[k][:R], non_blocking=True)
        self._keys[:R].copy_(self._keys_host[k][:R], non_blocking=True)
        out = self._out[:R]
        ops.sample(logits, self._temps[:R], self._keys[:R], out)
        self._ids_host[k][:R].copy_(out, non_blocking=True)
        event = None
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
            self._events[k] = event
        return SampleTicket(self._ids_host[k], R, event)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], keys: Sequence[int]) -> list[int]:
        """One token id per row of float32 logits [R, V]."""
        return self.sample_async(logits, temperatures, keys).result()
