"""The step function: one batch of (request, its next tokens) through the model.

`ModelRunner.step(entries)` runs exactly the tokens it is given, as one batch, from the
cache that earlier steps left, and returns float32 logits at the wanted places.  An
entry may be a whole prompt, a portion of one, a recomputation after preemption or a
single decoded token; any mix may stand side by side.  Sampling is a separate call, so
the same function serves generation and trace replay.

The reference's counterpart is ModelRunner.prepare_model_input + run_model
(engine/generation/model_runner.py:101-201): there the step's index tensors are built
from python lists and copied one by one; here they are packed into one pinned buffer and
cross to the device in a single copy.  Keys and values are always read through the
block tables (the reference switches between this step's tensors and the cache,
engine/nn/attention.py:190-191).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from tokensprint_b200.cache.manager import CacheManager, RequestCache
from tokensprint_b200.cache.tensors import CacheTensors, groups_of, page_bytes
from tokensprint_b200.models.model import Model
from tokensprint_b200.parts.base import GroupTables, StepContext


@dataclass
class StepEntry:
    """One request's share of a step."""

    cache: RequestCache
    tokens: Sequence[int]
    start: int  # absolute position of tokens[0]
    want: Sequence[int] = ()  # places among `tokens` whose logits are asked for


def _round4(n: int) -> int:
    return (n + 3) & ~3


class _Layout:
    """Offsets (in int32 elements) of a step's index arrays inside one packed buffer."""

    def __init__(self, T: int, B: int, R: int, widths: Sequence[int]) -> None:
        self.T, self.B, self.R, self.widths = T, B, R, list(widths)
        self.sections: dict[str, tuple[int, int]] = {}
        off = 0

        def add(name: str, n: int) -> None:
            nonlocal off
            self.sections[name] = (off, n)
            off += _round4(max(n, 1))

        add("token_ids", T)
        add("positions", T)
        add("seq_index", T)
        add("cu_seqlens_q", B + 1)
        add("context_lens", B)
        add("state_slots", B)
        add("rows", R)
        for g, w in enumerate(self.widths):
            add(f"slots{g}", T)
            add(f"table{g}", B * w)
        self.total = off

    def view(self, buf, name: str):
        off, n = self.sections[name]
        return buf[off : off + n]


class ModelRunner:
    def __init__(
        self,
        model: Model,
        *,
        page_size: int = 16,
        num_pages: Optional[int | Sequence[int]] = None,
        num_slots: int = 64,
        max_num_batched_tokens: int = 8192,
        gpu_memory_utilization: float = 0.9,
        poison_freed_pages: bool = False,
    ) -> None:
        if model.device.type != "cuda":
            raise RuntimeError("ModelRunner needs a CUDA device: the engine has no CPU path")
        self.model = model
        self.device = model.device
        self.page_size = page_size
        self.num_slots = num_slots
        self.max_num_batched_tokens = max_num_batched_tokens
        self.poison_freed_pages = poison_freed_pages
        self.vocab_size = model.spec.vocab_size

        needs = [p.need for p in model.cache_plan]
        self.groups, self.cache_group = groups_of(needs)
        itemsize = torch.empty((), dtype=model.dtype).element_size()
        self.page_bytes = [page_bytes(needs, self.cache_group, g, page_size, itemsize) for g in range(len(self.groups))]
        if num_pages is None:
            pages = self._pages_from_free_memory(gpu_memory_utilization)
        elif isinstance(num_pages, int):
            pages = [num_pages] * len(self.groups)
        else:
            pages = list(num_pages)
        if len(pages) != len(self.groups) or any(p < 1 for p in pages):
            raise ValueError(f"need one positive page count per cache group ({len(self.groups)}), got {pages}")
        self.num_pages = pages
        self.cache_manager = CacheManager(self.groups, page_size, pages, num_slots)
        self.cache_tensors = CacheTensors.allocate(
            needs, self.cache_group, pages, page_size, num_slots, self.device, model.dtype)
        self.layer_caches = [
            self.cache_tensors.layer_cache(model.run_cache[i], run.writes_cache)
            for i, run in enumerate(model.spec.run_order)
        ]
        self._pinned: list[torch.Tensor] = []
        self._pinned_events: list[Optional[torch.cuda.Event]] = []
        self._pinned_next = 0
        self.steps_run = 0
        self.h2d_bytes = 0  # bytes of step inputs copied to the device so far

    # -- sizing ---------------------------------------------------------------------

    def _pages_from_free_memory(self, utilization: float) -> list[int]:
        """Pages from what is free on the device (engine/generation/model_runner.py:392-411),
        less an allowance for the activations of the largest step."""
        free, _ = torch.cuda.mem_get_info(self.device)
        spec = self.model.spec
        widest = 0
        for entry in self.model.cache_plan:
            widest = max(widest, entry.need.kv_heads * entry.need.head_dim)
        act = self.max_num_batched_tokens * (24 * spec.hidden_size + 64 * widest) * 4
        act += 2 * self.num_slots * spec.vocab_size * 4 + (1 << 30)
        budget = int(free * utilization) - act
        per_page = sum(self.page_bytes)
        n = budget // max(per_page, 1)
        if n < 1:
            raise RuntimeError(
                f"Insufficient GPU memory for the cache: {budget} bytes after activations, {per_page} bytes per page")
        return [int(n)] * len(self.groups)

    # -- the step ----------------------------------------------------------------------

    def _pinned_buffer(self, n: int) -> tuple[torch.Tensor, int]:
        if len(self._pinned) < 4:
            self._pinned.append(torch.empty(max(n, 1 << 14), dtype=torch.int32, pin_memory=True))
            self._pinned_events.append(None)
            return self._pinned[-1], len(self._pinned) - 1
        i = self._pinned_next
        self._pinned_next = (i + 1) % len(self._pinned)
        ev = self._pinned_events[i]
        if ev is not None:
            ev.synchronize()
        if self._pinned[i].numel() < n:
            self._pinned[i] = torch.empty(n, dtype=torch.int32, pin_memory=True)
        return self._pinned[i], i

    def build_context(self, entries: Sequence[StepEntry]) -> tuple[StepContext, torch.Tensor, int]:
        """Packs the step's index arrays, copies them to the device once and returns the
        context, the rows whose logits are wanted and their number."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        P = self.page_size
        B = len(entries)
        lens = [len(e.tokens) for e in entries]
        if min(lens) < 1:
            raise ValueError("every entry of a step brings at least one token")
        T = sum(lens)
        R = sum(len(e.want) for e in entries)
        widths = []
        for g in range(len(self.groups)):
            widths.append(max(1, max(-(-(e.start + n) // P) for e, n in zip(entries, lens))))
        layout = _Layout(T, B, R, widths)
        pinned, slot_i = self._pinned_buffer(layout.total)
        host = pinned.numpy()[: layout.total]

        tok = layout.view(host, "token_ids")
        pos = layout.view(host, "positions")
        sidx = layout.view(host, "seq_index")
        cu = layout.view(host, "cu_seqlens_q")
        ctx_lens = layout.view(host, "context_lens")
        slots = layout.view(host, "state_slots")
        rows = layout.view(host, "rows")
        cu[0] = 0
        t0 = 0
        r0 = 0
        seen = set()
        for b, (e, n) in enumerate(zip(entries, lens)):
            rc = e.cache
            if rc.released:
                raise ValueError(f"request {rc.request!r} was freed and cannot be stepped")
            if id(rc) in seen:
                raise ValueError(f"request {rc.request!r} appears twice in one step")
            seen.add(id(rc))
            if e.start < 0 or e.start + n > rc.num_tokens:
                raise ValueError(
                    f"request {rc.request!r}: tokens {e.start}..{e.start + n - 1} have no place in the cache "
                    f"({rc.num_tokens} positions were given one)")
            ids = np.asarray(e.tokens, dtype=np.int64)
            if ids.min() < 0 or ids.max() >= self.vocab_size:
                raise ValueError(f"request {rc.request!r}: token id outside 0..{self.vocab_size - 1}")
            tok[t0 : t0 + n] = ids
            pos[t0 : t0 + n] = np.arange(e.start, e.start + n)
            sidx[t0 : t0 + n] = b
            cu[b + 1] = t0 + n
            ctx_lens[b] = e.start + n
            slots[b] = rc.slot
            for w in e.want:
                if not (0 <= w < n):
                    raise ValueError(f"request {rc.request!r}: wanted place {w} is outside its {n} tokens")
                rows[r0] = t0 + w
                r0 += 1
            for g in range(len(self.groups)):
                layout.view(host, f"slots{g}")[t0 : t0 + n] = self.cache_manager.slots_for(rc, g, e.start, n)
                table = layout.view(host, f"table{g}").reshape(B, widths[g])
                have = rc.tables[g][: widths[g]]
                table[b, : len(have)] = have
                table[b, len(have) :] = -1
            if rc.fresh_slot:
                self.cache_tensors.zero_slot(rc.slot)
                rc.fresh_slot = False
            t0 += n

        dev = torch.empty(layout.total, dtype=torch.int32, device=self.device)
        dev.copy_(pinned[: layout.total], non_blocking=True)
        self.h2d_bytes += layout.total * 4
        ev = torch.cuda.Event()
        ev.record()
        self._pinned_events[slot_i] = ev

        groups = [
            GroupTables(
                block_table=layout.view(dev, f"table{g}").view(B, widths[g]),
                slot_mapping=layout.view(dev, f"slots{g}"),
            )
            for g in range(len(self.groups))
        ]
        step = StepContext(
            num_tokens=T,
            num_seqs=B,
            token_ids=layout.view(dev, "token_ids"),
            positions=layout.view(dev, "positions"),
            seq_index=layout.view(dev, "seq_index"),
            cu_seqlens_q=layout.view(dev, "cu_seqlens_q"),
            context_lens=layout.view(dev, "context_lens"),
            state_slots=layout.view(dev, "state_slots"),
            groups=groups,
            page_size=P,
            max_seqlen_q=max(lens),
            max_context_len=max(e.start + n for e, n in zip(entries, lens)),
            host_seq_starts=[e.start for e in entries],
            host_seq_lens=lens,
            host_state_slots=[e.cache.slot for e in entries],
            decode_only=max(lens) == 1,
        )
        return step, layout.view(dev, "rows"), R

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Float32 logits [wanted, vocab], in the order of the entries and of their `want`."""
        step, rows, R = self.build_context(entries)
        self.steps_run += 1
        hidden, pending = self.model.forward_hidden(step, self.layer_caches)
        if R == 0:
            return torch.empty((0, self.vocab_size), device=self.device, dtype=torch.float32)
        return self.model.logits(hidden, pending, rows, R)

    # -- cache life cycle (thin wrappers that keep device memory in step) ------------------

    def free(self, rc: RequestCache) -> None:
        if self.poison_freed_pages:
            held = [[p for p in t if p >= 0] for t in rc.tables]
            self.cache_manager.free(rc)
            for g, pages in enumerate(held):
                self.cache_tensors.poison_pages(g, pages)
        else:
            self.cache_manager.free(rc)
