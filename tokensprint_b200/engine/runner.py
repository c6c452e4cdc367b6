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
    # A single token that the host does not know yet: row `feed` of the ids that the step's
    # caller names (what an earlier step sampled, still on the device) takes the place of tokens[0].
    feed: int = -1


@dataclass
class _DecodeGraph:
    bucket: int
    layout: "_Layout"
    dev: torch.Tensor  # static index buffer the captured kernels read
    host: torch.Tensor  # its pinned staging copy
    graph: "torch.cuda.CUDAGraph"
    logits: torch.Tensor  # [bucket, vocab] float32, rewritten by every replay
    kernels: int  # kernels of this library inside the graph
    event: Optional["torch.cuda.Event"] = None
    # per cache group: row of the batch -> (request cache, table entries written, first entry still held)
    row_marks: list = None


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
        add("feed_lanes", B)
        add("feed_rows", B)
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
        enforce_eager: bool = True,
        max_model_len: int = 4096,
        max_graph_batch: int = 256,
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
        self._needs = needs
        self._pinned: list[torch.Tensor] = []
        self._pinned_events: list[Optional[torch.cuda.Event]] = []
        self._pinned_next = 0
        self.steps_run = 0
        self.h2d_bytes = 0  # bytes of step inputs copied to the device so far
        # Decode-only steps replay a CUDA graph per batch bucket (engine/generation/
        # model_runner.py:310-390 of the reference); here the graph holds the whole step,
        # final norm and head included.
        self.max_model_len = max_model_len
        self.use_graphs = (not enforce_eager) and model.graph_safe
        most = max(1, min(max_graph_batch, num_slots))
        # sizes a decode step is padded to: from 64 sequences on in steps of 16, from 256 on of 32 (a
        # padded sequence costs no attention, but its row goes through every product and small kernel)
        sizes = [1, 2, 4, 8, 16, 24, 32, 48] + list(range(64, 256, 16)) + list(range(256, 513, 32))
        self.graph_buckets = [b for b in sizes if b <= most]
        if self.graph_buckets[-1] < most:
            # the largest batch has a graph too, whatever the number of slots is (a decode step of 33
            # sequences took 5.9 ms launched kernel by kernel, 4.8 ms as the graph of 40)
            self.graph_buckets.append(-(-most // 8) * 8)
        self._graphs: dict[int, "_DecodeGraph"] = {}
        self._graph_pool = None
        self._capture_stream: Optional[torch.cuda.Stream] = None
        self.graph_launches = 0  # kernels of this library replayed inside graphs so far
        self.sizing: Optional[dict] = None  # how the page count was derived, when it came from free memory

        if num_pages is None:
            pages = self._pages_from_free_memory(gpu_memory_utilization)
        elif isinstance(num_pages, int):
            pages = [num_pages] * len(self.groups)
        else:
            pages = list(num_pages)
        if len(pages) != len(self.groups) or any(p < 1 for p in pages):
            raise ValueError(f"need one positive page count per cache group ({len(self.groups)}), got {pages}")
        self._bind_cache(pages)

    def _bind_cache(self, pages: Sequence[int]) -> None:
        """A cache manager and device pools of `pages` pages per group, bound to the model's runs."""
        self.num_pages = list(pages)
        self.cache_manager = CacheManager(self.groups, self.page_size, self.num_pages, self.num_slots)
        self.cache_tensors = CacheTensors.allocate(
            self._needs, self.cache_group, self.num_pages, self.page_size, self.num_slots, self.device, self.model.dtype)
        self.layer_caches = [
            self.cache_tensors.layer_cache(self.model.run_cache[i], run.writes_cache)
            for i, run in enumerate(self.model.spec.run_order)
        ]

    # -- sizing ---------------------------------------------------------------------

    def _pages_from_free_memory(self, utilization: float) -> list[int]:
        """Pages from what is free on the device once the largest step has run.

        The reference sizes its cache from free memory less the peak of a warm-up run
        (engine/generation/model_runner.py:392-411).  Here the peak is measured the same way: a
        step of `max_num_batched_tokens` tokens runs once against a throw-away pool just large
        enough for it, torch's peak statistics give what its activations need, and the pool gets
        `utilization` of what is free afterwards less that peak and less what the decode graphs
        will hold (their static logits).  All groups get the same number of pages."""
        P = self.page_size
        tokens = max(1, self.max_num_batched_tokens)
        per_request = max(1, min(tokens, self.max_model_len - 1))
        lengths = [per_request] * (tokens // per_request) + ([tokens % per_request] if tokens % per_request else [])
        lengths = lengths[: self.num_slots]
        probe_pages = sum(-(-n // P) for n in lengths) + 1
        self._bind_cache([probe_pages] * len(self.groups))
        torch.cuda.synchronize(self.device)
        torch.cuda.reset_peak_memory_stats(self.device)
        before = torch.cuda.memory_allocated(self.device)
        entries = []
        for i, n in enumerate(lengths):
            rc = self.cache_manager.admit(("sizing", i))
            self.cache_manager.extend(rc, 0, n)
            entries.append(StepEntry(rc, [0] * n, 0, [n - 1]))
        graphs, self.use_graphs = self.use_graphs, False
        self.step(entries)
        self.use_graphs = graphs
        torch.cuda.synchronize(self.device)
        peak = torch.cuda.max_memory_allocated(self.device) - before
        self.steps_run = 0
        self.h2d_bytes = 0
        del entries
        self.cache_manager = self.cache_tensors = self.layer_caches = None
        torch.cuda.empty_cache()
        free, total = torch.cuda.mem_get_info(self.device)
        graph_reserve = 0
        if self.use_graphs:  # every bucket keeps its logits [bucket, vocab] float32, and a little beside
            graph_reserve = int(sum(self.graph_buckets) * self.vocab_size * 4 * 1.25)
        margin = 256 << 20
        budget = int(free * utilization) - peak - graph_reserve - margin
        per_page = sum(self.page_bytes)
        n = budget // max(per_page, 1)
        self.sizing = {"free_bytes": int(free), "total_bytes": int(total), "utilization": utilization,
                       "step_tokens": sum(lengths), "step_peak_bytes": int(peak), "graph_reserve_bytes": graph_reserve,
                       "margin_bytes": margin, "bytes_per_page": int(per_page), "pages": int(n)}
        if n < 1:
            raise RuntimeError(
                f"Insufficient GPU memory for the cache: {budget} bytes are left after a step of {sum(lengths)} tokens "
                f"({peak} bytes) and the graphs' reserve ({graph_reserve}); one page costs {per_page} bytes")
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

    def _feed(self, dev: torch.Tensor, layout: _Layout, feeds: int, fed_ids: Optional[torch.Tensor]) -> None:
        """Tokens that only the device knows go from `fed_ids` into the step's token lanes."""
        if feeds == 0:
            return
        from tokensprint_b200 import ops

        if fed_ids is None:
            raise ValueError("an entry names a row of fed ids, but the step was given none")
        ops.feed_tokens(layout.view(dev, "token_ids"), fed_ids, layout.view(dev, "feed_lanes"), layout.view(dev, "feed_rows"), feeds)

    def build_context(self, entries: Sequence[StepEntry], fed_ids: Optional[torch.Tensor] = None) -> tuple[StepContext, torch.Tensor, int]:
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
        # In a step that carries single decoded tokens beside portions of prompts the single tokens'
        # requests come first in the batch (a mixer then sees two ranges of sequences, one per kind);
        # the logits keep the order of the entries as they were given.
        row_base = None
        singles = sum(1 for n in lens if n == 1)
        if 0 < singles < B:
            order = sorted(range(B), key=lambda i: lens[i] != 1)  # stable: each kind keeps its order
            if order != list(range(B)):
                base, acc = [0] * B, 0
                for i, e in enumerate(entries):
                    base[i] = acc
                    acc += len(e.want)
                row_base = [base[i] for i in order]
                entries = [entries[i] for i in order]
                lens = [lens[i] for i in order]
        else:
            singles = B if singles == B else 0
        widths = []
        for g in range(len(self.groups)):
            widths.append(max(1, max(-(-(e.start + n) // P) for e, n in zip(entries, lens))))
        layout = _Layout(T, B, R, widths)
        pinned, slot_i = self._pinned_buffer(layout.total)
        host = pinned.numpy()[: layout.total]
        feeds = self._fill(host, layout, entries, lens, row_base=row_base)

        dev = torch.empty(layout.total, dtype=torch.int32, device=self.device)
        dev.copy_(pinned[: layout.total], non_blocking=True)
        self.h2d_bytes += layout.total * 4
        self._feed(dev, layout, feeds, fed_ids)
        ev = torch.cuda.Event()
        ev.record()
        self._pinned_events[slot_i] = ev
        step = self._context(dev, layout, max(lens), max(e.start + n for e, n in zip(entries, lens)))
        step.host_seq_starts = [e.start for e in entries]
        step.host_seq_lens = lens
        step.host_state_slots = [e.cache.slot for e in entries]
        step.rows_all = row_base is None and all(list(e.want) == list(range(n)) for e, n in zip(entries, lens))
        step.decode_seqs = singles
        return step, layout.view(dev, "rows"), R

    def _fill(self, host, layout: _Layout, entries: Sequence[StepEntry], lens: Sequence[int], row_marks=None, row_base=None) -> int:
        """Writes the step's index arrays into `host` (a numpy view of pinned memory).  A
        layout larger than the step (a graph bucket) is padded with lanes that belong to no
        request: sequence index -1, no cache slot, no tokens in their sequence.  Returns how
        many token lanes are to be fed on the device (entries with `feed`).  `row_base`: where in
        the list of wanted rows each entry's rows go (entries that were reordered); None: one after
        the other."""
        B, widths = layout.B, layout.widths
        tok = layout.view(host, "token_ids")
        pos = layout.view(host, "positions")
        sidx = layout.view(host, "seq_index")
        cu = layout.view(host, "cu_seqlens_q")
        ctx_lens = layout.view(host, "context_lens")
        slots = layout.view(host, "state_slots")
        rows = layout.view(host, "rows")
        feed_lanes = layout.view(host, "feed_lanes")
        feed_rows = layout.view(host, "feed_rows")
        feeds = 0
        cu[0] = 0
        t0 = 0
        r0 = 0
        seen = set()
        tables = [layout.view(host, f"table{g}").reshape(B, widths[g]) for g in range(len(self.groups))]
        slot_maps = [layout.view(host, f"slots{g}") for g in range(len(self.groups))]
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
            if e.feed >= 0:
                if n != 1:
                    raise ValueError(f"request {rc.request!r}: only a single token can be fed on the device")
                tok[t0] = 0
                feed_lanes[feeds] = t0
                feed_rows[feeds] = e.feed
                feeds += 1
                pos[t0] = e.start
                sidx[t0] = b
            elif n == 1:  # a decoded token: plain numbers instead of array operations
                token = e.tokens[0]
                if not 0 <= token < self.vocab_size:
                    raise ValueError(f"request {rc.request!r}: token id outside 0..{self.vocab_size - 1}")
                tok[t0] = token
                pos[t0] = e.start
                sidx[t0] = b
            else:
                ids = np.asarray(e.tokens, dtype=np.int64)
                if ids.min() < 0 or ids.max() >= self.vocab_size:
                    raise ValueError(f"request {rc.request!r}: token id outside 0..{self.vocab_size - 1}")
                tok[t0 : t0 + n] = ids
                pos[t0 : t0 + n] = np.arange(e.start, e.start + n)
                sidx[t0 : t0 + n] = b
            cu[b + 1] = t0 + n
            ctx_lens[b] = e.start + n
            slots[b] = rc.slot
            if row_base is not None:
                r0 = row_base[b]
            for w in e.want:
                if not (0 <= w < n):
                    raise ValueError(f"request {rc.request!r}: wanted place {w} is outside its {n} tokens")
                rows[r0] = t0 + w
                r0 += 1
            for g in range(len(self.groups)):
                table = rc.tables[g]
                if n == 1:
                    page = table[e.start // self.page_size]
                    if page < 0:
                        raise ValueError(f"request {rc.request!r}: position {e.start} lies in a page that was given back")
                    slot_maps[g][t0] = page * self.page_size + e.start % self.page_size
                else:
                    slot_maps[g][t0 : t0 + n] = self.cache_manager.slots_for(rc, g, e.start, n)
                count = min(len(table), widths[g])
                # A buffer that is filled step after step (a decode graph's) remembers what each
                # row holds: the same request in the same row only gets its new entries written
                # (and the entries a window gave back), not its whole table again.
                mark = None if row_marks is None else row_marks[g].get(b)
                if mark is not None and mark[0] is rc and mark[1] <= count and mark[2] <= rc.first_held[g]:
                    if mark[1] < count:
                        tables[g][b, mark[1] : count] = table[mark[1] : count]
                    if mark[2] < rc.first_held[g]:
                        tables[g][b, mark[2] : min(rc.first_held[g], count)] = -1
                else:
                    tables[g][b, :count] = table[:count]
                    tables[g][b, count:] = -1
                if row_marks is not None:
                    row_marks[g][b] = (rc, count, rc.first_held[g])
            if rc.fresh_slot:
                self.cache_tensors.zero_slot(rc.slot)
                rc.fresh_slot = False
            t0 += n
        # padding lanes of a fixed-size layout
        nb = len(entries)
        if t0 < layout.T:
            tok[t0:] = 0
            pos[t0:] = 0
            sidx[t0:] = -1
            for g in range(len(self.groups)):
                slot_maps[g][t0:] = -1
        if nb < B:
            cu[nb + 1 :] = t0
            ctx_lens[nb:] = 0
            slots[nb:] = 0
            for g in range(len(self.groups)):
                tables[g][nb:] = -1
                if row_marks is not None:
                    for b in range(nb, B):
                        row_marks[g].pop(b, None)
        if row_base is None and r0 < layout.R:
            rows[r0:] = 0
        return feeds

    def _context(self, dev: torch.Tensor, layout: _Layout, max_q: int, max_context: int) -> StepContext:
        B = layout.B
        groups = [
            GroupTables(
                block_table=layout.view(dev, f"table{g}").view(B, layout.widths[g]),
                slot_mapping=layout.view(dev, f"slots{g}"),
            )
            for g in range(len(self.groups))
        ]
        return StepContext(
            num_tokens=layout.T,
            num_seqs=B,
            token_ids=layout.view(dev, "token_ids"),
            positions=layout.view(dev, "positions"),
            seq_index=layout.view(dev, "seq_index"),
            cu_seqlens_q=layout.view(dev, "cu_seqlens_q"),
            context_lens=layout.view(dev, "context_lens"),
            state_slots=layout.view(dev, "state_slots"),
            groups=groups,
            page_size=self.page_size,
            max_seqlen_q=max_q,
            max_context_len=max_context,
            decode_only=max_q == 1,
        )

    # -- decode graphs ------------------------------------------------------------------------

    def _graph_bucket(self, entries: Sequence[StepEntry]) -> Optional[int]:
        if not self.use_graphs:
            return None
        B = len(entries)
        if B > self.graph_buckets[-1]:
            return None
        for e in entries:
            if len(e.tokens) != 1 or e.start + 1 > self.max_model_len:
                return None
        for b in self.graph_buckets:
            if b >= B:
                return b
        return None

    def _capture(self, bucket: int) -> "_DecodeGraph":
        """Captures one decode step for `bucket` sequences: every kernel from the embedding to
        the logits, reading its indices from one static buffer."""
        from tokensprint_b200 import ops

        width = max(1, -(-self.max_model_len // self.page_size))
        layout = _Layout(bucket, bucket, bucket, [width] * len(self.groups))
        dev = torch.zeros(layout.total, dtype=torch.int32, device=self.device)
        host = torch.empty(layout.total, dtype=torch.int32, pin_memory=True)
        # a harmless content for the warm-up and the capture: padding lanes only
        self._fill(host.numpy(), layout, [], [])
        host.numpy()[layout.sections["rows"][0] : layout.sections["rows"][0] + bucket] = np.arange(bucket)
        dev.copy_(host)
        step = self._context(dev, layout, 1, self.max_model_len)
        step.rows_all = True  # in a graph every lane's logits are computed
        rows = layout.view(dev, "rows")
        torch.cuda.synchronize(self.device)
        # The warm-up runs on the stream the capture will use: it loads libraries, sets kernel
        # attributes, fills the allocator and, above all, creates and zeroes the kernels' per-stream
        # scratch (ticket counters, partial sums, error word) outside any capture, so that no graph
        # holds the only memset of a buffer that later graphs rely on.
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(self.device)
        side = self._capture_stream
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.model.forward(step, self.layer_caches, rows, bucket)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(graph, pool=self._graph_pool, stream=side):
            logits = self.model.forward(step, self.layer_caches, rows, bucket)
        kernels = ops.launch_count - before
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        return _DecodeGraph(bucket, layout, dev, host, graph, logits, kernels, row_marks=[{} for _ in self.groups])

    def capture_graphs(self, largest_batch: Optional[int] = None) -> int:
        """Captures the decode graphs of every batch bucket up to `largest_batch` now (the reference
        captures at start-up too: engine/generation/model_runner.py:310-390), so that no step of a
        run pays for a capture.  Returns how many graphs there are."""
        if not self.use_graphs:
            return 0
        for bucket in self.graph_buckets:
            if largest_batch is not None and bucket > max(largest_batch, 1) and any(b >= largest_batch for b in self._graphs):
                break
            if bucket not in self._graphs:
                self._graphs[bucket] = self._capture(bucket)
        return len(self._graphs)

    def _step_graph(self, bucket: int, entries: Sequence[StepEntry], fed_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        g = self._graphs.get(bucket)
        if g is None:
            g = self._graphs[bucket] = self._capture(bucket)
        if g.event is not None:
            g.event.synchronize()
        feeds = self._fill(g.host.numpy(), g.layout, entries, [1] * len(entries), g.row_marks)
        # in a graph every lane's logits are computed; the wanted ones are picked afterwards
        rows_off = g.layout.sections["rows"][0]
        g.host.numpy()[rows_off : rows_off + bucket] = np.arange(bucket)
        g.dev.copy_(g.host, non_blocking=True)
        self.h2d_bytes += g.layout.total * 4
        if g.event is None:
            g.event = torch.cuda.Event()
        g.event.record()
        self._feed(g.dev, g.layout, feeds, fed_ids)
        g.graph.replay()
        self.graph_launches += g.kernels
        wanted = [b for b, e in enumerate(entries) if len(e.want)]
        if len(wanted) == len(entries):
            return g.logits[: len(entries)]
        if not wanted:
            return torch.empty((0, self.vocab_size), device=self.device, dtype=torch.float32)
        return g.logits.index_select(0, torch.tensor(wanted, device=self.device))

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], fed_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Float32 logits [wanted, vocab], in the order of the entries and of their `want`.
        `fed_ids` (int32, on the device): where entries with `feed` take their token from."""
        self.steps_run += 1
        bucket = self._graph_bucket(entries)
        if bucket is not None:
            for e in entries:
                if e.cache.released or e.start + 1 > e.cache.num_tokens or not (e.feed >= 0 or 0 <= e.tokens[0] < self.vocab_size):
                    raise ValueError(f"request {e.cache.request!r}: bad decode entry")
                if any(w != 0 for w in e.want):
                    raise ValueError(f"request {e.cache.request!r}: wanted place outside its 1 token")
            return self._step_graph(bucket, entries, fed_ids)
        step, rows, R = self.build_context(entries, fed_ids)
        with self.model.chain_scope(step.num_tokens):
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
