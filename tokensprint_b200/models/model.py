"""The runtime model: parts built from a ModelSpec, weights loaded, one forward per step."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Hashable, Optional

import torch

import tokensprint_b200.parts  # noqa: F401  (registers the built-in parts)
from tokensprint_b200 import ops
from tokensprint_b200.models.spec import ModelSpec
from tokensprint_b200.parts.base import BuildContext, CacheNeed, LayerCache, PreNormed, StepContext, TensorSpec, build_part
from tokensprint_b200.parts.linear import folding_possible, linear_float32_out, linear_scaled
from tokensprint_b200.weights.loader import LoadedTensors, WeightSource, check_tensors


@dataclass(frozen=True)
class CachePlanEntry:
    """One cache of the model: what it must hold and which run fills it."""

    need: CacheNeed
    writer_run: int


class Model:
    """Embedding -> blocks in run order -> final norm -> head (engine/model.py:58-86).

    Owns no cache: `forward` gets the step's context and one `LayerCache` per run.
    """

    def __init__(self, spec: ModelSpec, device: torch.device | str, dtype: torch.dtype) -> None:
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, got {dtype}")
        self.spec = spec
        self.device = torch.device(device)
        self.dtype = dtype
        ctx = BuildContext(device=self.device, dtype=dtype)
        self.blocks = [build_part("block", s, ctx) for s in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, ctx)
        self.embedding_transform = None if spec.embedding_transform is None else build_part("transform", spec.embedding_transform, ctx)
        self.logits_transform = None if spec.logits_transform is None else build_part("transform", spec.logits_transform, ctx)
        self._transforms = [t for t in (self.embedding_transform, self.logits_transform) if t is not None]
        self.graph_safe = (all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe
                           and all(t.graph_safe for t in self._transforms))
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

        # Which cache each run uses.
        keys: list[Hashable] = []
        self.run_cache: list[int] = []
        for i, run in enumerate(spec.run_order):
            key: Hashable = ("own", i) if run.cache is None else ("shared", run.cache)
            if key not in keys:
                keys.append(key)
            self.run_cache.append(keys.index(key))
        plan: list[Optional[CachePlanEntry]] = [None] * len(keys)
        for i, run in enumerate(spec.run_order):
            need = self.blocks[run.layer].mixer.cache_need()
            c = self.run_cache[i]
            if run.writes_cache:
                if plan[c] is not None:
                    raise ValueError(f"cache {keys[c]} has two writing runs ({plan[c].writer_run} and {i})")
                plan[c] = CachePlanEntry(need, i)
        for i, run in enumerate(spec.run_order):
            c = self.run_cache[i]
            if plan[c] is None:
                raise ValueError(f"run {i} reads cache {keys[c]} that no run writes")
            need = self.blocks[run.layer].mixer.cache_need()
            w = plan[c].need
            if (need.group_key, need.k_row, need.v_row, need.state_shape) != (w.group_key, w.k_row, w.v_row, w.state_shape):
                raise ValueError(f"run {i} and run {plan[c].writer_run} share a cache but need different ones")
        self.cache_plan: list[CachePlanEntry] = [p for p in plan if p is not None]

    # -- weights --------------------------------------------------------------

    def tensor_specs(self) -> list[TensorSpec]:
        return self.spec.tensor_specs()

    def load(self, source: WeightSource) -> None:
        specs = self.tensor_specs()
        check_tensors(specs, source.shapes(), ignorable=self.spec.ignorable_tensors, where=source.where)
        tensors = LoadedTensors(source, specs, self.device, self.dtype)
        self.embedding = tensors.keep(self.spec.embedding)
        # Tied: one buffer serves the table and the head (engine/nn/layers.py:22-23).
        self.head = self.embedding if self.spec.lm_head is None else tensors.keep(self.spec.lm_head)
        for block in self.blocks:
            block.load(tensors)
        self.final_norm.load(tensors)
        for transform in self._transforms:
            transform.load(tensors)

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once (the decode roofline's numerator)."""
        seen: set[int] = set()
        total = 0

        def walk(obj) -> None:
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor):
                    if v.data_ptr() not in seen:
                        seen.add(v.data_ptr())
                        total += v.numel() * v.element_size()
                elif hasattr(v, "tensor_specs") and not isinstance(v, type):
                    walk(v)

        for b in self.blocks:
            walk(b)
        walk(self.final_norm)
        for transform in self._transforms:
            walk(transform)
        if self.head is not None and self.head.data_ptr() not in seen:
            total += self.head.numel() * self.head.element_size()
        return total

    # -- one step ---------------------------------------------------------------

    def forward_hidden(self, step: StepContext, caches: list[LayerCache]) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Runs the blocks; returns the float32 residual and the last branch not yet added."""
        T = step.num_tokens
        step.shared.clear()  # what parts share lasts one run of the blocks (a step's description may be run again: warm-up, then capture)
        hidden = torch.empty((T, self.spec.hidden_size), device=self.device, dtype=torch.float32)
        ops.embed_gather(hidden, self.embedding, step.token_ids)
        if self.embedding_transform is not None:
            hidden = self.embedding_transform.forward(hidden, step)
        pending = None
        order = self.spec.run_order
        # the final norm may be prepared by the last block when every row's logits are wanted
        # and the head product is one that applies the missing 1/rms
        fold_final = step.rows_all and folding_possible(T, self.dtype, self.head)
        for i, run in enumerate(order):
            # what is read after this block: the next block's first matrix and first norm, or the head and the final norm
            last = i + 1 == len(order)
            step.weight_after = self.head if last else self.blocks[order[i + 1].layer].first_weight()
            step.norm_after = (self.final_norm if fold_final else None) if last else self.blocks[order[i + 1].layer].entry_norm()
            block = self.blocks[run.layer]
            if not block.reads_through_ops:
                ops.flush_gemm_chain()
            pending = block.forward(hidden, pending, step, caches[i])
        step.weight_after = step.norm_after = None
        return hidden, pending

    def chain_scope(self, num_tokens: int) -> "ops.gemm_chain":
        """The context in which a step of `num_tokens` tokens runs: where ops.GEMM_CHAIN is switched on,
        the engine's own products of a step of few tokens in bfloat16 that follow one another are
        launched together (ops.gemm_chain)."""
        return ops.gemm_chain(self.device, enabled=ops.GEMM_CHAIN and folding_possible(num_tokens, self.dtype))

    def logits(self, hidden: torch.Tensor, pending, rows: torch.Tensor, num_rows: int) -> torch.Tensor:
        """Final norm on the wanted rows only, then the head (and what the architecture does to the
        logits after it): float32 [R, V] (engine/model.py:75-86).
        `pending`: the last branch output not yet added, or a PreNormed of the final norm."""
        if not self.final_norm.reads_through_ops:
            ops.flush_gemm_chain()
        out = self._head_product(hidden, pending, rows, num_rows)
        ops.flush_gemm_chain()  # the logits leave this package's ops here
        if self.logits_transform is not None:
            out = self.logits_transform.forward(out, None)
        return out

    def _head_product(self, hidden: torch.Tensor, pending, rows: torch.Tensor, num_rows: int) -> torch.Tensor:
        if isinstance(pending, PreNormed):
            if num_rows == hidden.shape[0] and folding_possible(num_rows, self.dtype, self.head):
                return linear_scaled(pending, self.head, float32_out=True)
            pending = None  # `hidden` is complete: norm it as usual
        normed = torch.empty((num_rows, self.spec.hidden_size), device=self.device, dtype=self.dtype)
        self.final_norm.forward(hidden, pending, normed, row_index=rows)
        return linear_float32_out(normed, self.head)

    def forward(self, step: StepContext, caches: list[LayerCache], rows: torch.Tensor, num_rows: int) -> torch.Tensor:
        with self.chain_scope(step.num_tokens):
            hidden, pending = self.forward_hidden(step, caches)
            return self.logits(hidden, pending, rows, num_rows)
