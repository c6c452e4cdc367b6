"""Grouped-query attention over the paged cache, as a mixer part."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import (
    BuildContext,
    CacheNeed,
    LayerCache,
    Mixer,
    PartSpec,
    ResidualNorm,
    StepContext,
    TensorSpec,
    build_part,
    register_part,
)
from tokensprint_b200.parts.linear import folding_possible, linear, linear_into_residual, linear_scaled


@register_part("mixer", "attention")
class AttentionMixer(Mixer):
    """q/k/v projections, optional per-head q/k RMSNorm, position encoding, store of keys
    and values into the cache, causal softmax attention over the cache, output projection
    (engine/nn/attention.py:164-200).

    Parameters: `hidden_size`, `num_heads`, `num_kv_heads`, `head_dim` (free of the width:
    num_heads * head_dim need not equal hidden_size), `qk_norm` + `qk_norm_eps`, `window`
    (0: every earlier key; n: the last n keys, the query's own included), `scale`
    (default head_dim^-0.5, engine/nn/sdpa.py:56), `position` (a position-encoding spec or
    None) and the checkpoint names of the tensors.  q, k, v weights are stacked at load
    into one [(nq + 2 nkv) d, H] matrix.
    """

    folds_norms = True
    # its own kernels only; a position encoding that rewrites q and k itself gets them from a kernel
    # that has run (not from a product that may still wait in a chain)
    reads_through_ops = True

    def __init__(
        self,
        ctx: BuildContext,
        *,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        q: str,
        k: str,
        v: str,
        o: str,
        qk_norm: bool = False,
        qk_norm_eps: float = 1e-6,
        q_norm: Optional[str] = None,
        k_norm: Optional[str] = None,
        window: int = 0,
        scale: Optional[float] = None,
        position: Optional[PartSpec] = None,
    ) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} heads are no multiple of {num_kv_heads} key/value heads")
        if qk_norm and (q_norm is None or k_norm is None):
            raise ValueError("attention: qk_norm needs the names of both norm weights")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.num_kv_heads, self.head_dim = int(num_kv_heads), int(head_dim)
        self.qk_norm, self.qk_norm_eps = bool(qk_norm), float(qk_norm_eps)
        self.window = int(window or 0)
        self.scale = float(scale) if scale is not None else float(head_dim) ** -0.5
        self.names = {"q": q, "k": k, "v": v, "o": o, "q_norm": q_norm, "k_norm": k_norm}
        self.position = build_part("position_encoding", position, ctx) if position is not None else None
        # the kernels of this mixer read everything a step needs from device memory; a position
        # encoding that rewrites q and k itself decides for itself
        self.graph_safe = self.position is None or self.position.graph_safe
        self.dtype = ctx.dtype
        self.qkv_weight: Optional[torch.Tensor] = None
        self.o_weight: Optional[torch.Tensor] = None
        self.q_norm_weight: Optional[torch.Tensor] = None
        self.k_norm_weight: Optional[torch.Tensor] = None

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.qkv_weight

    def cache_need(self) -> CacheNeed:
        kind = "window" if self.window > 0 else "full"
        return CacheNeed(kind=kind, window=self.window, kv_heads=self.num_kv_heads, head_dim=self.head_dim)

    def tensor_specs(self) -> list[TensorSpec]:
        H, nq, nkv, d = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
        specs = [
            TensorSpec(self.names["q"], (nq * d, H)),
            TensorSpec(self.names["k"], (nkv * d, H)),
            TensorSpec(self.names["v"], (nkv * d, H)),
            TensorSpec(self.names["o"], (H, nq * d)),
        ]
        if self.qk_norm:
            specs.append(TensorSpec(self.names["q_norm"], (d,), "vector"))
            specs.append(TensorSpec(self.names["k_norm"], (d,), "vector"))
        if self.position is not None:
            specs.extend(self.position.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.qkv_weight = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.o_weight = tensors[n["o"]]
        if self.qk_norm:
            self.q_norm_weight = tensors[n["q_norm"]]
            self.k_norm_weight = tensors[n["k_norm"]]
        if self.position is not None:
            self.position.load(tensors)

    def can_fold(self, num_tokens: int, dtype: torch.dtype) -> bool:
        return folding_possible(num_tokens, dtype, self.qkv_weight, self.o_weight)

    def forward(self, x, step: StepContext, cache: LayerCache, fold: Optional[ResidualNorm] = None):
        """x: [T, H], or a PreNormed (its missing 1/rms is applied by the q/k/v product).  With
        `fold` the output projection adds its result into fold.hidden itself and the PreNormed of
        the norm that follows is returned instead of the branch output."""
        if cache.k_pages is None or cache.group < 0:
            raise ops.KernelError("attention: this mixer needs cache pages (none were bound to its run)")
        xt = x if isinstance(x, torch.Tensor) else x.x
        T = xt.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        tables = step.groups[cache.group]
        q = torch.empty((T, nq * d), device=xt.device, dtype=xt.dtype)
        inv_freq = self.position.rotary_inv_freq() if self.position is not None else None
        fused = self.position is None or inv_freq is not None
        if (fused and cache.writes and d == ops.GEMM_QK_ROPE_HEAD_DIM and (inv_freq is None or inv_freq.numel() == d // 2)
                and folding_possible(T, xt.dtype, self.qkv_weight)):
            # few tokens, heads of 128: norm, rotation and the store are the projection's own epilogue
            pre = None if isinstance(x, torch.Tensor) else x
            ops.gemm_qk_rope_store(
                xt, self.qkv_weight, q, cache.k_pages, cache.v_pages, tables.slot_mapping, step.positions,
                self.q_norm_weight, self.k_norm_weight, self.qk_norm_eps, inv_freq, nq, nkv,
                scale_ssq=None if pre is None else pre.ssq, scale_width=1 if pre is None else pre.width,
                scale_eps=0.0 if pre is None else pre.eps, prefetch=self.o_weight,
                cos_sin=None if inv_freq is None else self.position.rotary_cos_sin(step))
            out = torch.empty((T, nq * d), device=xt.device, dtype=xt.dtype)
            self._attend(q, out, step, cache, tables)
            if fold is not None:
                return linear_into_residual(out, self.o_weight, fold, next_weight=step.weight_after)
            return linear(out, self.o_weight, next_weight=step.weight_after)
        qkv = linear_scaled(x, self.qkv_weight, next_weight=self.o_weight)
        if fused and cache.writes:
            ops.qk_norm_rope_store(
                qkv, q, cache.k_pages, cache.v_pages, tables.slot_mapping, step.positions,
                self.q_norm_weight, self.k_norm_weight, self.qk_norm_eps, inv_freq, nq, nkv, d)
        elif fused:
            # Reads a cache that another run filled: only the queries are prepared.
            self._queries_only(qkv, q, step, inv_freq)
        else:
            self._unfused(qkv, q, step, cache, tables)
        out = torch.empty((T, nq * d), device=xt.device, dtype=xt.dtype)
        self._attend(q, out, step, cache, tables)
        if fold is not None:
            return linear_into_residual(out, self.o_weight, fold, next_weight=step.weight_after)
        return linear(out, self.o_weight, next_weight=step.weight_after)

    # -- attention proper ---------------------------------------------------

    def _attend(self, q, out, step: StepContext, cache: LayerCache, tables) -> None:
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        if q.dtype == torch.bfloat16 and ops.attention_mma_supported(d):
            B, singles = step.num_seqs, step.decode_seqs
            few_rows = (nq // nkv) <= ops.attention_decode_rows(d)
            if step.max_seqlen_q * (nq // nkv) <= ops.attention_decode_rows(d):
                # few rows per sequence: the decode kernels, keys spread over CTAs
                self._attend_decode(q, out, step, cache, tables, 0, B, step.max_seqlen_q)
                return
            prompts_on_tcgen05 = ops.attention_tcgen05_supported(nq, nkv, d, step.page_size)
            if prompts_on_tcgen05 and few_rows and 0 < singles < B:
                # Single decoded tokens beside portions of prompts (the runner put the single tokens'
                # requests first): each kind to its own kernel.  Through the prompt kernel a decoded
                # token is a CTA that walks its whole context for a tile of a few rows (measured at
                # Qwen3-14B's heads, 140 decoded tokens at context 1,500 beside 8 prompts of 1,000:
                # 587 us in one launch, 179 + 218 us in two).
                self._attend_decode(q[:singles], out[:singles], step, cache, tables, 0, singles, 1)
                ops.attention_prefill_tcgen05(
                    q, cache.k_pages, cache.v_pages, out, step.cu_seqlens_q[singles:], step.context_lens[singles:],
                    tables.block_table[singles:], step.page_size, B - singles, step.max_seqlen_q, nq, nkv, self.scale, self.window)
                return
            if prompts_on_tcgen05:
                # prompt portions: the tcgen05 kernel, where it takes the sizes
                ops.attention_prefill_tcgen05(
                    q, cache.k_pages, cache.v_pages, out, step.cu_seqlens_q, step.context_lens, tables.block_table,
                    step.page_size, step.num_seqs, step.max_seqlen_q, nq, nkv, self.scale, self.window)
                return
            ops.attention_paged_mma(
                q, cache.k_pages, cache.v_pages, out, step.cu_seqlens_q, step.context_lens, tables.block_table,
                step.seq_index, step.page_size, step.num_seqs, step.max_seqlen_q, nq, nkv, d, self.scale,
                self.window, 1, None, 0)
            return
        # float32 runs, and head sizes the tensor-core kernel does not take
        ops.attention_paged_simple(
            q, cache.k_pages, cache.v_pages, out, step.positions, step.seq_index, tables.block_table,
            step.page_size, self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window)

    def _attend_decode(self, q, out, step: StepContext, cache: LayerCache, tables, first: int, count: int, max_q: int) -> None:
        """Sequences [first, first + count) of the batch, each with at most `max_q` tokens (few enough
        rows for the decode kernels); q and out hold exactly their tokens."""
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        cu = step.cu_seqlens_q[first : first + count + 1]
        lens = step.context_lens[first : first + count]
        table = tables.block_table[first : first + count]
        seq_index = step.seq_index[: q.shape[0]] if first == 0 else step.seq_index
        # The count must not depend on the step's actual lengths (a captured graph is
        # replayed for all of them): plan for a typical context, each sequence then
        # divides its own keys evenly.
        context = ops.attention_decode_plan_context(step.max_context_len, self.window)
        splits = ops.attention_decode_splits(count, nkv, context, d)
        if (ops.attention_decode_prefers_flat(count, nkv, splits, d)
                and ops.attention_decode_flat_supported(nq, nkv, d, step.page_size, count, max_q)):
            # more (sequence, KV head) pairs than CTAs run at once: an even share of all key blocks per CTA
            ops.attention_decode_flat(
                q, cache.k_pages, cache.v_pages, out, cu, lens, table, seq_index, step.page_size, count, max_q, nq, nkv, d,
                self.scale, self.window)
            return
        scratch = None
        if splits > 1:
            scratch = torch.empty(ops.attention_scratch_floats(q.shape[0] * nq, splits, d), device=q.device, dtype=torch.float32)
        ops.attention_paged_mma(
            q, cache.k_pages, cache.v_pages, out, cu, lens, table, seq_index, step.page_size, count, max_q, nq, nkv, d,
            self.scale, self.window, splits, scratch, 0)

    # -- less common paths ----------------------------------------------------

    def _queries_only(self, qkv, q, step: StepContext, inv_freq) -> None:
        T = qkv.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        k_tmp = torch.empty((T, nkv, d), device=qkv.device, dtype=qkv.dtype)
        v_tmp = torch.empty((T, nkv, d), device=qkv.device, dtype=qkv.dtype)
        ops.qk_norm_rope_store(
            qkv, q, k_tmp, v_tmp, None, step.positions, self.q_norm_weight, self.k_norm_weight,
            self.qk_norm_eps, inv_freq, nq, nkv, d)

    def _unfused(self, qkv, q, step: StepContext, cache: LayerCache, tables) -> None:
        """A position encoding that the fused kernel does not know: norm into dense
        buffers, let the part rewrite q and k, then store keys and values."""
        T = qkv.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        k_tmp = torch.empty((T, nkv, d), device=qkv.device, dtype=qkv.dtype)
        v_tmp = torch.empty((T, nkv, d), device=qkv.device, dtype=qkv.dtype)
        ops.qk_norm_rope_store(
            qkv, q, k_tmp, v_tmp, None, step.positions, self.q_norm_weight, self.k_norm_weight,
            self.qk_norm_eps, None, nq, nkv, d)
        self.position.apply(q.view(T, nq, d), k_tmp, step)
        if cache.writes:
            kv = torch.cat([k_tmp.view(T, nkv * d), v_tmp.view(T, nkv * d)], dim=1).contiguous()
            scratch_q = torch.empty((T, 0), device=qkv.device, dtype=qkv.dtype)
            ops.qk_norm_rope_store(
                kv, scratch_q, cache.k_pages, cache.v_pages, tables.slot_mapping, step.positions,
                None, None, self.qk_norm_eps, None, 0, nkv, d)
