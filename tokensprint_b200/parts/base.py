"""Interfaces of the parts a layer is put together from, and their registries.

A layer is a *block* (the arrangement) around a *mixer* (attention here), a
*feed-forward* and *norms*; a mixer may use a *position encoding*.  Each kind has a
registry from a name to a class; a `PartSpec` (name + parameters) picks one, layer by
layer, so one model can mix different parts.  No part knows which model it is in: it
gets its sizes and constants as parameters and its tensor names as a table.

Activations are [tokens, width] in the compute dtype (bfloat16 or float32); the
residual stream is float32.  What a part needs of one step (positions, which request a
token belongs to, block tables, state slots) comes in a `StepContext`.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Optional

import torch

# ---------------------------------------------------------------------------
# specifications (pure data; safe to build without a GPU)


@dataclass(frozen=True)
class PartSpec:
    """Which registered part, with which parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part wants from the checkpoint.

    role: "matrix" is cast to the compute dtype; "vector" is held in float32 (a stored
    float32 stays exact, a stored bfloat16 widens without loss); "table" is held as int32.
    """

    name: str
    shape: tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class CacheNeed:
    """What one run of a mixer needs from the cache manager.

    kind "full": all keys stay; "window": keys older than `window` positions before the
    next query may be given back; "none": no pages.  `state_shape` asks for a slot of
    that fixed shape per request (None: no state).

    What is paged per token: `k_row` is the shape of one token's entry in the first pool and
    `v_row` that of the second pool (None: the mixer pages one tensor only, e.g. a latent).  The
    two may differ (values narrower than keys).  An attention mixer gives `kv_heads` and
    `head_dim` instead, which stand for k_row = v_row = (kv_heads, head_dim).
    """

    kind: str = "none"
    window: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    state_shape: Optional[tuple[int, ...]] = None
    state_dtype: torch.dtype = torch.float32
    k_row: Optional[tuple[int, ...]] = None
    v_row: Optional[tuple[int, ...]] = None
    single_pool: bool = False  # True: only the first pool exists (v_row stays None)

    def __post_init__(self) -> None:
        if self.kind == "none":
            return
        if self.k_row is None:
            if self.kv_heads <= 0 or self.head_dim <= 0:
                raise ValueError("a paged cache needs k_row, or kv_heads and head_dim")
            object.__setattr__(self, "k_row", (int(self.kv_heads), int(self.head_dim)))
        else:
            object.__setattr__(self, "k_row", tuple(int(n) for n in self.k_row))
        if self.v_row is None and not self.single_pool:
            object.__setattr__(self, "v_row", self.k_row)
        elif self.v_row is not None:
            object.__setattr__(self, "v_row", tuple(int(n) for n in self.v_row))

    @property
    def group_key(self) -> tuple[str, int]:
        return (self.kind, self.window if self.kind == "window" else 0)

    @property
    def token_elements(self) -> int:
        """Elements one token occupies in the pools of this cache."""
        n = 0
        for row in (self.k_row, self.v_row):
            if row is not None:
                size = 1
                for extent in row:
                    size *= extent
                n += size
        return n


# ---------------------------------------------------------------------------
# what one step brings


@dataclass
class GroupTables:
    """Block table and new-token slots of one cache group for this step."""

    block_table: torch.Tensor  # [B, max_blocks] i32, -1 where no page is held
    slot_mapping: torch.Tensor  # [T] i32, page * page_size + offset, -1 = do not store


@dataclass
class StepContext:
    """Device-side description of one batch of (request, its next tokens)."""

    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor  # [T] i32
    positions: torch.Tensor  # [T] i32 absolute position of each token in its request
    seq_index: torch.Tensor  # [T] i32 row of the batch each token belongs to (-1: padding)
    cu_seqlens_q: torch.Tensor  # [B+1] i32 prefix sums of the tokens per request
    context_lens: torch.Tensor  # [B] i32 tokens in the cache after this step
    state_slots: torch.Tensor  # [B] i32 per-request state slot
    groups: list[GroupTables]
    page_size: int
    max_seqlen_q: int
    max_context_len: int
    # host copies for parts that plan on the host (toy parts in tests do)
    host_seq_starts: list[int] = field(default_factory=list)
    host_seq_lens: list[int] = field(default_factory=list)
    host_state_slots: list[int] = field(default_factory=list)
    decode_only: bool = False
    # how many sequences at the front of the batch bring exactly one token each (the runner puts them
    # first in a step that also carries portions of prompts, so that a mixer may treat the two kinds apart)
    decode_seqs: int = 0
    rows_all: bool = False  # the logits of every token are wanted, in the tokens' order
    # A hint, set by whoever calls a part: the first weight matrix that will be read after the
    # part returns (the part may hand it to its last product for prefetching; may be None).
    weight_after: Optional[torch.Tensor] = None
    # Likewise the norm that will read the residual stream after the part returns (a block's
    # last part may prepare that norm's input, see ResidualNorm).
    norm_after: Optional["Norm"] = None
    # What a part computes once in a step and parts of its kind in other layers use again (the key
    # names the thing and the constants it was made from); it lives as long as the step.
    shared: dict = field(default_factory=dict)


@dataclass
class NormParams:
    """What a norm of the form x * rsqrt(mean(x^2) + eps) * weight is made of, for a part that
    offers to fold it into its own kernels."""

    weight: torch.Tensor  # [width] float32
    eps: float
    width: int


@dataclass
class ResidualNorm:
    """A request to a part's last product: do not return the branch output, add it into the
    float32 residual `hidden` yourself and prepare the input of the norm that follows."""

    hidden: torch.Tensor  # [T, width] float32, updated in place
    norm: NormParams


@dataclass
class PreNormed:
    """Rows on which a norm is all but done: `x` = bf16(hidden * norm weight) and `ssq` the sums
    of squares of the hidden rows per 128 columns ([tiles, T] float32); the 1/rms that is still
    missing is a factor per row, which a product of x with a matrix can apply to its result."""

    x: torch.Tensor
    ssq: torch.Tensor
    width: int
    eps: float


@dataclass
class LayerCache:
    """What one run of a mixer may touch of the cache."""

    group: int = -1  # index into StepContext.groups; -1: no pages
    k_pages: Optional[torch.Tensor] = None  # [pages, page, *k_row] (attention: [pages, page, kv_heads, head_dim])
    v_pages: Optional[torch.Tensor] = None  # [pages, page, *v_row], or None for a cache of one pool
    state: Optional[torch.Tensor] = None  # [slots, *state_shape]
    writes: bool = True  # False: reads a cache that another run filled


# ---------------------------------------------------------------------------
# part interfaces


class Part:
    """Base of all parts: declares its tensors and takes them once loaded."""

    # True when a decode step of this part is a fixed sequence of kernels that read all
    # per-step values from device memory (no host decisions, no shapes that depend on the
    # data): only a model whose parts all say so has its decode steps captured in CUDA graphs.
    graph_safe = False

    # True when the part touches the tensors it is handed (inputs, the residual stream, the cache)
    # only through the ops of this package.  Those launch any chained products that are still
    # pending before they run (ops.gemm_chain); before a part that does not say so, its caller
    # launches them itself.  A part written with torch operations leaves this False.
    reads_through_ops = False

    def first_weight(self) -> Optional[torch.Tensor]:
        """The first large weight this part reads in a step, for the part before it to prefetch."""
        return None

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """`tensors` maps the declared names to device tensors."""


class Norm(Part):
    def params(self) -> Optional[NormParams]:
        """The norm's weight, eps and width if it is a plain RMS norm that other parts may fold
        into their kernels; None keeps it a step of its own."""
        return None

    def forward(
        self,
        hidden: torch.Tensor,
        delta: Optional[torch.Tensor],
        out: torch.Tensor,
        row_index: Optional[torch.Tensor] = None,
    ) -> None:
        """hidden (float32 residual) += delta if given; out = norm(hidden)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Either hands rotary parameters to the fused kernel or rewrites q and k itself."""

    def rotary_inv_freq(self) -> Optional[torch.Tensor]:
        """[rot/2] float32 inverse frequencies for the fused rotate-half kernel, or None."""
        return None

    def rotary_cos_sin(self, step: StepContext) -> Optional[torch.Tensor]:
        """[T, rot/2, 2] float32 cosines and sines of the step's angles (position * inverse frequency)
        for a kernel that would otherwise compute them itself, or None."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, step: StepContext) -> None:
        """In-place encoding of q [T,nq,d] and k [T,nkv,d] for encodings the kernel lacks."""
        raise NotImplementedError


class Mixer(Part):
    # True if forward() also takes `x` as PreNormed and a keyword `fold: ResidualNorm`, and then
    # may return a PreNormed instead of its output (see blocks.PreNormBlock); False: plain
    # tensors in and out, the block does the norms and the residual sums around it.
    folds_norms = False

    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    folds_norms = False  # as for Mixer

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Transform(Part):
    """A step on the way into or out of the stack of blocks that belongs to no layer: what an
    architecture does to the embedding rows before the first block (a multiplier, an added
    table) or to the logits after the head (a scale, a soft cap, a bias).  A `ModelSpec` names
    them as `embedding_transform` and `logits_transform`; the model calls them and knows
    nothing of what they do."""

    def forward(self, x: torch.Tensor, step: Optional[StepContext]) -> torch.Tensor:
        """Returns the transformed tensor (it may be `x`, changed in place).  Embedding rows:
        float32 [T, width] with the step's context; logits: float32 [rows, vocab], step None."""
        raise NotImplementedError


class Block(Part):
    """An arrangement of mixer, feed-forward and norms around the residual stream.

    A block sets `graph_safe` from the parts it holds."""

    mixer: Mixer

    def entry_norm(self) -> Optional["Norm"]:
        """The norm that reads the residual stream first in this block, if the part before may
        prepare its input (see ResidualNorm); None: nobody may."""
        return None

    def forward(
        self,
        hidden: torch.Tensor,
        pending,
        step: StepContext,
        cache: LayerCache,
    ):
        """Runs the layer on the float32 residual `hidden` ([T,H], updated in place).

        `pending` is a branch output not yet added to `hidden` (the next norm adds it
        in the same pass); the return value is this layer's own pending output.  A block that
        names its entry_norm() may be handed a PreNormed for it instead, and a block may return
        one made for `step.norm_after`.
        """
        raise NotImplementedError


# ---------------------------------------------------------------------------
# registries


@dataclass
class BuildContext:
    """What a part's constructor may ask about the run it is built for."""

    device: torch.device
    dtype: torch.dtype  # compute dtype: torch.bfloat16 or torch.float32


PartFactory = Callable[..., Part]

MIXERS: dict[str, PartFactory] = {}
FEED_FORWARDS: dict[str, PartFactory] = {}
NORMS: dict[str, PartFactory] = {}
POSITION_ENCODINGS: dict[str, PartFactory] = {}
BLOCKS: dict[str, PartFactory] = {}
TRANSFORMS: dict[str, PartFactory] = {}

_TABLES = {
    "mixer": MIXERS,
    "feed_forward": FEED_FORWARDS,
    "norm": NORMS,
    "position_encoding": POSITION_ENCODINGS,
    "block": BLOCKS,
    "transform": TRANSFORMS,
}


def register_part(category: str, name: str, *, replace: bool = False) -> Callable[[PartFactory], PartFactory]:
    """Decorator: `@register_part("mixer", "attention")` on a class or factory.

    The factory is called as `factory(build_ctx, **spec.params)`.
    """
    table = _TABLES[category]

    def _register(factory: PartFactory) -> PartFactory:
        if name in table and not replace:
            raise ValueError(f"{category} '{name}' already registered.")
        table[name] = factory
        return factory

    return _register


def unregister_part(category: str, name: str) -> None:
    _TABLES[category].pop(name, None)


def build_part(category: str, spec: PartSpec, ctx: BuildContext) -> Part:
    table = _TABLES[category]
    if spec.kind not in table:
        raise ValueError(f"Unknown {category} '{spec.kind}'. Registered: {sorted(table)}")
    return table[spec.kind](ctx, **dict(spec.params))
