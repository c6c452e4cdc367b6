"""What an architecture's builder returns: layers as data, and the order they run in."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from tokensprint_b200.parts.base import BuildContext, PartSpec, TensorSpec, build_part


@dataclass(frozen=True)
class RunSpec:
    """One entry of the run order.

    layer: index into `ModelSpec.layers` (a layer may be named by several entries: its
    weights are shared, each run has a cache of its own unless told otherwise).
    cache: id of the cache this run uses; None gives the run a fresh cache of its own.
    Two runs with the same id share it; the one with `writes_cache` fills it, the others
    read what it stored.
    """

    layer: int
    cache: Optional[int] = None
    writes_cache: bool = True


@dataclass
class ModelSpec:
    """A whole model as data: embedding, layers (block specs), run order, final norm, head."""

    vocab_size: int
    hidden_size: int
    embedding: str  # checkpoint name of the [V, H] table
    layers: list[PartSpec]  # block specs
    final_norm: PartSpec
    lm_head: Optional[str]  # checkpoint name of the [V, H] head; None: tied to the embedding
    run_order: list[RunSpec] = field(default_factory=list)
    max_positions: int = 0
    eos_token_id: int = -1
    # Names that may sit in a checkpoint without being used (lm_head beside tied embeddings).
    ignorable_tensors: tuple[str, ...] = ()
    # Optional "transform" parts: what happens to the embedding rows before the first block
    # (float32 [T, width]) and to the logits after the head (float32 [rows, vocab]).
    embedding_transform: Optional[PartSpec] = None
    logits_transform: Optional[PartSpec] = None

    def __post_init__(self) -> None:
        if not self.run_order:
            self.run_order = [RunSpec(layer=i) for i in range(len(self.layers))]
        for run in self.run_order:
            if not (0 <= run.layer < len(self.layers)):
                raise ValueError(f"run order names layer {run.layer}, the model has {len(self.layers)}")

    def tensor_specs(self) -> list[TensorSpec]:
        """Every tensor the model wants, each name once (built on a CPU context, no GPU needed)."""
        import torch

        ctx = BuildContext(device=torch.device("cpu"), dtype=torch.float32)
        specs: dict[str, TensorSpec] = {}

        def add(spec: TensorSpec) -> None:
            old = specs.get(spec.name)
            if old is not None and tuple(old.shape) != tuple(spec.shape):
                raise ValueError(f"tensor {spec.name} is declared with shapes {old.shape} and {spec.shape}")
            specs.setdefault(spec.name, spec)

        add(TensorSpec(self.embedding, (self.vocab_size, self.hidden_size)))
        for layer in self.layers:
            for s in build_part("block", layer, ctx).tensor_specs():
                add(s)
        for s in build_part("norm", self.final_norm, ctx).tensor_specs():
            add(s)
        for transform in (self.embedding_transform, self.logits_transform):
            if transform is not None:
                for s in build_part("transform", transform, ctx).tensor_specs():
                    add(s)
        if self.lm_head is not None:
            add(TensorSpec(self.lm_head, (self.vocab_size, self.hidden_size)))
        return list(specs.values())
