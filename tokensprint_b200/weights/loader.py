"""Weights by tensor name: from a safetensors folder, or random from a seed.

A model declares the tensors it wants (`TensorSpec`: name, shape, role).  A source
answers by name.  Before anything is copied the declared list is checked against what
the source has; one `WeightsError` lists every missing tensor, every unexpected tensor
and every wrong shape (the reference relies on `load_state_dict(strict=True)` for this,
engine/models/_api.py:45).

Dtypes on the device: a "matrix" takes the compute dtype of the run (bfloat16 stays
bfloat16 in a bfloat16 run); a "vector" (norm weights) is held in float32, so a tensor
stored in 32-bit stays so and a bfloat16 one widens exactly; a "table" is int32.

The reference has no random-weights mode (its model is `to_empty` until a checkpoint is
loaded, engine/models/_api.py:44).  Here `write_random_model` writes a model folder
(config.json + model.safetensors) from a config and a seed: matrices N(0, std),
vectors 1 + N(0, vector_std), each tensor from its own generator keyed by (seed, name),
so any reader of the folder and any direct user of `RandomSource` see the same values.
"""

from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Iterable, Mapping, Optional, Sequence

import torch

from tokensprint_b200.parts.base import TensorSpec
from tokensprint_b200.weights.safetensors_io import SafetensorsFolder, save_safetensors


class WeightsError(RuntimeError):
    """The checkpoint does not match the model; the message lists every difference."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str], wrong_shape: Sequence[str], where: str) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights in {where} do not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        super().__init__("\n".join(lines))


def check_tensors(
    specs: Iterable[TensorSpec],
    available: Mapping[str, tuple[int, ...]],
    *,
    ignorable: Iterable[str] = (),
    where: str = "the checkpoint",
) -> None:
    """Raises one WeightsError if names or shapes differ.  `ignorable` names may be present
    without being wanted (a stray lm_head.weight beside tied embeddings)."""
    wanted = {s.name: s for s in specs}
    ignorable = set(ignorable)
    missing = [n for n in wanted if n not in available]
    unexpected = [n for n in available if n not in wanted and n not in ignorable]
    wrong = [
        f"{n}: expected {list(wanted[n].shape)}, found {list(available[n])}"
        for n in wanted
        if n in available and tuple(available[n]) != tuple(wanted[n].shape)
    ]
    if missing or unexpected or wrong:
        raise WeightsError(sorted(missing), sorted(unexpected), wrong, where)


def _device_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role == "matrix":
        return compute_dtype
    if role == "vector":
        return torch.float32
    if role == "table":
        return torch.int32
    raise ValueError(f"unknown tensor role {role!r}")


class WeightSource:
    """Name -> tensor.  `shapes()` is cheap; `fetch` copies one tensor to the device."""

    where = "the weight source"

    def shapes(self) -> dict[str, tuple[int, ...]]:
        raise NotImplementedError

    def fetch(self, spec: TensorSpec, device: torch.device, compute_dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError


class FolderSource(WeightSource):
    def __init__(self, folder: str | Path) -> None:
        self.folder = SafetensorsFolder(folder)
        self.where = str(folder)

    def shapes(self) -> dict[str, tuple[int, ...]]:
        return {name: self.folder.shape(name) for name in self.folder.keys()}

    def fetch(self, spec: TensorSpec, device: torch.device, compute_dtype: torch.dtype) -> torch.Tensor:
        host = self.folder.tensor(spec.name)
        return host.to(device=device, dtype=_device_dtype(spec.role, compute_dtype)).contiguous()


def _name_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(
    spec: TensorSpec,
    seed: int,
    *,
    std: float = 0.02,
    vector_std: float = 0.05,
    device: torch.device | str = "cpu",
) -> torch.Tensor:
    """Float32 values of one tensor: N(0, std) for matrices, 1 + N(0, vector_std) for vectors.

    On the CPU the values depend only on (seed, name, shape).  Generating on a CUDA device
    is faster for full-size models and gives other (equally valid) values.
    """
    gen = torch.Generator(device=device)
    gen.manual_seed(_name_seed(seed, spec.name))
    if spec.role == "table":
        return torch.randint(0, 2**15, spec.shape, generator=gen, device=device, dtype=torch.int32)
    x = torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32)
    if spec.role == "vector":
        return 1.0 + vector_std * x
    return std * x


class RandomSource(WeightSource):
    """Seeded random weights without a file (the benchmark's full-size models)."""

    def __init__(
        self,
        specs: Iterable[TensorSpec],
        seed: int,
        *,
        std: float = 0.02,
        vector_std: float = 0.05,
        generate_on_device: bool = False,
    ) -> None:
        self.specs = {s.name: s for s in specs}
        self.seed, self.std, self.vector_std = seed, std, vector_std
        self.generate_on_device = generate_on_device
        self.where = f"random weights (seed {seed})"

    def shapes(self) -> dict[str, tuple[int, ...]]:
        return {n: tuple(s.shape) for n, s in self.specs.items()}

    def fetch(self, spec: TensorSpec, device: torch.device, compute_dtype: torch.dtype) -> torch.Tensor:
        where = device if self.generate_on_device else "cpu"
        x = random_tensor(spec, self.seed, std=self.std, vector_std=self.vector_std, device=where)
        return x.to(device=device, dtype=_device_dtype(spec.role, compute_dtype)).contiguous()


class LoadedTensors(Mapping):
    """Lazy name -> device tensor table handed to the parts; each fetch copies once."""

    def __init__(self, source: WeightSource, specs: Iterable[TensorSpec], device: torch.device, compute_dtype: torch.dtype) -> None:
        self._source = source
        self._specs = {s.name: s for s in specs}
        self._device = device
        self._dtype = compute_dtype
        self._kept: dict[str, torch.Tensor] = {}

    def __getitem__(self, name: str) -> torch.Tensor:
        if name in self._kept:
            return self._kept[name]
        return self._source.fetch(self._specs[name], self._device, self._dtype)

    def keep(self, name: str) -> torch.Tensor:
        """Fetches once and remembers: for tensors that two parts share (tied embeddings)."""
        if name not in self._kept:
            self._kept[name] = self._source.fetch(self._specs[name], self._device, self._dtype)
        return self._kept[name]

    def __iter__(self):
        return iter(self._specs)

    def __len__(self) -> int:
        return len(self._specs)


def write_random_model(
    folder: str | Path,
    config,
    seed: int,
    *,
    dtype: str | torch.dtype = "float32",
    std: float = 0.02,
    vector_std: float = 0.05,
    specs: Optional[Iterable[TensorSpec]] = None,
) -> Path:
    """Writes config.json and model.safetensors for `config` (a typed model config).

    The tensor list comes from the architecture's own model spec, so the folder holds
    exactly the names the loader will ask for.
    """
    from tokensprint_b200.config.registry import architecture_for

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    config.save(folder)
    if specs is None:
        arch = architecture_for(config.to_dict())
        specs = arch.build_spec(config).tensor_specs()
    if isinstance(dtype, str):
        dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]

    def tensors():
        for spec in specs:
            x = random_tensor(spec, seed, std=std, vector_std=vector_std)
            yield spec.name, (x if spec.role == "table" else x.to(dtype))

    save_safetensors(folder / "model.safetensors", tensors())
    return folder
