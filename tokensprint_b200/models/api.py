"""From a model folder (or a registered name) to a loaded model."""

from __future__ import annotations

from pathlib import Path
from typing import Any, Optional

import torch

from tokensprint_b200.config.engine_config import canonical_dtype
from tokensprint_b200.config.registry import architecture_for, load_model_config
from tokensprint_b200.models.model import Model
from tokensprint_b200.weights.loader import FolderSource, RandomSource, WeightSource

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def torch_dtype(name: str | torch.dtype) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    return TORCH_DTYPES[canonical_dtype(name)]


def build_model(config: Any, *, device: torch.device | str = "cuda", dtype: str | torch.dtype = "bfloat16") -> Model:
    """An unloaded model for a typed config; its architecture is the one the config names."""
    arch = architecture_for(config.to_dict())
    return Model(arch.build_spec(config), device, torch_dtype(dtype))


def load_model(
    model_dir: str | Path,
    *,
    device: torch.device | str = "cuda",
    dtype: str | torch.dtype = "bfloat16",
    source: Optional[WeightSource] = None,
) -> tuple[Model, Any]:
    """Reads `model_dir/config.json`, builds the model its architecture names and loads
    `model_dir/*.safetensors` by tensor name (engine/models/_api.py:31-59 of the reference,
    without the download and the tokenizer).  Returns the model and its typed config."""
    arch, config = load_model_config(model_dir)
    model = Model(arch.build_spec(config), device, torch_dtype(dtype))
    model.load(source if source is not None else FolderSource(model_dir))
    return model, config


def random_model(
    config: Any,
    seed: int,
    *,
    device: torch.device | str = "cuda",
    dtype: str | torch.dtype = "bfloat16",
    std: float = 0.02,
    vector_std: float = 0.05,
    generate_on_device: bool = False,
) -> Model:
    """A model with seeded random weights, without a file in between."""
    model = build_model(config, device=device, dtype=dtype)
    model.load(RandomSource(model.tensor_specs(), seed, std=std, vector_std=vector_std, generate_on_device=generate_on_device))
    return model
