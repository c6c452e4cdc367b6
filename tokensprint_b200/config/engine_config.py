"""Engine options and sampling options.

Names and meanings follow engine/generation/config.py:7-55 of the reference.  What
differs: `kvcache_block_size` may be any positive number of tokens (the reference
demands a multiple of 256 for its attention library, config.py:38-42), there is no
`tensor_parallel_size` (one GPU), greedy sampling is allowed (`temperature == 0`;
the reference refuses it, config.py:13-15) and a `seed` keys the sampling noise.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

DTYPE_NAMES = {
    "bfloat16": "bfloat16",
    "bf16": "bfloat16",
    "float32": "float32",
    "fp32": "float32",
    "f32": "float32",
}


def canonical_dtype(name: str) -> str:
    """'bfloat16' or 'float32' from the spellings the command lines accept."""
    key = str(name).replace("torch.", "").lower()
    if key not in DTYPE_NAMES:
        raise ValueError(f"dtype must be one of {sorted(DTYPE_NAMES)}, got {name!r}")
    return DTYPE_NAMES[key]


@dataclass
class SamplingParams:
    temperature: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False
    seed: int = 0

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be >= 1, got {self.max_tokens}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 1e-10


@dataclass
class Config:
    model: str
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 512
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    enforce_eager: bool = False
    eos: int = -1
    kvcache_block_size: int = 16
    num_kvcache_blocks: int = -1
    chunked_prefill: bool = False
    dtype: str = "bfloat16"
    # Launch a step before the host has read the ids that the step before sampled (they are fed
    # on the device), so that the device does not wait for the host between steps.  A request's
    # end is then seen one step later; what that step computed for it is dropped.
    overlap_steps: bool = True

    def __post_init__(self) -> None:
        if not os.path.isdir(self.model):
            raise FileNotFoundError(f"Model directory does not exist: {self.model}")
        if self.kvcache_block_size < 1:
            raise ValueError(f"kvcache_block_size must be positive, got {self.kvcache_block_size}")
        if self.max_num_batched_tokens < 1 or self.max_num_seqs < 1 or self.max_model_len < 2:
            raise ValueError(
                "max_num_batched_tokens and max_num_seqs must be >= 1 and max_model_len >= 2, got "
                f"{self.max_num_batched_tokens}, {self.max_num_seqs}, {self.max_model_len}"
            )
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError(
                f"gpu_memory_utilization must be in (0, 1], got {self.gpu_memory_utilization}"
            )
        self.dtype = canonical_dtype(self.dtype)
