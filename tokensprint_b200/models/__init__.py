"""Architectures.  Importing this package registers them (config/registry.py)."""

from tokensprint_b200.models import qwen3  # noqa: F401
