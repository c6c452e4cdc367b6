"""What every architecture's typed configuration shares: the error type and the checked reading
of config.json keys.  The configuration class of an architecture lives beside its model spec
under `tokensprint_b200/models/` (Qwen3: models/qwen3.py) and is registered with it.

The reference keeps a model's constants in registry presets (engine/models/_registry.py:12-40)
and never reads config.json (engine/generation/config.py:27,49-52 is commented out).  Here the
file is the source: every size and constant of a model comes from it, and the presets of the
registry are such files too.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that this engine cannot run; the message names the key."""


def require(d: dict[str, Any], key: str, kind: type) -> Any:
    """d[key] as `kind` (int or float); a missing key or a value of another kind raises ConfigError."""
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    value = d[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
    if kind is float and (isinstance(value, bool) or not isinstance(value, (int, float))):
        raise ConfigError(f"config.json: '{key}' must be a number, got {value!r}")
    return kind(value)


def read_config_json(path: str | Path) -> dict[str, Any]:
    """The content of a config.json, given the file or its folder."""
    path = Path(path)
    if path.is_dir():
        path = path / "config.json"
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def write_config_json(folder: str | Path, content: dict[str, Any]) -> None:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    with open(folder / "config.json", "w", encoding="utf-8") as f:
        json.dump(content, f, indent=2)
