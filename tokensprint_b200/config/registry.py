"""One registry: architecture name -> (typed config, model builder), and model names -> presets.

Two tables live here.

* Architectures.  config.json names its architecture (`architectures[0]`, else
  `model_type`); the entry gives the typed config class and the function that turns a
  config into a `ModelSpec` (the list of layers, their parts and the order they run
  in).  A new architecture is one `register_architecture` call; nothing else in the
  package switches on an architecture's name.

* Model names, in the reference's manner (engine/models/_registry.py:130-263): a short
  name such as `qwen3-8b` belongs to a family (`qwen`), `family/short` is its repo id,
  both spellings resolve, unknown names raise with the list of known ones.  A preset
  is a config.json kept under `config/presets/`; no size stands in code.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

PRESET_DIR = Path(__file__).resolve().parent / "presets"


@dataclass(frozen=True)
class Architecture:
    name: str
    model_types: tuple[str, ...]
    config_from_dict: Callable[[dict[str, Any]], Any]
    build_spec: Callable[[Any], Any]


ARCHITECTURES: dict[str, Architecture] = {}
_MODEL_TYPE_TO_ARCH: dict[str, str] = {}



def register_architecture(
    name: str,
    *,
    model_types: tuple[str, ...] = (),
    config_from_dict: Callable[[dict[str, Any]], Any],
) -> Callable[[Callable[[Any], Any]], Callable[[Any], Any]]:
    """Decorator for the function `config -> ModelSpec` of one architecture."""

    def _register(build_spec: Callable[[Any], Any]) -> Callable[[Any], Any]:
        if name in ARCHITECTURES:
            raise ValueError(f"Architecture {name} already registered.")
        for model_type in model_types:
            if model_type in _MODEL_TYPE_TO_ARCH:
                raise ValueError(f"model_type {model_type} already registered.")
        ARCHITECTURES[name] = Architecture(name, tuple(model_types), config_from_dict, build_spec)
        for model_type in model_types:
            _MODEL_TYPE_TO_ARCH[model_type] = name
        return build_spec

    return _register


def unregister_architecture(name: str) -> None:
    """Removes an entry (tests register toy architectures and take them out again)."""
    arch = ARCHITECTURES.pop(name, None)
    if arch is not None:
        for model_type in arch.model_types:
            _MODEL_TYPE_TO_ARCH.pop(model_type, None)


def _ensure_registered() -> None:
    # Importing the model packages runs their register_* calls.
    import tokensprint_b200.models  # noqa: F401


def architecture_for(config_dict: dict[str, Any]) -> Architecture:
    """The architecture entry that a config.json (as a dict) names."""
    _ensure_registered()
    names = config_dict.get("architectures") or []
    for name in names:
        if name in ARCHITECTURES:
            return ARCHITECTURES[name]
    model_type = config_dict.get("model_type")
    if model_type in _MODEL_TYPE_TO_ARCH:
        return ARCHITECTURES[_MODEL_TYPE_TO_ARCH[model_type]]
    raise ValueError(
        f"Unsupported architecture: architectures={list(names)!r}, model_type={model_type!r}. "
        f"Registered architectures: {sorted(ARCHITECTURES)}"
    )


def load_model_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """Reads `model_dir/config.json`; returns the architecture entry and its typed config."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"No config.json in model folder {model_dir}")
    with open(path, "r", encoding="utf-8") as f:
        config_dict = json.load(f)
    arch = architecture_for(config_dict)
    return arch, arch.config_from_dict(config_dict)


# ---------------------------------------------------------------------------
# model names and presets


@dataclass(frozen=True)
class Preset:
    """A named model: `family/name` is its repo id, `path` its config.json."""

    name: str
    family: str
    path: Path

    @property
    def repo_id(self) -> str:
        return f"{self.family}/{self.name}"


# short name -> preset, in registration order (oldest first)
PRESETS: dict[str, Preset] = {}


def register_preset(family: str, name: str, path: Path) -> None:
    if name in PRESETS:
        raise ValueError(f"Model {name} already registered.")
    PRESETS[name] = Preset(name, family, Path(path))


def _find_preset(spelling: str) -> Preset | None:
    """A preset by its short name or by `family/short`; None if neither is known."""
    _ensure_registered()
    family, _, short = spelling.rpartition("/")
    preset = PRESETS.get(short)
    if preset is None or (family and family != preset.family):
        return None
    return preset


def _preset(spelling: str) -> Preset:
    preset = _find_preset(spelling)
    if preset is None:
        known = ", ".join(sorted(p.repo_id for p in PRESETS.values()))
        raise ValueError(f"Unsupported model_name '{spelling}'. Available models: [{known}]")
    return preset


def _ordered(presets, newest_first: bool) -> list[Preset]:
    presets = list(presets)
    if newest_first:
        presets.reverse()
    return presets


def resolve_model_name(model_name: str) -> str:
    """The short name of either spelling (engine/models/_registry.py:194-215 of the reference)."""
    return _preset(model_name).name


def model_is_registered(model_name: str) -> bool:
    return _find_preset(model_name) is not None


def get_model_family(model: str) -> str:
    return _preset(model).family


def get_model_repo_id(model: str) -> str:
    return _preset(model).repo_id


def all_registered_models(newest_first: bool = True) -> list[str]:
    _ensure_registered()
    return [p.name for p in _ordered(PRESETS.values(), newest_first)]


def get_models_from_family(family: str, newest_first: bool = True) -> list[str]:
    _ensure_registered()
    return [p.name for p in _ordered((p for p in PRESETS.values() if p.family == family), newest_first)]


def all_registered_repo_ids(newest_first: bool = True) -> list[str]:
    _ensure_registered()
    return [p.repo_id for p in _ordered(PRESETS.values(), newest_first)]


def registered_families() -> dict[str, list[Preset]]:
    """family -> its presets, oldest first; families in alphabetical order."""
    _ensure_registered()
    out: dict[str, list[Preset]] = {}
    for preset in sorted(PRESETS.values(), key=lambda p: p.family):
        out.setdefault(preset.family, []).append(preset)
    return out


def get_preset_dict(model_name: str) -> dict[str, Any]:
    """The config.json content of a registered model name."""
    with open(_preset(model_name).path, "r", encoding="utf-8") as f:
        return json.load(f)


def get_model_config(model_name: str) -> Any:
    """Typed config of a registered model name (engine/models/_api.py:22-23)."""
    config_dict = get_preset_dict(model_name)
    return architecture_for(config_dict).config_from_dict(config_dict)


def get_local_model_dir(model_name: str, *, cache_dir: str | Path) -> Path:
    """`cache_dir/<last part of the repo id>` (engine/models/_api.py:26-28)."""
    return Path(cache_dir) / get_model_repo_id(model_name).split("/")[-1]
