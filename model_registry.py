"""Lists the registered models, family by family, each with its repo id (the output format
of the reference's model_registry.py)."""

from __future__ import annotations

from tokensprint_b200.config.registry import registered_families


def listing() -> str:
    families = registered_families()
    if not families:
        return "No models are currently registered."
    lines = ["Registered models:"]
    for family, presets in families.items():
        lines += ["", f"{family}:"]
        lines += [f"  - {p.name} ({p.repo_id})" for p in presets]
    return "\n".join(lines)


if __name__ == "__main__":
    print(listing())
