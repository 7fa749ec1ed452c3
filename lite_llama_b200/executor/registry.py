"""Architecture registry: which config parser, weight mapper and model class serve a checkpoint directory.

Plays the role of the reference's model registry (lite_llama/models/registry.py:24-92: ``model_type`` ->
builder/spec); here the key is the ``architecture`` field of ``config.json``.  A design registers with
:func:`register`; ``executor.layered_decoder`` registers the layer-list families when it is imported.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], Any]               # config.json dict -> config object
    map_weights: Callable[..., Any]                   # (config, {name: tensor}, device, dtype) -> weights object
    model_cls: Any                                    # (config, weights, device=..., dtype=...) -> model
    ragged_steps: bool = True                         # serves prompt portions and decode tokens in one flat batch
    sources: tuple[str, ...] | None = None            # CUDA sources its forward launches (``build(sources=...)``)


_REGISTRY: dict[str, Architecture] = {}


def register(arch: Architecture) -> None:
    _REGISTRY[arch.name.lower()] = arch


def lookup(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _REGISTRY[name.lower()]
    except KeyError:
        raise ValueError(f"unknown architecture {name!r}; registered: {sorted(_REGISTRY)}") from None


def names() -> list[str]:
    _ensure_builtin()
    return sorted(a.name for a in _REGISTRY.values())


def architecture_of(model_dir: str | Path) -> tuple[Architecture, dict]:
    """The registry entry a checkpoint directory's ``config.json`` names, and the raw configuration."""
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    name = raw.get("architecture") or (raw.get("architectures") or [None])[0] or raw.get("model_type")
    if not name:
        raise ValueError("config.json names no architecture")
    return lookup(name), raw


def read_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """``config.json`` of a checkpoint directory -> (architecture entry, parsed config)."""
    arch, raw = architecture_of(model_dir)
    cfg = arch.parse_config(raw)
    cfg.validate()
    return arch, cfg


def _ensure_builtin() -> None:
    from . import layered_decoder  # noqa: F401  (registers on import)
