"""One registry from an architecture's name to its configuration class and its model recipe.

The reference picks its model by a substring test on ``config.model_type``
(rollout/engine_actor.py:24-32) and raises ``ValueError`` for anything else.  Here the key is
``architectures[0]`` of config.json, with ``model_type`` as a fallback.  An architecture gives:
``config_cls`` (typed, ``from_dict``), ``decoder_spec(cfg, max_positions)`` -> DecoderSpec,
``weight_sources(cfg)`` -> {parameter: Source}, ``ignorable_tensors(cfg)`` (names, or name -> twin
it must equal).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    config_cls: type
    decoder_spec: Callable
    weight_sources: Callable
    ignorable_tensors: Callable = lambda cfg: set()
    # rows of each checkpoint tensor inside a fused parameter, or None for an even split
    split_rows: Callable = lambda cfg, param: None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architectures():
    return sorted(_ARCHITECTURES)


def resolve(raw_config: dict) -> Architecture:
    """The architecture a config.json (as a dict) asks for."""
    names = raw_config.get("architectures") or []
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = str(raw_config.get("model_type", "")).lower()
    if not names:
        for arch in _ARCHITECTURES.values():
            if arch.model_type == mt:
                return arch
    raise ValueError(f"no model for architectures={names!r} model_type={mt!r}; known: {architectures()}")


def read_config(model_dir: str):
    """(architecture, typed configuration) of a model folder."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{model_dir} has no config.json")
    with open(path) as f:
        raw = json.load(f)
    arch = resolve(raw)
    return arch, arch.config_cls.from_dict(raw)


def _register_builtin() -> None:
    from ..models import qwen3
    from .model_config import Qwen3Config
    register_architecture(Architecture(
        name="Qwen3ForCausalLM", model_type="qwen3", config_cls=Qwen3Config,
        decoder_spec=qwen3.decoder_spec, weight_sources=qwen3.weight_sources,
        ignorable_tensors=qwen3.ignorable_tensors, split_rows=qwen3.split_rows))


_register_builtin()
