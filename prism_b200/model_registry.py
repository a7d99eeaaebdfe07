"""Registry from an architecture's name (``architectures[0]`` of config.json)
to what builds it: a typed-config parser and a function from that config to a
``ModelSpec``.

andre-fu/prism's file of this name is a checkpoint LRU
(engine/model_registry.py:34-68); architectures are recognised there only by a
substring allow-list (engine/server.py:171-173) and a shape tuple
(engine/scheduler.py:25-28).  This registry is the missing map from a name to
code.

An architecture is a module under ``prism_b200/models`` that calls
``register_architecture`` when it is imported; every module of that package
is imported the first time a name is looked up, so adding an architecture
adds a file and edits none.  (Code outside the package may register one at
any time by calling ``register_architecture`` itself.)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

import importlib
import pkgutil

from .config.model_config import ConfigError
from .models.decoder import DecoderModel, ModelSpec


@dataclass
class Architecture:
    name: str
    parse_config: Callable[[dict], object]       # raw config.json dict -> typed config
    build_spec: Callable[[object], ModelSpec]    # typed config -> layer plan


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec) -> None:
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


_builtin_loaded = False


def _load_builtin() -> None:
    """Import every module of ``prism_b200.models`` once (each registers its architecture)."""
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    from . import models
    for m in pkgutil.iter_modules(models.__path__):
        importlib.import_module(f"{models.__name__}.{m.name}")


def registered_architectures():
    _load_builtin()
    return sorted(_ARCHITECTURES)


def resolve(raw_config: dict) -> Architecture:
    """The architecture a raw config.json names."""
    _load_builtin()
    archs = raw_config.get("architectures") or []
    if not archs:
        raise ConfigError(f"config.json has no 'architectures'; registered: {registered_architectures()}")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; registered: {registered_architectures()}")
    return _ARCHITECTURES[name]


def build_model(raw_config: dict):
    """``(typed config, DecoderModel)`` for a raw config.json dict."""
    arch = resolve(raw_config)
    cfg = arch.parse_config(raw_config)
    return cfg, DecoderModel(arch.build_spec(cfg))
