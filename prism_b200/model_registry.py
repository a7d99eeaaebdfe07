"""Registry from an architecture's name (``architectures[0]`` of config.json)
to what builds it: a typed-config parser and a function from that config to a
``ModelSpec``.

andre-fu/prism's file of this name is a checkpoint LRU
(engine/model_registry.py:34-68); architectures are recognised there only by a
substring allow-list (engine/server.py:171-173) and a shape tuple
(engine/scheduler.py:25-28).  This registry is the missing map from a name to
code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from .config.model_config import ConfigError, Qwen2Config
from .models.decoder import DecoderModel, ModelSpec
from .models.qwen2 import qwen2_spec


@dataclass
class Architecture:
    name: str
    parse_config: Callable[[dict], object]       # raw config.json dict -> typed config
    build_spec: Callable[[object], ModelSpec]    # typed config -> layer plan


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec) -> None:
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve(raw_config: dict) -> Architecture:
    """The architecture a raw config.json names."""
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


register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, qwen2_spec)
