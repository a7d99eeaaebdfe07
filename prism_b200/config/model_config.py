"""What every architecture's configuration shares: the error type and the
reader of ``config.json``.  The typed configuration of an architecture lives
beside its layer plan (``prism_b200/models/<architecture>.py``); nothing in
this package knows an architecture's name or keys.

andre-fu/prism has no typed model configuration: its executor reads an
``AutoConfig`` object with ``getattr`` defaults (engine/executor.py:34-48).
"""

from __future__ import annotations

import json
import os


class ConfigError(ValueError):
    """A ``config.json`` that is missing a key, inconsistent, or asks for an
    option this engine does not compute."""


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path) as f:
        return json.load(f)
