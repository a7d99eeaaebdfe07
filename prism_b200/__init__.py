"""prism_b200: a single-GPU inference engine for the Qwen2.5 dense decoder,
written for B200 (sm_100a).  ``Engine`` is the entry point for programs,
``python -m prism_b200`` the command line, ``bin/trace_run`` the replay."""

from .config.engine_config import EngineConfig, ModelConfig, SchedulerConfig  # noqa: F401
from .sampling.sampler import SamplingParams  # noqa: F401


def __getattr__(name):
    if name == "Engine":
        from .engine.llm import Engine
        return Engine
    raise AttributeError(name)
