"""``python -m engine`` is the command line's name in andre-fu/prism
(engine/__main__.py); this package forwards it to ``prism_b200``."""

from prism_b200 import EngineConfig, ModelConfig, SchedulerConfig, SamplingParams  # noqa: F401


def __getattr__(name):
    import prism_b200
    return getattr(prism_b200, name)
