"""Deployment configuration: the names of andre-fu/prism's dataclasses
(engine/config.py:8-40) with the fields a single-model, single-GPU engine
reads.  Fields the reference declares but never reads (``policy``,
``prefetch_queue_threshold``, tier budgets) are dropped; ``max_batch_tokens``
(engine/config.py:39, unread there) is the scheduler's token budget here.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence


@dataclass
class ModelConfig:
    """Where the model comes from (engine/config.py:9-20)."""
    model_id: str                       # a local folder with config.json + model.safetensors
    name: str = ""
    dtype: str = "bfloat16"             # "bfloat16" | "float32"

    def __post_init__(self):
        if not self.name:
            self.name = self.model_id.rstrip("/").split("/")[-1]
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")


@dataclass
class SchedulerConfig:
    """Continuous-batching knobs (engine/config.py:35-40)."""
    max_batch_tokens: int = 4096        # tokens per step, decode tokens first
    max_num_seqs: int = 64              # requests running at once
    prefill_chunk: int = 2048           # most prompt tokens of one request per step
    async_decode: bool = True           # launch the next decode step before reading the last one's tokens


@dataclass
class EngineConfig:
    """Cache and execution knobs (engine/config.py:24-31)."""
    gpu_id: int = 0
    kv_page_size: int = 64              # tokens per page
    num_pages: Optional[int] = None     # explicit pool size of the groups that keep all keys (windowed groups get what
                                        # their window needs, never more than this; cache.manager.pool_sizes), or
    kv_cache_budget_gb: float = 35.0    # ... derived from this budget (engine/scheduler.py:100-103)
    max_seq_len: Optional[int] = None   # block-table width; default max_position_embeddings
    use_cuda_graph: bool = True
    graph_batch_sizes: Sequence[int] = (1, 2, 4, 8, 16, 32, 64)
    seed: int = 0
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
