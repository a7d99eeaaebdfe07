"""``Engine``: the Python entry point.  A model folder (or a configuration and
a seed) in, generated tokens out, on one GPU.

In andre-fu/prism the same job is split over ``WeightManager.load_model``
(engine/weight_manager.py:45), ``StaticWeightPool`` (engine/weight_pool.py:29),
``FlashAttnKVCache`` (engine/kv_cache.py:15), ``FlashAttnExecutorV3.generate``
(engine/executor.py:411-429) and the scheduler thread
(engine/scheduler.py:377-395).  ``Engine.generate`` keeps ``generate``'s
meaning - prompt token ids in, generated token ids out, greedy unless a
temperature is given - for a list of prompts batched continuously.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from ..config.engine_config import EngineConfig, ModelConfig
from ..cache.manager import pool_sizes
from ..config.model_config import read_config_json
from ..model_registry import build_model
from ..sampling.sampler import Sampler, SamplingParams
from ..weights.loader import load_weights
from ..weights.random_init import random_pool
from .request import GenerationResult
from .runner import ModelRunner, cache_groups
from .scheduler import Scheduler

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class Engine:
    def __init__(self, model: Union[str, ModelConfig, None] = None, engine_config: Optional[EngineConfig] = None,
                 *, dtype: Optional[str] = None, config: Optional[dict] = None, random_seed: Optional[int] = None):
        """``model``: a folder with config.json and model.safetensors (or a
        ``ModelConfig`` naming one).  Random-weights mode instead: ``config``
        (a raw config.json dict) and ``random_seed``; the weights are drawn on
        the device and no file is written."""
        if not torch.cuda.is_available():
            raise RuntimeError("prism_b200 needs a CUDA device; there is no CPU path")
        self.engine_config = ec = engine_config or EngineConfig()
        if isinstance(model, str):
            model = ModelConfig(model_id=model, dtype=dtype or "bfloat16")
        self.model_config = model
        self.dtype_name = dtype or (model.dtype if model else "bfloat16")
        self.dtype = _DTYPES[self.dtype_name]
        self.device = torch.device(f"cuda:{ec.gpu_id}")
        torch.cuda.set_device(self.device)
        if model is not None:
            raw = read_config_json(model.model_id)
            self.config, self.model = build_model(raw)
            self.pool = load_weights(self.model, model.model_id, self.device, self.dtype)
        else:
            if config is None:
                raise ValueError("give a model folder, or config= and random_seed= for random weights")
            self.config, self.model = build_model(config)
            self.pool = random_pool(self.model, random_seed or 0, self.device, self.dtype)
        spec = self.model.spec
        max_seq_len = min(ec.max_seq_len or spec.max_positions, spec.max_positions)
        num_pages = self._pages_per_group(ec, max_seq_len)
        self.runner = ModelRunner(self.model, self.device, self.dtype, ec.kv_page_size, num_pages,
                                  ec.scheduler.max_num_seqs, max_seq_len, ec.use_cuda_graph,
                                  ec.graph_batch_sizes)
        self.sampler = Sampler(self.device)
        self.scheduler = Scheduler(self.runner, self.sampler, ec.scheduler, spec.eos_token_id, ec.seed)

    def _pages_per_group(self, ec: EngineConfig, max_seq_len: int) -> List[int]:
        """Pool size of every cache group: ``ec.num_pages`` if given, else from the byte budget
        ``min(budget, 0.7 * free)`` (engine/scheduler.py:100-103); see ``cache.manager.pool_sizes``."""
        groups, _ = cache_groups(self.model)
        budget = None
        if not ec.num_pages:
            budget = min(ec.kv_cache_budget_gb * 1e9, 0.7 * torch.cuda.mem_get_info(self.device)[0])
        return pool_sizes(groups, ec.kv_page_size, 4 if self.dtype == torch.float32 else 2, max_seq_len,
                          ec.scheduler.max_num_seqs, ec.scheduler.prefill_chunk, ec.num_pages, budget)

    # ---- generation ---------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[GenerationResult]:
        """Generate for every prompt (lists of token ids); requests are batched
        continuously.  Returns results in the order of the prompts."""
        if sampling is None or isinstance(sampling, SamplingParams):
            sampling = [sampling or SamplingParams()] * len(prompts)
        reqs = [self.scheduler.add_request(p, s) for p, s in zip(prompts, sampling)]
        self.scheduler.run_to_completion()
        self.runner.check_errors()
        return [GenerationResult(r.generated_tokens, r.finish_reason, r.ttft, r.tbt, r.num_preemptions, r.error)
                for r in reqs]

    def warmup(self, batch_sizes: Optional[Sequence[int]] = None) -> None:
        """Capture the decode graphs before the first request (engine/executor.py:312-318 does it for a list of
        batch sizes): every bucket's graphs up to ``max_num_seqs``, or those of ``batch_sizes``.  Without it each
        graph is captured at its first use, which that step pays for (tens of milliseconds)."""
        self.runner.warmup_graphs(batch_sizes)

    @property
    def stats(self):
        return self.scheduler.stats

    @property
    def cache(self):
        return self.runner.cache

    def step_fn(self, segments):
        """The step function itself, for replay and verification."""
        return self.runner.step(segments)
