"""Random-weights mode: from a configuration and a seed, either write a model
folder (``config.json`` + ``model.safetensors``) or fill a pool on the device.

andre-fu/prism has no such mode (its only fake weights are an unseeded
``torch.randn`` test fixture, tests/test_model_upload.py:28-43).  The recipe:
matrices and embeddings ``normal(0, 0.02)``, biases ``normal(0, 0.02)``, norm
weights ``1 + normal(0, 0.02)``.  For a folder the values come from one CPU
generator in float32, tensor after tensor in the order the model's parts list
them (embedding, layers in order - norm, q, k, v, their biases, o, norm, gate,
up, down - final norm, head unless tied), and are then rounded to the stored
dtype.  For a pool each tensor is drawn on the device from a generator seeded
with ``seed + its index`` in that same order, so large models need no host
memory and no file; a folder written with ``device="cuda"`` draws the same way
and so holds exactly the tensors of the pool with that seed (in bfloat16).
"""

from __future__ import annotations

import json
import os
from typing import Iterator, Tuple

import torch

from ..model_registry import build_model
from .pool import StaticWeightPool

STD = 0.02


def file_tensors(model) -> Iterator[Tuple[str, tuple, str]]:
    """``(tensor name, shape, init kind)`` of every tensor a model file holds."""
    for _, spec in model.named_params():
        if spec.optional and spec.alias_of:
            continue                      # a tied head has no tensor of its own
        for s in spec.sources:
            yield s.name, tuple(s.shape), s.init


def _draw(shape, init: str, gen: torch.Generator, device="cpu") -> torch.Tensor:
    t = torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * STD
    return t + 1.0 if init == "norm" else t


def write_model_folder(raw_config: dict, seed: int, out_dir: str,
                       store_dtype: torch.dtype = torch.bfloat16, device="cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``raw_config``.  ``device``: where the values
    are drawn.  ``"cpu"``: one generator, tensor after tensor.  A CUDA device (for models of billions of
    parameters, where the host's generator takes minutes): every tensor from a generator of its own,
    seeded ``seed + index``, as ``random_pool`` draws them."""
    from safetensors.torch import save_file
    raw = dict(raw_config)           # must name its architecture, as a config.json does
    _, model = build_model(raw)
    if torch.device(device).type == "cpu":
        gen = torch.Generator().manual_seed(int(seed))
        tensors = {name: _draw(shape, init, gen).to(store_dtype).contiguous()
                   for name, shape, init in file_tensors(model)}
    else:
        tensors = {}
        for idx, (name, shape, init) in enumerate(file_tensors(model)):
            gen = torch.Generator(device=device).manual_seed(int(seed) + idx)
            t = torch.empty(shape, dtype=store_dtype, device=device).normal_(0.0, STD, generator=gen)
            tensors[name] = (t.add_(1.0) if init == "norm" else t).cpu()
    os.makedirs(out_dir, exist_ok=True)
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(store_dtype, str(store_dtype))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    return out_dir


def random_pool(model, seed: int, device, compute_dtype: torch.dtype) -> StaticWeightPool:
    """Allocate a pool in ``compute_dtype`` and fill it on the device."""
    named = list(model.named_params())
    plan = [(q, s, None if (s.optional and s.alias_of) else compute_dtype) for q, s in named]
    pool = StaticWeightPool(plan, device)
    idx = 0
    for q, spec, dt in plan:
        if dt is None:
            continue
        for i, s in enumerate(spec.sources):
            gen = torch.Generator(device=device).manual_seed(int(seed) + idx)
            view = pool.source_view(q, i)
            view.normal_(0.0, STD, generator=gen)
            if s.init == "norm":
                view.add_(1.0)
            idx += 1
    model.bind(pool.tensors, torch.device(device), compute_dtype)
    return pool
