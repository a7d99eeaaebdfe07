"""Loads a model folder (``config.json`` + ``*.safetensors``) by tensor name
into a ``StaticWeightPool`` and binds the parts to it.

andre-fu/prism reads every shard with ``load_file`` into pinned memory
(engine/weight_manager.py:58-81) and copies by name with q/k/v and gate/up
fusion (engine/weight_pool.py:142-199); a missing tensor surfaces there as a
bare ``KeyError`` and extra tensors are ignored.  The names, the fusion order
and the tied-head rule are the same here; validation is explicit and happens
before anything is allocated: one ``WeightError`` lists every missing tensor,
every unexpected tensor and every wrong shape.
"""

from __future__ import annotations

import glob
import json
import os
import struct
from typing import Dict, List, Tuple

import torch

from ..config.model_config import read_config_json
from ..model_registry import build_model
from .pool import StaticWeightPool

_FLOAT_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16}
_INT_DTYPES = {"I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8}
_ST_DTYPES = {**_FLOAT_DTYPES, **_INT_DTYPES}
IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


class WeightError(ValueError):
    """The model file does not hold what the architecture asks for."""

    def __init__(self, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.other = list(wrong_shape), list(other)
        lines = ["model weights do not match the architecture:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        lines += [f"  {o}" for o in self.other]
        super().__init__("\n".join(lines))


def read_safetensors_header(path: str) -> Dict[str, Tuple[tuple, str]]:
    """``name -> (shape, dtype string)`` from the file's JSON header."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    return {k: (tuple(v["shape"]), v["dtype"]) for k, v in header.items() if k != "__metadata__"}


def find_shards(model_dir: str) -> List[str]:
    """Shard list from ``model.safetensors.index.json`` if present, else a
    sorted glob (weight_manager.py:62); none -> FileNotFoundError (:63-64)."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        paths = [os.path.join(model_dir, x) for x in files]
    else:
        paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not paths:
        raise FileNotFoundError(f"No safetensors found in {model_dir}")
    return paths


def resolve_dtype(stored: List[str], compute_dtype: torch.dtype) -> torch.dtype:
    """Precision a parameter is kept in.  float32 engine: float32.  bf16
    engine: bf16/fp16 tensors are kept in bf16, a tensor stored in 32-bit stays
    float32, integer tables become int32."""
    dts = [_ST_DTYPES[s] for s in stored]
    if all(not d.is_floating_point for d in dts):
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    return torch.float32 if any(d == torch.float32 for d in dts) else torch.bfloat16


def validate(named_params, header: Dict[str, Tuple[tuple, str]], allow_extra_head: bool = True):
    """Compare what the parts ask for with what the file has.  Returns the pool
    plan stub ``[(qname, spec, present)]``; raises ``WeightError``."""
    missing, wrong, other, plan = [], [], [], []
    wanted = set()
    for qname, spec in named_params:
        have = [s.name in header for s in spec.sources]
        wanted.update(s.name for s in spec.sources)
        if not any(have) and spec.optional:
            plan.append((qname, spec, False))
            continue
        for s, h in zip(spec.sources, have):
            if not h:
                missing.append(s.name)
            elif tuple(header[s.name][0]) != tuple(s.shape):
                wrong.append((s.name, header[s.name][0], s.shape))
            elif header[s.name][1] not in (_INT_DTYPES if s.init == "table" else _FLOAT_DTYPES):
                other.append(f"unsupported dtype {header[s.name][1]} for {s.name}: " +
                             ("an integer table is stored as " + "/".join(_INT_DTYPES) if s.init == "table"
                              else "weights are stored as " + "/".join(_FLOAT_DTYPES)))
        plan.append((qname, spec, True))
    unexpected = sorted(n for n in header if n not in wanted and not n.endswith(IGNORED_SUFFIXES))
    if missing or unexpected or wrong or other:
        raise WeightError(sorted(missing), unexpected, wrong, other)
    return plan


def load_weights(model, model_dir: str, device, compute_dtype: torch.dtype) -> StaticWeightPool:
    from safetensors import safe_open
    shards = find_shards(model_dir)
    header, where, dup = {}, {}, []
    for p in shards:
        for name, meta in read_safetensors_header(p).items():
            if name in header:
                dup.append(name)
            header[name] = meta
            where[name] = p
    if dup:
        raise WeightError(other=[f"tensor stored in more than one shard: {', '.join(sorted(dup))}"])
    named = list(model.named_params())
    handles = {p: safe_open(p, framework="pt", device="cpu") for p in shards}
    # A parameter tied to another one (the head to the embedding) has no tensor of its own.  If the
    # file stores one all the same (exports often do), it must be the tied tensor over again; a file
    # whose two tensors differ was not made for a tied model, and using either one would be a guess.
    # (andre-fu/prism overwrites the file's tensor with the alias unseen, weight_manager.py:84-86.)
    by_qname = dict(named)
    differs = []
    for qname, spec in named:
        if not (spec.alias_of and spec.optional):
            continue
        target = by_qname[spec.alias_of]
        for s, ts in zip(spec.sources, target.sources):
            if s.name not in header:
                continue
            if ts.name in header and tuple(header[s.name][0]) == tuple(header[ts.name][0]):
                a = handles[where[s.name]].get_tensor(s.name)
                b = handles[where[ts.name]].get_tensor(ts.name)
                if not torch.equal(a.float(), b.float()):
                    differs.append(f"{s.name} is stored although it is tied to {ts.name}, and the two differ")
            elif ts.name in header:
                differs.append(f"{s.name} is stored although it is tied to {ts.name}, with another shape "
                               f"({list(header[s.name][0])} against {list(header[ts.name][0])})")
            del header[s.name]
    if differs:
        raise WeightError(other=differs)
    plan = validate(named, header)
    pool_plan = []
    for qname, spec, present in plan:
        dt = resolve_dtype([header[s.name][1] for s in spec.sources], compute_dtype) if present else None
        pool_plan.append((qname, spec, dt))
    pool = StaticWeightPool(pool_plan, device)
    for qname, spec, dt in pool_plan:
        if dt is None:
            continue
        for i, s in enumerate(spec.sources):
            t = handles[where[s.name]].get_tensor(s.name)
            pool.source_view(qname, i).copy_(t.to(dt), non_blocking=False)
    model.bind(pool.tensors, torch.device(device), compute_dtype)
    return pool


def load_model_folder(model_dir: str, device, dtype: torch.dtype):
    """``(typed config, bound model, pool)`` for a folder; the model class is
    chosen by config.json's ``architectures``."""
    raw = read_config_json(model_dir)
    cfg, model = build_model(raw)
    pool = load_weights(model, model_dir, device, dtype)
    return cfg, model, pool
