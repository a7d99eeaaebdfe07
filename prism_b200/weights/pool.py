"""Static weight pool: every parameter of the model lives in one device
arena, allocated once, at a fixed address (CUDA graphs keep raw pointers).

andre-fu/prism's pool (engine/weight_pool.py:26-85) allocates one tensor per
weight and a second ``[V, H]`` buffer for the head even when it is tied
(:47-48,157-160).  Here the arena is a single allocation with 256-byte
aligned views, a tied head shares the embedding's view, and each parameter
keeps the precision the loader decides for it (bf16 tensors stay bf16, a
tensor the file stores in 32-bit stays float32, integer tables are int32).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import ParamSpec

ALIGN = 256


def _nbytes(shape, dtype: torch.dtype) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n * torch.empty((), dtype=dtype).element_size()


class StaticWeightPool:
    """``plan``: list of ``(qualified name, ParamSpec, dtype or None)``; dtype
    None marks an absent optional parameter (alias, zeros or none per spec)."""

    def __init__(self, plan: List[Tuple[str, ParamSpec, Optional[torch.dtype]]], device):
        self.device = torch.device(device)
        self.specs: Dict[str, ParamSpec] = {q: s for q, s, _ in plan}
        offsets, total = {}, 0
        for q, spec, dt in plan:
            if dt is None and spec.absent != "zeros":
                continue
            dt = dt or torch.float32
            offsets[q] = (total, dt)
            total += (_nbytes(spec.shape, dt) + ALIGN - 1) // ALIGN * ALIGN
        self.total_bytes = total
        self.arena = torch.zeros(max(total, ALIGN), dtype=torch.uint8, device=self.device)
        self.tensors: Dict[str, Optional[torch.Tensor]] = {}
        for q, spec, dt in plan:
            if q in offsets:
                off, d = offsets[q]
                nb = _nbytes(spec.shape, d)
                self.tensors[q] = self.arena[off:off + nb].view(d).view(spec.shape)
        for q, spec, dt in plan:                     # aliases after their targets exist
            if q not in offsets:
                self.tensors[q] = self.tensors.get(spec.alias_of) if spec.alias_of else None

    @property
    def total_gb(self) -> float:
        return self.total_bytes / 1e9

    def __getitem__(self, name: str):
        return self.tensors[name]

    def source_view(self, qname: str, source_index: int) -> torch.Tensor:
        """The rows of a fused parameter that one file tensor fills."""
        spec = self.specs[qname]
        start = sum(s.shape[0] for s in spec.sources[:source_index])
        return self.tensors[qname][start:start + spec.sources[source_index].shape[0]]
