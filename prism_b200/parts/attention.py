"""Attention mixer.  ``gqa_attention``: andre-fu/prism's attention sub-layer
(engine/executor.py:109-122): fused q/k/v projection with bias, position
encoding of q and k, append of k and v to the paged cache, causal
grouped-query attention over the cache with scale ``hd^-1/2``, output
projection.  Head counts, head size, bias, window and the position encoding
are parameters."""

from __future__ import annotations

import warnings
from typing import Optional

import torch

from ..config.model_config import ConfigError
from .base import CacheNeed, Mixer, ParamSpec, PartSpec, WeightSource, build_part, register_part
from .. import ops


_warned = set()
MAX_HEAD_DIM = 256        # the shape-generic attention kernel keeps one head's row in a warp's registers


@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool = True, o_bias: bool = False, window: Optional[int] = None,
                 position: Optional[PartSpec] = None, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ConfigError(f"num_heads {num_heads} not divisible by num_kv_heads {num_kv_heads}")
        if not 2 <= int(head_dim) <= MAX_HEAD_DIM or int(head_dim) % 2:
            raise ConfigError(f"head_dim {head_dim}: the attention kernels take even head sizes from 2 to "
                              f"{MAX_HEAD_DIM}")
        self.hidden_size, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.qkv_bias, self.o_bias = bool(qkv_bias), bool(o_bias)
        self.window = None if window is None else int(window)
        self.scale = float(scale) if scale is not None else self.hd ** -0.5
        self.position = self.add_child("position", build_part("position", position)) if position else None

    @property
    def q_size(self):
        return self.nh * self.hd

    @property
    def kv_size(self):
        return self.nkv * self.hd

    def cache_need(self):
        return CacheNeed("paged", self.nkv, self.hd, self.window)

    def params(self):
        H, qs, kvs = self.hidden_size, self.q_size, self.kv_size
        ps = [ParamSpec("qkv_w", (WeightSource("q_proj.weight", (qs, H)),
                                  WeightSource("k_proj.weight", (kvs, H)),
                                  WeightSource("v_proj.weight", (kvs, H))))]
        if self.qkv_bias:
            ps.append(ParamSpec("qkv_b", (WeightSource("q_proj.bias", (qs,), "bias"),
                                          WeightSource("k_proj.bias", (kvs,), "bias"),
                                          WeightSource("v_proj.bias", (kvs,), "bias"))))
        ps.append(ParamSpec("o_w", (WeightSource("o_proj.weight", (H, qs)),)))
        if self.o_bias:
            ps.append(ParamSpec("o_b", (WeightSource("o_proj.bias", (H,), "bias"),)))
        return ps

    def on_bound(self):
        # Said once, when the model is built, not found out from the step time: in bfloat16 the tensor-core
        # attention kernels take head sizes in steps of 16 up to 128 with up to 16 query heads per kv head; every
        # other shape runs on the shape-generic kernel (one warp per token and head), correct but far slower.
        if self.dtype == torch.bfloat16 and not ops.attention_bf16_shape_ok(self.hd, self.nh, self.nkv):
            key = (self.hd, self.nh, self.nkv)
            if key not in _warned:
                _warned.add(key)
                warnings.warn(f"attention with head_dim {self.hd}, {self.nh} heads, {self.nkv} kv heads runs on the "
                              f"shape-generic kernel in bfloat16 (the tensor-core kernels take head_dim 16, 32, ... 128 "
                              f"and up to 16 query heads per kv head): correct, but much slower", RuntimeWarning,
                              stacklevel=2)

    def forward(self, ctx, x, cache):
        T, qs, kvs = x.shape[0], self.q_size, self.kv_size
        rot = self.position.rotary() if self.position is not None else None
        if rot is None and self.position is not None:
            # a position encoding that is not rotary: project, let it encode q and k, then store
            qkv = ops.linear(x, self.w["qkv_w"], self.w.get("qkv_b"))
            q = qkv[:, :qs].view(T, self.nh, self.hd)
            k = qkv[:, qs:qs + kvs].view(T, self.nkv, self.hd)
            v = qkv[:, qs + kvs:].view(T, self.nkv, self.hd)
            self.position.apply(ctx, q, k)
            ops.rope_kv_write(q, k, v, ctx.positions, ctx.tok_seg, None, 0,
                              cache.k if cache.write else None, cache.v if cache.write else None,
                              cache.block_table, cache.num_pages, ctx.max_positions, ctx.err)
        else:
            attn = ctx.alloc((T, qs), x.dtype)
            ops.qkv_attention(ctx, x, self.w["qkv_w"], self.w.get("qkv_b"), self.nh, self.nkv, self.hd, rot, cache,
                              self.window, self.scale, attn)
            return ops.linear_delta(attn, self.w["o_w"], self.w.get("o_b"))
        attn = ctx.alloc((T, qs), x.dtype)
        ops.attention(ctx, q, attn, cache, self.window, self.scale)
        return ops.linear_delta(attn, self.w["o_w"], self.w.get("o_b"))
