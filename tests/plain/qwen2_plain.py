"""Plain, slow, whole-sequence implementation of the Qwen2 dense decoder.

This file is the oracle of the test-suite.  It is written from the formulas
of andre-fu/prism's executor (cited per function as ``file:line`` inside that
project) and shares no code with the ``prism_b200`` package: it reads
``config.json`` with ``json`` and ``model.safetensors`` with the safetensors
library, keeps every tensor in float32 (on the CPU, or on the device the
folder is loaded to: every function works where its tensors are), has no
cache, no paging and no batching.  One function per part.

Where the executor computes in reduced precision (bf16 RoPE tables, bf16
stores) this file computes in float32: it states the mathematics, and the
engine is compared against it with a tolerance that depends on the engine's
dtype.

Two options go beyond what the executor reads and are documented where they
are implemented: ``head_dim`` as an explicit key and the sliding window
(``use_sliding_window`` / ``sliding_window`` / ``max_window_layers``).
"""

from __future__ import annotations

import json
import os

import torch
from safetensors.torch import load_file


# --------------------------------------------------------------------------
# model folder
# --------------------------------------------------------------------------

def load_folder(model_dir: str, device="cpu"):
    """Read ``config.json`` and every tensor of ``model.safetensors`` (as
    float32, onto ``device``).  Tied heads: ``lm_head.weight`` is the embedding
    matrix (engine/weight_manager.py:84-86, engine/weight_pool.py:157-160)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {k: v.to(device=device, dtype=torch.float32) for k, v in
               load_file(os.path.join(model_dir, "model.safetensors")).items()}
    if "lm_head.weight" not in tensors:
        tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"]
    return cfg, tensors


def sizes(cfg: dict):
    """Derived sizes (engine/executor.py:35-43).  The executor fixes
    ``head_dim = hidden_size // num_attention_heads`` (executor.py:37); an
    explicit ``head_dim`` key overrides it here."""
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    return nh, nkv, hd


def layer_window(cfg: dict, layer: int):
    """Sliding window of a layer, or None.  The executor never reads these
    keys (its attention is always full).  Here, as the configuration's own
    keys say: when ``use_sliding_window`` is true, layers with index >=
    ``max_window_layers`` see only the last ``sliding_window`` positions
    (the query's own position included)."""
    if not cfg.get("use_sliding_window", False):
        return None
    w = cfg.get("sliding_window")
    if w is None:
        return None
    if layer >= cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return int(w)
    return None


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embed(tokens: torch.Tensor, embed_w: torch.Tensor) -> torch.Tensor:
    """Row gather, no scaling (engine/executor.py:74-75)."""
    return embed_w[tokens]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w`` (engine/fused_kernels.py:41-49)."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * torch.rsqrt(ms + eps) * w


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """``freqs = pos (x) theta^(-2j/hd)`` (engine/executor.py:48-52), float32."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    return torch.outer(positions.to(torch.float32), inv_freq.to(positions.device))      # [T, hd/2]


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """``cat(-x2, x1)`` (engine/executor.py:18-21)."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    """``cos``, ``sin`` of the angles, each [T, hd/2] float32 (engine/executor.py:53-54
    without the rounding to bf16 that the executor applies there)."""
    ang = rope_angles(positions, head_dim, theta)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x*cos + rotate_half(x)*sin`` with cos/sin repeated over both halves
    (engine/executor.py:55-57,117-118).  x: [T, heads, hd]; cos, sin: [T, hd/2]."""
    cos = torch.cat([cos, cos], dim=-1)[:, None, :]
    sin = torch.cat([sin, sin], dim=-1)[:, None, :]
    return x * cos + rotate_half(x) * sin


def attention(q, k, v, window=None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence: scale
    ``hd^-1/2``, q-head h uses kv-head ``h // (nh/nkv)``, softmax over keys
    ``<=`` the query's position (what ``flash_attn_with_kvcache(causal=True)``
    computes for a whole prompt, engine/executor.py:119-120).  ``window``:
    only keys ``j > pos - window`` are seen.  q: [T, nh, hd]; k, v: [T, nkv, hd]."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.empty_like(q)
    pos = torch.arange(T, device=q.device)
    mask = pos[None, :] <= pos[:, None]
    if window is not None:
        mask &= pos[None, :] > pos[:, None] - window
    for h in range(nh):
        s = (q[:, h, :] @ k[:, h // g, :].T) * (hd ** -0.5)
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, h // g, :]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up``, ``silu(z) = z * sigmoid(z)`` (engine/executor.py:127)."""
    return gate * torch.sigmoid(gate) * up


def decoder_layer(x, t, i, cfg, positions, cos_sin=None, store=None):
    """One pre-norm block (engine/executor.py:106-127): norm, fused qkv with
    bias, rope on q and k, attention, o-projection + residual, norm, gate/up,
    SwiGLU, down-projection + residual.  ``store`` (default: nothing) is applied
    wherever the executor stores an activation in its compute dtype - norm
    output, q/k/v, rotated q and k, attention output, SwiGLU output - so that
    ``store=lambda v: v.bfloat16().float()`` shows what that rounding alone does
    to the result (the residual stream and all arithmetic stay float32)."""
    store = store or (lambda v: v)
    nh, nkv, hd = sizes(cfg)
    eps = cfg.get("rms_norm_eps", 1e-6)
    p = f"model.layers.{i}."
    T = x.shape[0]
    h = store(rms_norm(x, t[p + "input_layernorm.weight"], eps))
    q = h @ t[p + "self_attn.q_proj.weight"].T
    k = h @ t[p + "self_attn.k_proj.weight"].T
    v = h @ t[p + "self_attn.v_proj.weight"].T
    if p + "self_attn.q_proj.bias" in t:                 # engine/weight_pool.py:176-182
        q = q + t[p + "self_attn.q_proj.bias"]
        k = k + t[p + "self_attn.k_proj.bias"]
        v = v + t[p + "self_attn.v_proj.bias"]
    cos, sin = cos_sin if cos_sin is not None else rope_cos_sin(positions, hd, cfg.get("rope_theta", 10000.0))
    q = store(apply_rope(q.view(T, nh, hd), cos, sin))
    k = store(apply_rope(k.view(T, nkv, hd), cos, sin))
    a = store(attention(q, k, store(v).view(T, nkv, hd), layer_window(cfg, i)))
    x = x + a.reshape(T, nh * hd) @ t[p + "self_attn.o_proj.weight"].T
    h = store(rms_norm(x, t[p + "post_attention_layernorm.weight"], eps))
    gate = h @ t[p + "mlp.gate_proj.weight"].T
    up = h @ t[p + "mlp.up_proj.weight"].T
    x = x + store(swiglu(gate, up)) @ t[p + "mlp.down_proj.weight"].T
    return x


def forward(cfg: dict, t: dict, tokens, cos_sin=None, store=None) -> torch.Tensor:
    """Logits at every position of one whole sequence, float32 [T, V]
    (engine/executor.py:99-130, with the head applied to all rows).
    ``cos_sin``: rotary tables to use instead of the float32 ones.
    ``store``: see ``decoder_layer``."""
    dev = t["model.embed_tokens.weight"].device
    tokens = torch.as_tensor(tokens, dtype=torch.long, device=dev)
    positions = torch.arange(tokens.shape[0], device=dev)
    x = embed(tokens, t["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, t, i, cfg, positions, cos_sin, store)
    h = rms_norm(x, t["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    return (store(h) if store else h) @ t["lm_head.weight"].T


# --------------------------------------------------------------------------
# sampling and generation
# --------------------------------------------------------------------------

_M64 = (1 << 64) - 1


def uniform(seed: int, request_index: int, step_index: int) -> float:
    """Counter-based uniform in [0, 1): three rounds of the splitmix64
    finaliser over (seed, request, step), top 24 bits.  The executor draws
    from torch's global generator (engine/executor.py:426-427), which cannot
    be replayed; this is the seeded stand-in both sides use."""
    z = (seed * 0x9E3779B97F4A7C15 + request_index * 0xBF58476D1CE4E5B9
         + step_index * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & _M64
    for _ in range(3):
        z = (z + 0x9E3779B97F4A7C15) & _M64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def sample(logits: torch.Tensor, temperature: float, u: float) -> int:
    """Greedy when ``temperature <= 0`` (engine/executor.py:423-424; lowest
    index on ties), else ``softmax(logits / T)`` (executor.py:426) and the
    first index whose inclusive cumulative probability exceeds ``u``."""
    if temperature <= 0:
        return int(torch.argmax(logits))
    p = torch.softmax(logits.to(torch.float32) / temperature, dim=-1)
    c = torch.cumsum(p.to(torch.float64), dim=-1)
    idx = int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=torch.float64), right=True))
    return min(idx, p.shape[0] - 1)


def generate(cfg, t, prompt, max_new_tokens, temperature=0.0, seed=0, request_index=0,
             eos_token_id=None):
    """Generation loop of engine/executor.py:411-429 on whole sequences (every
    step recomputes the full forward): sample, stop at eos or at the count."""
    seq = list(prompt)
    out = []
    for step in range(max_new_tokens):
        logits = forward(cfg, t, seq)[-1]
        tok = sample(logits, temperature, uniform(seed, request_index, step))
        out.append(tok)
        seq.append(tok)
        if eos_token_id is not None and tok == eos_token_id:
            break
    return out
