"""Python face of the hand-written CUDA kernels (``prism_b200/csrc``).

Every function takes CUDA tensors, checks what the kernel assumes (dtype,
contiguity, sizes), and launches on torch's current stream.  There is no CPU
path, and nothing steps in for a missing kernel: if the shared library cannot
be built or loaded, or a tensor is not on a CUDA device, the call raises.
(The one library call is by design, not a fallback: the bf16 matrix product
of more than a few tokens, see ``linear``.)

Which of andre-fu/prism's call sites each op replaces:

==================  ==========================================================
``embed``           ``F.embedding`` (engine/executor.py:74-75)
``add_rmsnorm``     residual add + ``fused_rms_norm`` (executor.py:108,122-124,130)
``linear``          ``F.linear`` (executor.py:109,122,125,127,130)
``rope_kv_write``   eager RoPE (executor.py:117-118) + the cache append inside
                    ``flash_attn_with_kvcache`` (executor.py:119-120)
``attention``       ``flash_attn_with_kvcache`` (executor.py:119-120)
``swiglu``          ``F.silu(gate) * up`` (executor.py:127)
``sample``          argmax / softmax + multinomial (engine/scheduler.py:266-272)
==================  ==========================================================
"""

from __future__ import annotations

import ctypes
import math
import os
import threading
from typing import Optional

import numpy as np
import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_lib = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    """A kernel refused its arguments or a launch failed."""


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def lib():
    """The loaded shared library; built at the first call if it is missing or stale."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.build(verbose=True)
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the prism_b200 CUDA kernels from {path}: {e}") from e
        for name in dir(_Sig):
            if name.startswith("prism_"):
                fn = getattr(_lib, name)
                fn.restype = ctypes.c_int
                fn.argtypes = getattr(_Sig, name)
        _lib.prism_set_pdl(0 if os.environ.get("PRISM_PDL", "1") == "0" else 1)
    return _lib


def library_file() -> Optional[str]:
    return _build.library_path()


_p, _i, _f, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


class _Sig:
    prism_embed = [_p, _p, _i, _p, _i, _i, _i, _p, _p]
    prism_add_rmsnorm = [_p, _p, _i, _i, _ll, _p, _i, _f, _p, _i, _p, _i, _i, _p]
    prism_rope_table = [_p, _p, _i, _i, _p, _p]
    prism_rope_kv_write_partial = [_p, _i, _p, _i, _p, _i, _i, _p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i,
                                   _i, _p, _p]
    prism_rope_kv_write = [_p, _p, _p, _i, _i, _p, _p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i,
                           _i, _i, _p, _p]
    prism_attention_generic = [_p, _i, _p, _i, _p, _p, _i, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i,
                               _i, _f, _p, _p]
    prism_attention_bf16_supported = [_i, _i, _i]
    prism_attention_decode_bf16 = [_p, _i, _p, _i, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f,
                                   _p, _p, _i, _p, _p, _i, _p, _p]
    prism_attention_decode_qkv_bf16 = [_p, _i, _p, _i, _p, _i, _p, _i, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i,
                                       _i, _f, _p, _p, _i, _p, _p, _i, _p, _p]
    prism_attention_prefill_bf16 = [_p, _i, _p, _i, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i,
                                    _f, _p, _p]
    prism_attention_prefill_tc_supported = [_i, _i, _i, _i]
    prism_attention_prefill_tc = [_p, _i, _i, _p, _i, _p, _p, _i, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i,
                                  _f, _p, _i, _p, _p, _p]
    prism_attention_merge_bf16 = [_p, _p, _i, _p, _i, _i, _i, _i, _p]
    prism_swiglu = [_p, _p, _i, _i, _i, _p]
    prism_sgemm_nt = [_p, _i, _p, _i, _p, _i, _p, _i, _i, _i, _i, _p]
    prism_sample = [_p, _i, _i, _i, _p, _p, _p, _p]
    prism_argmax_split = [_p, _i, _i, _i, _i, _p, _p, _p, _p, _p]
    prism_set_pdl = [_i]
    prism_gemm_tcgen05_supported = [_i, _i, _i]
    prism_gemm_tcgen05 = [_p, _i, _p, _i, _p, _i, _p, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p]
    prism_gemv_bf16_supported = [_i, _i, _i]
    prism_gemv_bf16 = [_p, _i, _p, _i, _p, _i, _p, _i, _i, _i, _i, _i, _p]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("prism_b200 kernels run on CUDA tensors only; there is no CPU path")


launch_count = 0      # kernels of this library launched (or captured) by this process


def _check(code: int, what: str):
    global launch_count
    launch_count += 1
    if code != 0:
        if code == 1:       # cudaErrorInvalidValue: the launcher refused the sizes
            raise KernelError(f"{what}: sizes not supported by this kernel")
        raise KernelError(f"{what}: CUDA error {code}")


# --------------------------------------------------------------------------

def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor):
    """``out[t] = table[ids[t]]`` as float32.  ids int32 [T]; table [V, H]."""
    _cuda(ids, table, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32
    assert table.is_contiguous() and out.is_contiguous()
    T, (V, H) = ids.shape[0], table.shape
    assert out.shape == (T, H)
    _check(lib().prism_embed(_ptr(ids), _ptr(table), _dt(table), _ptr(out), T, H, V, _ptr(err),
                             _stream()), "embed")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None):
    """``residual += delta`` in place (float32; ``delta`` None, ``[T, H]`` or a
    stack ``[k, T, H]`` of partial sums), then ``out = rmsnorm(residual) * weight``
    for every row, or for the rows listed in ``rows`` (int32)."""
    _cuda(residual, delta, weight, out, rows)
    assert residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous()
    T, H = residual.shape
    nsplit, stride = 0, 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-2:] == (T, H)
        nsplit = 1 if delta.dim() == 2 else delta.shape[0]
        stride = T * H
    n = T if rows is None else rows.shape[0]
    assert out.shape == (n, H) and weight.shape == (H,)
    _check(lib().prism_add_rmsnorm(_ptr(residual), _ptr(delta), F32 if delta is None else _dt(delta),
                                   nsplit, stride, _ptr(weight), _dt(weight), float(eps), _ptr(out),
                                   _dt(out), _ptr(rows), n, H, _stream()), "add_rmsnorm")


def sgemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor):
    """True float32 ``out = x @ w.T + bias`` on CUDA cores."""
    _cuda(x, w, bias, out)
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32
    assert x.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    _check(lib().prism_sgemm_nt(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias),
                                F32 if bias is None else _dt(bias), _ptr(out), out.stride(0), M, N, K,
                                _stream()), "sgemm")


USE_GEMV = os.environ.get("PRISM_GEMV", "1") != "0"
GEMV_MAX_M = int(os.environ.get("PRISM_GEMV_MAX_M", "16"))      # above 16 tokens it streams at half the bandwidth
EPI_BF16, EPI_F32, EPI_SWIGLU = 0, 1, 2


def gemv_supported(M: int, N: int, K: int) -> bool:
    return USE_GEMV and bool(lib().prism_gemv_bf16_supported(M, N, K))


def gemv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, epi: int = EPI_BF16):
    """Weight-streaming product for a few tokens: ``out = x @ w.T (+ bias)`` in
    bf16 (``EPI_BF16``) or float32 (``EPI_F32``); or, with ``w`` the fused
    ``[2I, K]`` gate/up weight, ``out[M, I] = silu(x @ gate.T) * (x @ up.T)``
    (``EPI_SWIGLU``)."""
    _cuda(x, w, bias, out)
    M, K = x.shape
    N = out.shape[1]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == M
    assert w.shape[0] == (2 * N if epi == EPI_SWIGLU else N)
    assert out.dtype == (torch.float32 if epi == EPI_F32 else torch.bfloat16)
    _check(lib().prism_gemv_bf16(_ptr(w), w.stride(0), _ptr(x), x.stride(0) if M > 1 else K, _ptr(bias),
                                 F32 if bias is None else _dt(bias), _ptr(out), out.stride(0) if M > 1 else N,
                                 M, N, K, epi, _stream()), "gemv_bf16")


EPI_PARTIAL = 3
_tc_err = {}


def _tc_err_word(device) -> torch.Tensor:
    """Device error word for the tensor-core GEMM's bounded waits (one per device)."""
    key = torch.device(device).index or 0
    if key not in _tc_err:
        _tc_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_err[key]


_tc_ws = {}
_tc_ws_retired = []       # outgrown workspaces: never freed, a captured graph may still hold their addresses


def _tc_workspace(device, floats: int, tiles: int):
    """Split-K workspace of the tensor-core GEMM: partial sums and one counter per
    tile.  Grown outside graph capture only; kernels leave the counters at zero.
    A workspace that a later call outgrows is kept alive for the life of the process:
    decode graphs captured earlier replay with its addresses, and memory given back to
    the allocator could by then hold somebody's activations."""
    key = torch.device(device).index or 0
    ws = _tc_ws.get(key)
    if ws is None or ws[0].numel() < floats or ws[1].numel() < tiles:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the split-K workspace must be sized before graph capture (run one step eagerly first)")
        if ws is not None:
            _tc_ws_retired.append(ws)
        ws = (torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device),
              torch.zeros(max(tiles, 4096), dtype=torch.int32, device=device))
        _tc_ws[key] = ws
    return ws


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
            epi: int = EPI_BF16, ksplit: int = 1, err: Optional[torch.Tensor] = None):
    """tcgen05 + TMA weight-streaming product for up to 64 tokens.  ``epi``:
    ``EPI_BF16`` / ``EPI_F32`` (``out [M, N]``, + bias), ``EPI_SWIGLU`` (``w`` is
    the fused ``[2N, K]`` gate/up weight), ``EPI_PARTIAL`` (``out`` float32
    ``[ksplit, M, N]`` partial sums over K for the next kernel to add)."""
    _cuda(x, w, bias, out)
    M, K = x.shape
    N = out.shape[-1]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.is_contiguous()
    assert w.shape[0] == (2 * N if epi == EPI_SWIGLU else N)
    if epi == EPI_PARTIAL:
        assert out.dtype == torch.float32 and out.shape == (ksplit, M, N) and bias is None
    else:
        assert out.shape == (M, N) and (ksplit == 1 or epi != EPI_SWIGLU)
        assert out.dtype == (torch.float32 if epi == EPI_F32 else torch.bfloat16)
    err = err if err is not None else _tc_err_word(x.device)
    ws = cnt = None
    if ksplit > 1 and epi != EPI_PARTIAL:
        ws, cnt = _tc_workspace(x.device, ksplit * M * N, (N + 127) // 128)
    _check(lib().prism_gemm_tcgen05(_ptr(w), w.stride(0), _ptr(x), x.stride(0) if M > 1 else K, _ptr(bias),
                                    F32 if bias is None else _dt(bias), _ptr(out), N, M, N, K, epi, ksplit,
                                    _ptr(ws), _ptr(cnt), _ptr(err), _stream()), "gemm_tcgen05")


USE_TC_GEMM = os.environ.get("PRISM_TC_GEMM", "1") != "0"
TC_GEMM_MAX_M = int(os.environ.get("PRISM_TC_GEMM_MAX_M", "16"))


# products with a long K (the down projection) stay on the tcgen05 kernel up to more tokens
# the fused gate/up + SwiGLU product stays on it up to 64 tokens: 14B layer sizes at batch 32, 8 layers + head:
# 1.66 ms against 1.67 ms with the library product + SwiGLU kernel (and 2.00 ms with the mma.sync small-M GEMM)
TC_GEMM_MAX_M_SWIGLU = int(os.environ.get("PRISM_TC_GEMM_MAX_M_SWIGLU", "64"))
TC_KSPLIT_FORCED = int(os.environ.get("PRISM_TC_KSPLIT", "0"))       # experiments: a fixed K-split
TC_GEMM_LONG_K = int(os.environ.get("PRISM_TC_GEMM_LONG_K", "8192"))
TC_GEMM_MAX_M_LONG_K = int(os.environ.get("PRISM_TC_GEMM_MAX_M_LONG_K", "64"))    # batch 64 decode step: 4.79 -> 4.66 ms


def tc_gemm_ok(x: torch.Tensor, w: torch.Tensor, max_m: Optional[int] = None) -> bool:
    """Whether the tcgen05 weight-streaming product takes this call (``max_m``: a caller's own
    limit on the tokens, instead of the general one)."""
    M, K = x.shape
    limit = TC_GEMM_MAX_M if max_m is None else max_m
    if K >= TC_GEMM_LONG_K:
        limit = max(limit, TC_GEMM_MAX_M_LONG_K)
    return (USE_TC_GEMM and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= limit
            and x.stride(1) == 1 and w.stride(1) == 1 and (M == 1 or x.stride(0) % 8 == 0) and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(lib().prism_gemm_tcgen05_supported(M, w.shape[0], K)))


def tc_ksplit(N: int, K: int, sms: Optional[int] = None, M: Optional[int] = None) -> int:
    """CTAs that share one 128-row tile's K range: about one CTA per SM in all (``sms``: the device's
    count), at least 8 blocks of 64 k each.  With up to 16 tokens (``M``) two of the kernel's CTAs fit on an
    SM, so the count is rounded to the nearest instead of down (14B qkv projection, 56 tiles: 3 splits = 168
    CTAs instead of 2 = 112: 6.003 -> 5.880 ms a step at batch 8), and a product with a long K (the down
    projection) is shared half as finely again, 32 blocks each at least: the CTAs that double up have twice
    the weights on their way before the dependency wait (7B down projection, 5 -> 7 splits: 3.008 -> 2.992 ms
    a step at batch 8, 2.831 -> 2.804 at batch 1, 3.218 -> 3.181 at batch 16; 14B and 32B steps 1.9 % shorter).
    With 32 tokens and more one CTA fills an SM's shared memory: never more CTAs than SMs."""
    tiles = (N + 127) // 128
    if TC_KSPLIT_FORCED:
        return TC_KSPLIT_FORCED
    n_sms = sms or num_sms()
    kblocks = (K + 63) // 64
    few = M is not None and M <= 16
    ks = max(1, min((2 * n_sms + tiles) // (2 * tiles) if few else n_sms // tiles, kblocks // 8))
    if few and kblocks // ks >= 48:
        ks = max(ks, min((3 * n_sms // 2) // tiles, kblocks // 32))
    return ks


def check_tc_errors():
    """Raise if a bounded wait of the tensor-core GEMM ran out (synchronises)."""
    for word in _tc_err.values():
        code = int(word.item())
        if code:
            word.zero_()
            raise KernelError(f"tensor-core GEMM: device error {code} (a bounded wait ran out)")


def linear_delta(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A projection whose result will be added to the residual stream by the
    next norm: like ``linear``, but it may return a float32 stack ``[k, M, N]``
    of partial sums over K, which the fused add + norm kernel adds up."""
    if bias is None and tc_gemm_ok(x, w):
        N, K = w.shape
        ks = tc_ksplit(N, K, M=x.shape[0])
        if ks > 1:
            out = torch.empty((ks, x.shape[0], N), dtype=torch.float32, device=x.device)
            gemm_tc(x, w, None, out, EPI_PARTIAL, ksplit=ks)
            return out
    return linear(x, w, bias)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x @ w.T + bias`` with ``w`` in the ``[out, in]`` layout of the model
    file.  float32 activations, or a float32 weight under bf16 activations
    (a tensor the model file stores in 32-bit), go through the true-float32
    kernel; bf16 x bf16 goes to the library matrix product (cuBLAS through
    torch), as in andre-fu/prism (executor.py:109)."""
    _cuda(x, w, bias)
    M, N = x.shape[0], w.shape[0]
    want = out_dtype or (out.dtype if out is not None else x.dtype)
    if x.dtype == torch.float32 or w.dtype == torch.float32:
        x32 = x if x.dtype == torch.float32 else x.float()
        w32 = w if w.dtype == torch.float32 else w.float()
        o32 = out if (out is not None and out.dtype == torch.float32) else \
            torch.empty((M, N), dtype=torch.float32, device=x.device)
        sgemm(x32, w32, bias, o32)
        if want == torch.float32:
            return o32
        if out is not None:
            out.copy_(o32)
            return out
        return o32.to(want)
    if want in (torch.float32, torch.bfloat16) and tc_gemm_ok(x, w) and (out is None or out.is_contiguous()):
        if out is None or out.dtype != want:
            out = torch.empty((M, N), dtype=want, device=x.device)
        gemm_tc(x, w, bias, out, EPI_F32 if want == torch.float32 else EPI_BF16, ksplit=tc_ksplit(N, x.shape[1]))
        return out
    # bf16 x bf16, library product with float32 accumulation
    if want == torch.float32:
        res = torch.mm(x, w.t(), out_dtype=torch.float32)
        if bias is not None:
            res += bias.float()
        if out is not None:
            out.copy_(res)
            return out
        return res
    b = bias if (bias is None or bias.dtype == torch.bfloat16) else bias.to(torch.bfloat16)
    if out is None:
        return torch.nn.functional.linear(x, w, b)
    if b is None:
        return torch.mm(x, w.t(), out=out)
    return torch.addmm(b, x, w.t(), out=out)


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor):
    """``out[t, j] = (cos, sin)(positions[t] * inv_freq[j])`` in float32, shared
    by every layer and head of a step."""
    _cuda(positions, inv_freq, out)
    T, half = positions.shape[0], inv_freq.shape[0]
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, half, 2)
    _check(lib().prism_rope_table(_ptr(positions), _ptr(inv_freq), half, T, _ptr(out), _stream()), "rope_table")


def rope_kv_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor,
                  tok_seg: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  block_table: Optional[torch.Tensor], num_pages: int, max_pos: int,
                  err: torch.Tensor, table: Optional[torch.Tensor] = None):
    """Rotate ``q [T, nh, hd]`` and ``k [T, nkv, hd]`` in place (views of one
    row-strided buffer) and store k, v at their positions in the paged cache
    ``[pages, P, nkv, hd]``.  ``k_cache`` None: rotate only.  ``table``: the
    step's cos/sin table from ``rope_table`` (lets the vector kernel run)."""
    _cuda(q, k, v, positions, tok_seg, inv_freq, k_cache, v_cache, block_table)
    T, nh, hd = q.shape
    nkv = k.shape[1]
    rs = q.stride(0)
    assert T == 1 or (k.stride(0) == rs and v.stride(0) == rs), "q, k, v must be views of one buffer"
    assert q.stride(2) == 1 and q.stride(1) == hd and k.stride(1) == hd and v.stride(1) == hd
    assert positions.dtype == torch.int32 and tok_seg.dtype == torch.int32
    P = W = 0
    if k_cache is not None:
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == q.dtype
        assert k_cache.shape[2:] == (nkv, hd) and block_table.dtype == torch.int32
        P, W = k_cache.shape[1], block_table.shape[1]
    if inv_freq is not None:
        assert inv_freq.dtype == torch.float32 and inv_freq.shape[0] * 2 == rotary_dim
    if T == 1:
        rs = 0                  # a single row: its stride is never used
    if table is not None:
        assert table.dtype == torch.float32 and table.shape == (T, rotary_dim // 2, 2)
    _check(lib().prism_rope_kv_write(_ptr(q), _ptr(k), _ptr(v), _dt(q), rs, _ptr(positions),
                                     _ptr(tok_seg), _ptr(inv_freq), _ptr(table), rotary_dim, _ptr(k_cache),
                                     _ptr(v_cache), _ptr(block_table), W, P, num_pages, T, nh, nkv,
                                     hd, max_pos, _ptr(err), _stream()), "rope_kv_write")


def rope_kv_write_partial(parts: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                          positions: torch.Tensor, tok_seg: torch.Tensor, table: torch.Tensor, rotary_dim: int,
                          k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                          block_table: Optional[torch.Tensor], num_pages: int, max_pos: int, nkv: int,
                          err: torch.Tensor):
    """``rope_kv_write`` for a qkv projection that arrives as float32 partial
    sums ``parts [k, T, (nh + 2 nkv) * hd]`` (+ ``bias``): the sum, the bias, the
    rotation and the cache store in one kernel; rotated q goes to ``q_out [T, nh, hd]``."""
    _cuda(parts, bias, q_out, positions, tok_seg, table, k_cache, v_cache, block_table)
    ks, T, D = parts.shape
    _, nh, hd = q_out.shape
    assert parts.dtype == torch.float32 and parts.is_contiguous() and D == (nh + 2 * nkv) * hd
    assert q_out.is_contiguous() and table.dtype == torch.float32 and table.shape == (T, rotary_dim // 2, 2)
    P = W = 0
    if k_cache is not None:
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == q_out.dtype
        assert k_cache.shape[2:] == (nkv, hd)
        P, W = k_cache.shape[1], block_table.shape[1]
    _check(lib().prism_rope_kv_write_partial(_ptr(parts), ks, _ptr(bias), F32 if bias is None else _dt(bias),
                                             _ptr(q_out), nh * hd, _dt(q_out), _ptr(positions), _ptr(tok_seg),
                                             _ptr(table), rotary_dim, _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
                                             W, P, num_pages, T, nh, nkv, hd, max_pos, _ptr(err), _stream()),
           "rope_kv_write_partial")


# The qkv projection of a few tokens: K-split tcgen05 GEMM -> float32 partial sums -> one kernel that adds them and
# the bias, rotates and stores (several CTAs per token).  PRISM_QKV_LIBRARY=1 (with PRISM_QKV_PARTIAL=0): the
# library product and the rotary kernel, for comparison.
QKV_LIBRARY = os.environ.get("PRISM_QKV_LIBRARY", "0") == "1"


def qkv_rotate_store(ctx, x: torch.Tensor, qkv_w: torch.Tensor, qkv_b: Optional[torch.Tensor], nh: int, nkv: int,
                     hd: int, rot, cache) -> torch.Tensor:
    """The front half of an attention layer: qkv projection (+ bias), rotary
    encoding of q and k (``rot``: RotaryParams or None), store of k, v into the
    cache plane.  Returns q ``[T, nh, hd]``.  For a few tokens the projection runs
    K-split on the tensor-core GEMM and its partial sums are added, biased,
    rotated and stored by one kernel."""
    T = x.shape[0]
    qs, kvs = nh * hd, nkv * hd
    table = None
    if rot is not None and rot.rotary_dim:
        key = ("rotary_table", rot.inv_freq.data_ptr())          # one table per step for all layers
        table = ctx.scratch.get(key)
        if table is None:
            table = ctx.scratch[key] = ctx.alloc((T, rot.rotary_dim // 2, 2), torch.float32)
            rope_table(ctx.positions, rot.inv_freq, table)
    kc, vc = (cache.k, cache.v) if cache.write else (None, None)
    rd = rot.rotary_dim if rot is not None else 0
    if QKV_PARTIAL and table is not None and tc_gemm_ok(x, qkv_w) and hd % 8 == 0 and rot.rotary_dim % 16 == 0:
        ks = tc_ksplit(qkv_w.shape[0], qkv_w.shape[1], M=T)
        if ks > 1:
            parts = ctx.alloc((ks, T, qs + 2 * kvs), torch.float32)
            gemm_tc(x, qkv_w, None, parts, EPI_PARTIAL, ksplit=ks)
            q = ctx.alloc((T, nh, hd), x.dtype)
            rope_kv_write_partial(parts, qkv_b, q, ctx.positions, ctx.tok_seg, table, rot.rotary_dim, kc, vc,
                                  cache.block_table, cache.num_pages, ctx.max_positions, nkv, ctx.err)
            return q
    if QKV_LIBRARY and x.dtype == torch.bfloat16:
        b = qkv_b if (qkv_b is None or qkv_b.dtype == torch.bfloat16) else qkv_b.to(torch.bfloat16)
        qkv = torch.nn.functional.linear(x, qkv_w, b)
    else:
        qkv = linear(x, qkv_w, qkv_b)
    q = qkv[:, :qs].view(T, nh, hd)
    k = qkv[:, qs:qs + kvs].view(T, nkv, hd)
    v = qkv[:, qs + kvs:].view(T, nkv, hd)
    rope_kv_write(q, k, v, ctx.positions, ctx.tok_seg, rot.inv_freq if rot else None, rot.rotary_dim if rot else 0,
                  kc, vc, cache.block_table, cache.num_pages, ctx.max_positions, ctx.err, table=table)
    return q


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, block_table: torch.Tensor, positions: torch.Tensor,
                      tok_seg: torch.Tensor, num_pages: int, window: Optional[int], scale: float,
                      err: torch.Tensor):
    """Shape-generic paged causal GQA attention; ``q [T, nh, hd]`` row-strided,
    ``out [T, nh*hd]``."""
    _cuda(q, out, k_cache, v_cache, block_table, positions, tok_seg)
    T, nh, hd = q.shape
    nkv, P = k_cache.shape[2], k_cache.shape[1]
    assert q.stride(2) == 1 and q.stride(1) == hd and out.stride(1) == 1
    assert k_cache.dtype == q.dtype and out.dtype == q.dtype
    if hd > 256:
        raise KernelError(f"attention: head_dim {hd} > 256 is not supported")
    _check(lib().prism_attention_generic(_ptr(q), q.stride(0), _ptr(out), out.stride(0),
                                         _ptr(k_cache), _ptr(v_cache), _dt(q), _ptr(block_table),
                                         block_table.shape[1], _ptr(positions), _ptr(tok_seg), T, nh,
                                         nkv, hd, P, num_pages, int(window or 0), float(scale),
                                         _ptr(err), _stream()), "attention_generic")


def swiglu(gu: torch.Tensor, out: torch.Tensor):
    """``out = silu(gu[:, :I]) * gu[:, I:]``."""
    _cuda(gu, out)
    T, I2 = gu.shape
    assert gu.is_contiguous() and out.is_contiguous() and out.shape == (T, I2 // 2) and out.dtype == gu.dtype
    _check(lib().prism_swiglu(_ptr(gu), _ptr(out), _dt(gu), T, I2 // 2, _stream()), "swiglu")


_argmax_ws = {}


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], u: Optional[torch.Tensor],
           out: torch.Tensor):
    """Per row: argmax if its temperature <= 0, else inverse-CDF sampling of
    ``softmax(logits / temperature)`` at the uniform number ``u``."""
    _cuda(logits, temperature, u, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    R, V = logits.shape
    if temperature is None and V >= 8192 and R <= 4096 and not torch.cuda.is_current_stream_capturing():
        # greedy over a large vocabulary: many blocks per row
        key = torch.device(logits.device).index or 0
        ws = _argmax_ws.get(key)
        nb = 32
        if ws is None or ws[0].numel() < R * nb:
            n = max(R * nb, 4096 * nb)
            ws = _argmax_ws[key] = (torch.empty(n, dtype=torch.float32, device=logits.device),
                                    torch.empty(n, dtype=torch.int32, device=logits.device),
                                    torch.zeros(4096, dtype=torch.int32, device=logits.device))
        _check(lib().prism_argmax_split(_ptr(logits), logits.stride(0), R, V, nb, _ptr(ws[0]), _ptr(ws[1]),
                                        _ptr(ws[2]), _ptr(out), _stream()), "argmax_split")
        return
    _check(lib().prism_sample(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(u),
                              _ptr(out), _stream()), "sample")


# --------------------------------------------------------------------------
# composites: the places where a faster kernel is chosen for a shape
# --------------------------------------------------------------------------

_num_sms = {}


def num_sms(device=None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current CUDA device), asked of the driver
    once per device.  The grid shapes below (K-splits, attention splits) are sized by it."""
    if not torch.cuda.is_available():
        raise KernelError("the number of SMs is a property of a CUDA device; pass sms= to size a grid without one")
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    n = _num_sms.get(idx)
    if n is None:
        n = _num_sms[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return n


FORCE_GENERIC_ATTENTION = os.environ.get("PRISM_ATTENTION", "") == "generic"


QKV_PARTIAL = os.environ.get("PRISM_QKV_PARTIAL", "1") != "0"


def _check_decode_scratch(items, starts, T, nh, hd, nsplit, part_o, part_ml):
    slots = T * nsplit                                   # partial results: one per (token, split) ...
    if items is not None:                                # ... or one per work item
        assert starts is not None and items.dtype == torch.int32 and starts.dtype == torch.int32
        assert items.dim() == 2 and items.shape[1] == 4 and items.is_contiguous() and items.data_ptr() % 16 == 0
        assert starts.numel() == T and starts.is_contiguous() and items.shape[0] <= 65535
        slots = items.shape[0]
    if nsplit > 1:
        assert part_o.dtype == torch.float32 and part_o.numel() >= slots * nh * hd
        assert part_ml.dtype == torch.float32 and part_ml.numel() >= slots * nh * 2


def attention_decode_bf16(q, out, k_cache, v_cache, block_table, positions, tok_seg, num_pages, window,
                          scale, nsplit, part_o, part_ml, err, items: Optional[torch.Tensor] = None,
                          starts: Optional[torch.Tensor] = None):
    """Tensor-core decode attention (one token per request) with the keys split
    over ``nsplit`` CTAs per (token, kv head); ``part_o [T, nh, nsplit, hd]`` and
    ``part_ml [T, nh, nsplit, 2]`` are float32 scratch for the partial results.
    With ``items`` (device int32 ``[n, 4]``) and ``starts`` (``[T]``), the step's work items
    (``decode_work_items``), every token's keys are shared among the CTAs chosen for it; ``nsplit``
    is then the most items of a token and the scratch ``[n, nh, hd]`` and ``[n, nh, 2]``."""
    _cuda(q, out, k_cache, v_cache, block_table, positions, tok_seg, part_o, part_ml, items, starts)
    T, nh, hd = q.shape
    nkv, P = k_cache.shape[2], k_cache.shape[1]
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(2) == 1 and q.stride(1) == hd and out.stride(1) == 1
    _check_decode_scratch(items, starts, T, nh, hd, nsplit, part_o, part_ml)
    _check(lib().prism_attention_decode_bf16(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache),
                                             _ptr(v_cache), _ptr(block_table), block_table.shape[1],
                                             _ptr(positions), _ptr(tok_seg), T, nh, nkv, hd, P, num_pages,
                                             int(window or 0), float(scale), _ptr(part_o), _ptr(part_ml),
                                             int(nsplit), _ptr(items), _ptr(starts), 0 if items is None else items.shape[0],
                                             _ptr(err), _stream()), "attention_decode_bf16")
    if nsplit > 1:
        global launch_count
        launch_count += 1          # the merge kernel


def attention_decode_qkv_bf16(parts, bias, table, max_pos, out, k_cache, v_cache, block_table, positions, tok_seg,
                              num_pages, nh, window, scale, nsplit, part_o, part_ml, err,
                              items: Optional[torch.Tensor] = None, starts: Optional[torch.Tensor] = None):
    """Decode attention that finishes the qkv projection itself: ``parts [ks, T, (nh + 2 nkv) * hd]`` are the
    projection's float32 partial sums, ``bias`` its bias or None, ``table [T, hd / 2, 2]`` the step's cos/sin.
    Every CTA adds, biases and rotates the query rows it needs; the CTA that holds a token's own position
    does the same for the token's key and value, stores them in the cache and uses them.  The whole head is
    rotated (rotary_dim == hd)."""
    _cuda(parts, bias, table, out, k_cache, v_cache, block_table, positions, tok_seg, part_o, part_ml)
    ks, T, D = parts.shape
    nkv, P, hd = k_cache.shape[2], k_cache.shape[1], k_cache.shape[3]
    assert parts.dtype == torch.float32 and parts.is_contiguous() and D == (nh + 2 * nkv) * hd
    assert table.dtype == torch.float32 and table.is_contiguous() and table.shape == (T, hd // 2, 2)
    assert k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.shape == (T, nh * hd)
    _cuda(items, starts)
    _check_decode_scratch(items, starts, T, nh, hd, nsplit, part_o, part_ml)
    _check(lib().prism_attention_decode_qkv_bf16(_ptr(parts), ks, _ptr(bias), F32 if bias is None else _dt(bias),
                                                 _ptr(table), int(max_pos), _ptr(out), out.stride(0), _ptr(k_cache),
                                                 _ptr(v_cache), _ptr(block_table), block_table.shape[1],
                                                 _ptr(positions), _ptr(tok_seg), T, nh, nkv, hd, P, num_pages,
                                                 int(window or 0), float(scale), _ptr(part_o), _ptr(part_ml),
                                                 int(nsplit), _ptr(items), _ptr(starts),
                                                 0 if items is None else items.shape[0], _ptr(err), _stream()),
           "attention_decode_qkv_bf16")
    if nsplit > 1:
        global launch_count
        launch_count += 1          # the merge kernel


def attention_prefill_bf16(q, out, k_cache, v_cache, block_table, seg_start, cached_len, max_q_len,
                           num_pages, window, scale, err):
    """Tensor-core attention for segments of any length (portions of prompts,
    and single tokens among them)."""
    _cuda(q, out, k_cache, v_cache, block_table, seg_start, cached_len)
    T, nh, hd = q.shape
    nkv, P = k_cache.shape[2], k_cache.shape[1]
    S = cached_len.shape[0]
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(2) == 1 and q.stride(1) == hd and out.stride(1) == 1 and seg_start.shape[0] == S + 1
    _check(lib().prism_attention_prefill_bf16(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache),
                                              _ptr(v_cache), _ptr(block_table), block_table.shape[1],
                                              _ptr(seg_start), _ptr(cached_len), S, int(max_q_len), nh, nkv, hd,
                                              P, num_pages, int(window or 0), float(scale), _ptr(err),
                                              _stream()), "attention_prefill_bf16")


PREFILL_SPLIT_MIN_TILES = 16      # key tiles (of 64) a split CTA should keep
PREFILL_SPLIT_FROM_TILES = 64     # fewer key tiles than this are not split: the merge costs as much as it saves ...
PREFILL_SPLIT_FROM_TILES_FEW_CTAS = 32    # ... unless the query tiles fill under a quarter of the GPU


def prefill_splits(S: int, max_q_len: int, nh: int, max_kv_len: int, window: Optional[int],
                   sms: Optional[int] = None) -> int:
    """CTAs that share the key tiles of one (head, 128 query rows) in the tcgen05 prefill kernel: 1 unless
    the query tiles alone leave most of the GPU idle and the keys are many (a short portion against a
    long cache); then as many as fill the two CTAs per SM, each with at least PREFILL_SPLIT_MIN_TILES.
    (Measured at the 7B head counts, 128 new tokens: 2,048 cached 42 -> 34 us in 2 splits, 8,192 cached
    127 -> 46 us in 8, 32,768 cached 471 -> 86 us in 10; 512 new tokens after 2,048: 48 us whole, 55 us in 2.)"""
    if os.environ.get("PRISM_PREFILL_SPLITS"):
        return int(os.environ["PRISM_PREFILL_SPLITS"])
    NUM_SMS = sms or num_sms()
    ctas = S * nh * ((max_q_len + 127) // 128)
    span = min(max_kv_len, window + max_q_len) if window else max_kv_len
    tiles = (span + 63) // 64
    if tiles < (PREFILL_SPLIT_FROM_TILES_FEW_CTAS if 4 * ctas <= 2 * NUM_SMS else PREFILL_SPLIT_FROM_TILES):
        return 1
    return max(1, min((2 * NUM_SMS) // max(1, ctas), tiles // PREFILL_SPLIT_MIN_TILES, 16))


def attention_merge(part_o: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor):
    """``out[t, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)`` over the splits' partial results
    ``part_o [T, nh, nsplit, hd]`` / ``part_ml [T, nh, nsplit, 2]`` (float32); ``out`` bf16 ``[T, nh * hd]``."""
    _cuda(part_o, part_ml, out)
    T, nh, ns, hd = part_o.shape
    assert part_o.is_contiguous() and part_ml.is_contiguous() and part_ml.shape == (T, nh, ns, 2)
    assert part_o.dtype == torch.float32 and part_ml.dtype == torch.float32 and out.dtype == torch.bfloat16
    assert out.stride(1) == 1 and out.shape == (T, nh * hd)
    _check(lib().prism_attention_merge_bf16(_ptr(part_o), _ptr(part_ml), ns, _ptr(out), out.stride(0), T, nh, hd,
                                            _stream()), "attention_merge")


def attention_prefill_tc(q, out, k_cache, v_cache, block_table, seg_start, cached_len, max_q_len,
                         num_pages, window, scale, err, nsplit: int = 1, first_token: int = 0):
    """The same on the 5th-generation tensor cores (tcgen05, TMA, tensor memory): 128 query
    rows per CTA.  Head size 64 or 128, pages of a multiple of 64 tokens.  ``nsplit`` > 1: that many
    CTAs share a query tile's keys and a second kernel merges their partial results (of the tokens
    from ``first_token`` on: the segments given must cover exactly those)."""
    _cuda(q, out, k_cache, v_cache, block_table, seg_start, cached_len)
    T, nh, hd = q.shape
    nkv, P = k_cache.shape[2], k_cache.shape[1]
    S = cached_len.shape[0]
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(2) == 1 and q.stride(1) == hd and out.stride(1) == 1 and seg_start.shape[0] == S + 1
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
    po = pml = None
    if nsplit > 1:
        po = torch.empty((T, nh, nsplit, hd), dtype=torch.float32, device=q.device)
        pml = torch.empty((T, nh, nsplit, 2), dtype=torch.float32, device=q.device)
    _check(lib().prism_attention_prefill_tc(_ptr(q), q.stride(0), T, _ptr(out), out.stride(0), _ptr(k_cache),
                                            _ptr(v_cache), k_cache.shape[0], _ptr(block_table), block_table.shape[1],
                                            _ptr(seg_start), _ptr(cached_len), S, int(max_q_len), nh, nkv, hd,
                                            P, num_pages, int(window or 0), float(scale), _ptr(err), int(nsplit),
                                            _ptr(po), _ptr(pml), _stream()), "attention_prefill_tc")
    if nsplit > 1:
        attention_merge(po[first_token:], pml[first_token:], out[first_token:])


def attention_prefill_tc_supported(hd: int, nh: int, nkv: int, page_size: int) -> bool:
    return bool(lib().prism_attention_prefill_tc_supported(hd, nh, nkv, page_size))


ATTENTION_TC = os.environ.get("PRISM_ATTN_TC", "1") != "0"
ATTENTION_TC_MIN_Q = int(os.environ.get("PRISM_ATTN_TC_MIN_Q", "64"))     # shorter portions: 64-row mma.sync tiles


LONG_CONTEXT = int(os.environ.get("PRISM_LONG_CONTEXT", "4096"))      # keys from which a lone CTA per query tile is too slow


def prefill_on_tc(max_q_len: int, max_kv_len: int, window: Optional[int]) -> bool:
    """Portions of 64 tokens and more go to the tcgen05 kernel (128-row query tiles), shorter ones to the
    mma.sync kernel (64-row tiles, cheaper to start) - unless the cache is long: the tcgen05 kernel can share
    a query tile's keys among CTAs, the mma.sync kernel walks them with one CTA per head (128 tokens behind
    32,768: 86 us against 729 us), and a prompt's last portion can be a few tokens behind all the others."""
    span = min(max_kv_len, window + max_q_len) if window else max_kv_len
    return max_q_len >= ATTENTION_TC_MIN_Q or span >= LONG_CONTEXT


def decoders_apart(n_leading_single: int, their_max_kv_len: int, window: Optional[int]) -> bool:
    """In a mixed step: whether the decoding requests at the head of the batch go to the decode kernel.  Worth
    a launch of its own from ``MIXED_SPLIT_MIN`` of them on - or from one, if their contexts are long: as
    one-token segments of the prefill kernel each would be a single CTA per head walking all its keys."""
    if n_leading_single <= 0:
        return False
    span = min(their_max_kv_len, window + 64) if window else their_max_kv_len
    return n_leading_single >= MIXED_SPLIT_MIN or span >= LONG_CONTEXT


def attention_bf16_shape_ok(hd: int, nh: int, nkv: int) -> bool:
    """The rule of ``prism_attention_bf16_supported`` (csrc/attention_bf16.cu), for callers that have no
    library loaded (a model built on a host without a GPU)."""
    return 16 <= hd <= 128 and hd % 16 == 0 and nkv > 0 and nh % nkv == 0 and nh // nkv <= 16


def attention_bf16_supported(hd: int, nh: int, nkv: int) -> bool:
    return bool(lib().prism_attention_bf16_supported(hd, nh, nkv))


def decode_tiles(position: int, window: Optional[int]) -> int:
    """64-key tiles the token at ``position`` sees (its own key included)."""
    lo = max(0, position - window + 1) if window else 0
    return position // 64 - lo // 64 + 1


def decode_used_splits(tiles: int, target_x16: int, cap: int) -> int:
    """CTAs that share one request's keys under a target of ``target_x16 / 16`` tiles per CTA: as many as keep
    each at or below the target, none with fewer than ``DECODE_MIN_TILES`` tiles, at most ``cap``."""
    target = max(target_x16, DECODE_MIN_TILES * 16)
    return min(max(min(-(-tiles * 16 // target), tiles // DECODE_MIN_TILES), 1), cap)


# Where one wave leaves a quarter of the CTAs or more at less than half the longest CTA's length (many requests too
# short to be split hold a place each and leave it early), the plan goes to CTAs of about half the size in two
# waves: the second wave moves into the places the short CTAs have left.  Equal contexts never qualify (all CTAs are
# the longest), and there two waves lose: batch 48 at 2,100 keys 4.19 -> 4.28 ms a step, batch 56 4.40 -> 4.64 ms.
DECODE_SHORT_CTA = 0.5
DECODE_SECOND_WAVE_FROM_SHARE = 0.25


def _tiles_of(positions, window: Optional[int]):
    pos = np.asarray(positions, dtype=np.int64)
    lo = np.maximum(pos - window + 1, 0) if window else 0
    return pos // 64 - lo // 64 + 1


def _used_splits(tiles, target_x16: int, cap: int = 64):
    """``decode_used_splits`` for an array of requests."""
    target = max(target_x16, DECODE_MIN_TILES * 16)
    used = np.minimum((tiles * 16 + (target - 1)) // target, np.minimum(tiles // DECODE_MIN_TILES, cap))
    return np.maximum(used, 1, out=used)


def _smallest_target(tiles, nkv: int, places: int) -> int:
    """The smallest target (tiles per CTA, in sixteenths), from the tiles divided by the places on, with which
    the requests' CTAs fit into ``places``.  It is seldom much more than that: the search widens from there."""
    tiles16, most = tiles * 16, np.minimum(tiles // DECODE_MIN_TILES, 64)

    def fits(target):
        used = np.minimum((tiles16 + (target - 1)) // target, most)
        return (int(used.sum()) + int(np.count_nonzero(used == 0))) * nkv <= places
    lo = max(DECODE_MIN_TILES * 16, -(-int(tiles.sum()) * nkv * 16 // places))
    if fits(lo):
        return lo
    top = max(lo, int(tiles.max()) * 16)                      # one CTA each: fits, or nothing does
    step = max(1, lo // 8)
    hi = min(top, lo + step)
    while hi < top and not fits(hi):
        lo, step = hi, step * 2
        hi = min(top, lo + step)
    lo += 1                                                   # lo does not fit, hi does
    while lo < hi:
        mid = (lo + hi) // 2
        if fits(mid):
            hi = mid
        else:
            lo = mid + 1
    return lo


# Splitting has to pay: where even the best plan leaves the longest CTA above this fraction of the longest request
# (many requests of about the same length and only a few places to spare), every request keeps a single CTA and
# the step needs no merge kernel (64 requests of 1,024 to 1,536 keys on 8 kv heads: ten of them could be halved,
# the eleventh decides the kernel's time all the same).
DECODE_SPLIT_GAIN = 0.75


def decode_split_target(positions, nkv: int, window: Optional[int], sms: Optional[int] = None,
                        n_real: Optional[int] = None) -> int:
    """The decode kernel's plan for a step: 64-key tiles per CTA, in sixteenths - the smallest target with which
    the CTAs of the step's decoding requests (``decode_used_splits`` for each, times the kv heads) still fit on
    the GPU at once, two per SM.  A long context among short ones is then shared among many CTAs while the short
    ones take one each, and no CTA runs much longer than the rest.  For equal contexts this is the rule measured
    before: 11 CTAs per (token, kv head) at batch 1 and 2,100 keys, 9 at batch 8, 4 at batch 16, 1 from batch 48
    on.  Where many short requests hold most of the places, so that many CTAs are far shorter than the
    longest (``DECODE_SECOND_WAVE_FROM_SHARE``), the target is the one that fits into twice the places: the short
    CTAs end early and the second wave takes their places (64 requests of 128 to 4,096 keys, 4 kv heads: 5.31 ->
    4.93 ms a step; 32 requests, 8 kv heads: 9.28 -> 8.74 ms; 8 requests, whose CTAs are all about as long:
    3.03 -> 3.16 ms, which is why it is no general rule).  A batch so large that one CTA per (token, kv head) is
    more than fits at once: the same, from the waves that this takes.  ``n_real``: the requests after the first
    ``n_real`` are padding (rows of a captured graph's bucket): they take a place each, but say nothing about
    how unequal the step's CTAs are."""
    slots = 2 * (sms or num_sms())
    tiles = _tiles_of(positions, window)
    real = slice(0, len(tiles) if n_real is None else n_real)
    places = slots * max(1, -(-len(tiles) * nkv // slots))       # the waves that one CTA each needs in any case
    target = _smallest_target(tiles, nkv, places)
    used = _used_splits(tiles, target)
    per = tiles[real] / used[real]
    if used[real][per < DECODE_SHORT_CTA * per.max()].sum() >= DECODE_SECOND_WAVE_FROM_SHARE * used[real].sum():
        target = _smallest_target(tiles, nkv, places + slots)
        used = _used_splits(tiles, target)
    if (tiles / used).max() > DECODE_SPLIT_GAIN * tiles.max():
        target = int(tiles.max()) * 16                           # one CTA each
    return target


def decode_plan_for(positions, nkv: int, window: Optional[int], sms: Optional[int] = None,
                    n_real: Optional[int] = None):
    """``(target_x16, cap)`` for a step's decoding requests: the plan and the most CTAs any request gets under
    it.  Many requests (a third of a wave of CTAs or more) with long contexts of about one length
    (``DECODE_LONG_FROM_TILES``) get equal splits chosen by how they fill whole waves, see below; the older
    rule for one CTA each at 16,384 keys and more (``DECODE_BALANCE_FROM_TILES``) remains for what that leaves."""
    n_sms = sms or num_sms()
    target = decode_split_target(positions, nkv, window, n_sms, n_real)
    tiles = _tiles_of(positions, window)
    cap = int(_used_splits(tiles, target).max())
    real = tiles if n_real is None else tiles[:n_real]
    least, most = int(real.min()), int(real.max())
    slots = 2 * n_sms
    if least >= DECODE_LONG_FROM_TILES and 4 * least >= 3 * most and 3 * len(tiles) * nkv >= slots:
        # many requests with long contexts of about one length: all get the same number of CTAs - one that
        # fills its last wave to 85 % or more, and among those the one that makes about two waves (measured at
        # 8,192 and 16,384 keys on 4 kv heads: 32 requests best in 4 CTAs each, 40 in 5, 48 in 4 or 3, 64 in 2
        # or 3; up to 11 % of the kernel's time against one wave's worth)
        def waves(k):
            return len(tiles) * nkv * k / slots
        ks = [k for k in range(1, 9) if k == 1 or least // k >= 16]
        full = [k for k in ks if waves(k) / -(-waves(k) // 1) >= 0.85]
        k = min(full, key=lambda k: abs(waves(k) - 2.0)) if full else max(ks, key=lambda k: waves(k) / -(-waves(k) // 1))
        target = -(-most * 16 // k)
        cap = int(_used_splits(tiles, target).max())
    elif cap == 1 and least >= DECODE_BALANCE_FROM_TILES:
        def fill(k):
            m = len(tiles) * nkv * k / n_sms
            return m / -(-m // 1)
        for k in range(2, 9):
            if least // k < 16:
                break
            if fill(k) >= 0.95 > fill(1):
                target = max(DECODE_MIN_TILES * 16, -(-least * 16 // k))
                cap = int(_used_splits(tiles, target).max())
                break
    return target, cap


def decode_work_items(positions, nkv: int, window: Optional[int], sms: Optional[int] = None,
                      n_real: Optional[int] = None, memo: Optional[dict] = None):
    """The decode attention kernel's work for a step: ``(items [n, 4], starts [B], most)`` as int32 arrays
    and the most items any request has.  Request b (at ``positions[b]``, token and segment b of the step) gets
    ``decode_plan_for``'s number of CTAs per kv head, less where fewer already leave each the same number of
    tiles: ``used`` items ``{b, split | used << 16, position, b}`` from item ``first`` on, ``starts[b] = first |
    used << 16``.  The requests whose CTAs are longest come first, so that when the items are more than fit on
    the GPU at once the short ones run last.  ``n_real``: the requests after these are a graph bucket's padding.
    ``memo``: a dict the caller keeps between steps; the items depend on the positions only through the
    requests' tile counts, which change once in 64 steps, so the step before has usually left all but the
    position column."""
    pos = np.asarray(positions, dtype=np.int64)
    tiles = _tiles_of(pos, window)
    key = None
    if memo is not None:
        key = (tiles.tobytes(), n_real, nkv, window, sms)
        if memo.get("key") == key:
            items, tok, starts, most = memo["value"]
            items = items.copy()
            items[:, 2] = pos[tok]
            return items, starts, most
    target, cap = decode_plan_for(positions, nkv, window, sms, n_real)
    used = _used_splits(tiles, target, cap)
    per = -(-tiles // used)
    used = -(-tiles // per)                                # no CTA without a tile
    order = np.argsort(-per, kind="stable")
    first = np.empty(len(pos), dtype=np.int64)
    first[order] = np.cumsum(used[order]) - used[order]
    tok = np.repeat(order, used[order])
    split = np.arange(len(tok)) - first[tok]
    items = np.stack([tok, split | (used[tok] << 16), pos[tok], tok], axis=1).astype(np.int32)
    starts, most = (first | (used << 16)).astype(np.int32), int(used.max())
    if memo is not None:
        memo["key"], memo["value"] = key, (items, tok, starts, most)
    return items, starts, most


DECODE_LONG_FROM_TILES = 128         # 8,192 keys
DECODE_MIN_TILES = 3                # 64-key tiles a split CTA keeps at least (csrc/attention_bf16.cuh: DEC_MIN_TILES)
DECODE_BALANCE_FROM_TILES = 256     # 16,384 keys: below, the merge costs what the balance gains (batch 64: 8,192 keys
                                    # 203 -> 201 us in 4 splits, 32,768 keys 717 -> 673 us)


def decode_splits(T: int, nkv: int, max_kv_len: int, window: Optional[int], balance: bool = True,
                  sms: Optional[int] = None) -> int:
    """How many CTAs share one (token, kv head)'s keys: as many as fill one wave
    of two CTAs per SM, at most one per ``DECODE_MIN_TILES`` 64-key tiles.  More, shorter CTAs lose:
    each pays the same fixed latencies (position, block table, first bytes, merge), and the merge grows
    with them (batch 1 at 2,100 keys: 33 splits of one tile 2.90 ms a step, 12 splits 2.81, 8 splits 2.87).
    ``max_kv_len`` is the longest context of the batch, or, when a graph is captured, the longest the
    graph may ever see - the kernel itself keeps ``DECODE_MIN_TILES`` tiles per CTA for the context it
    finds and leaves the splits it does not need empty.  ``balance`` (the few splits of a large batch
    against long contexts) is for the former only: a bound of 32,768 says nothing about the contexts a
    replay will meet."""
    if os.environ.get("PRISM_DECODE_SPLITS", "0") != "0":
        return int(os.environ["PRISM_DECODE_SPLITS"])
    NUM_SMS = sms or num_sms()
    span = min(max_kv_len, window + 64) if window else max_kv_len
    tiles = max(1, (span + 63) // 64)
    fill = (2 * NUM_SMS) // max(1, T * nkv)
    n = max(1, min(-(-tiles // DECODE_MIN_TILES), 64, fill))
    if balance and n == 1 and tiles >= DECODE_BALANCE_FROM_TILES:
        # A large batch against long contexts: one CTA per (token, kv head) fills the GPU, but unevenly (256
        # CTAs are two on 108 SMs and one on 40, and the kernel lasts as long as the pairs).  A few splits
        # make the CTAs small enough to spread evenly: the fewest (each keeping 16 tiles or more) that
        # load every SM to within 5 % of the busiest.
        def balance(k):
            m = T * nkv * k / NUM_SMS
            return m / -(-m // 1)
        for k in range(1, 9):
            if k > 1 and tiles // k < 16:
                break
            if balance(k) >= 0.95:
                return k
    return n


# A mixed step hands its leading single-token segments to the decode kernel when there are at least
# this many (measured on 7B shapes, 512-token portion beside them: 8 decoders 1.72 vs 1.65 ms per
# 4 layers with / without the split, 64 decoders 2.09 vs 2.90 ms).
MIXED_SPLIT_MIN = int(os.environ.get("PRISM_MIXED_SPLIT_MIN", "12"))


def _leading_single_token_segments(ctx) -> int:
    """How many segments at the start of the batch bring exactly one token (the scheduler
    puts the decoding requests first).  Known on the host only; 0 inside a captured graph."""
    if ctx.host is None:
        return 0
    n = ctx.scratch.get("lead_single")
    if n is None:
        n = 0
        for q in ctx.host["q_len"]:
            if q != 1:
                break
            n += 1
        ctx.scratch["lead_single"] = n
    return n


def _attention_portions(ctx, q, out, cache, window, scale, first_seg: int):
    """Segments ``first_seg ..`` of the batch with the prefill kernels."""
    T, nh, hd = q.shape
    nkv = cache.k.shape[2]
    seg_start, cached_len, bt = ctx.seg_start[first_seg:], ctx.cached_len[first_seg:], cache.block_table[first_seg:]
    if (ATTENTION_TC and prefill_on_tc(ctx.max_q_len, ctx.max_kv_len, window) and scale > 0 and cache.k.is_contiguous()
            and cache.v.is_contiguous() and attention_prefill_tc_supported(hd, nh, nkv, cache.k.shape[1])):
        ns = prefill_splits(cached_len.shape[0], ctx.max_q_len, nh, ctx.max_kv_len, window)
        attention_prefill_tc(q, out, cache.k, cache.v, bt, seg_start, cached_len, ctx.max_q_len, cache.num_pages,
                             window, scale, ctx.err, nsplit=ns, first_token=first_seg)
    else:
        attention_prefill_bf16(q, out, cache.k, cache.v, bt, seg_start, cached_len, ctx.max_q_len, cache.num_pages,
                               window, scale, ctx.err)


def _decode_scratch(ctx, cache, nd: int, nh: int, nkv: int, hd: int, window: Optional[int]):
    """``(nsplit, part_o, part_ml, items, starts)`` for the decode kernel.  A step whose descriptor carries work
    items for this cache group (the runner makes them from the requests' real contexts) runs on them; otherwise
    the splits are equal for all requests and chosen from the longest context."""
    work = getattr(ctx, "decode_work", {}).get(getattr(cache, "group", None))
    if work is not None and work[3] == nd:
        items, starts, most = work[0], work[1][:nd], work[2]
        n = items.shape[0]
        return most, ctx.alloc((n, nh, hd), torch.float32), ctx.alloc((n, nh, 2), torch.float32), items, starts
    nsplit = decode_splits(nd, nkv, ctx.max_kv_len, window, balance=ctx.host is not None)
    return nsplit, ctx.alloc((nd, nh, nsplit, hd), torch.float32), ctx.alloc((nd, nh, nsplit, 2), torch.float32), None, None


def attention(ctx, q: torch.Tensor, out: torch.Tensor, cache, window: Optional[int], scale: float):
    """Attention of the step's tokens over one cache plane.  ``cache`` is a
    ``PagedCacheView``; the kernel is chosen by dtype and shape, and the
    shape-generic kernel takes whatever the faster ones refuse.  In a mixed
    step the decoding requests at the head of the batch go to the decode kernel
    (one CTA set per kv head, GQA-packed) and only the prompt portions to the
    prefill kernel, whose query tiles a single token would leave almost empty."""
    T, nh, hd = q.shape
    nkv = cache.k.shape[2]
    if q.dtype == torch.bfloat16 and not FORCE_GENERIC_ATTENTION and attention_bf16_supported(hd, nh, nkv):
        nd = T if ctx.decode_only else _leading_single_token_segments(ctx)
        if not ctx.decode_only:
            longest = max(ctx.host["cached_len"][:nd]) + 1 if nd else 0      # keys of the longest decoding request
            if not decoders_apart(nd, longest, window):
                nd = 0
        if nd > 0:
            nsplit, part_o, part_ml, items, starts = _decode_scratch(ctx, cache, nd, nh, nkv, hd, window)
            attention_decode_bf16(q[:nd], out[:nd], cache.k, cache.v, cache.block_table, ctx.positions[:nd],
                                  ctx.tok_seg[:nd], cache.num_pages, window, scale, nsplit, part_o, part_ml, ctx.err,
                                  items=items, starts=starts)
        if nd < ctx.S:
            _attention_portions(ctx, q, out, cache, window, scale, nd)
        return
    attention_generic(q, out, cache.k, cache.v, cache.block_table, ctx.positions, ctx.tok_seg,
                      cache.num_pages, window, scale, ctx.err)


# PRISM_QKV_IN_ATTENTION=1: in a pure decode step the qkv projection's partial sums go straight to the decode
# attention kernel, which adds, biases, rotates and stores (no kernel between the projection and attention).
# Off by default: one launch fewer, the same step time (3.08 ms both ways at batch 8).  The attention CTAs then
# become resident beside the projection's CTAs, of which only one fits per SM next to them, so half of them start
# after the projection has ended and ask for their keys only then; with the small rotary kernel in between all of
# them are resident and have their first tiles on the way before they are released.
QKV_IN_ATTENTION = os.environ.get("PRISM_QKV_IN_ATTENTION", "0") == "1"


def qkv_attention(ctx, x: torch.Tensor, qkv_w: torch.Tensor, qkv_b: Optional[torch.Tensor], nh: int, nkv: int, hd: int,
                  rot, cache, window: Optional[int], scale: float, out: torch.Tensor):
    """An attention layer between its input and its output projection: qkv projection (+ bias), rotary
    encoding of q and k, store of k and v, attention over the cache plane into ``out [T, nh * hd]``.
    ``qkv_rotate_store`` followed by ``attention``; with ``QKV_IN_ATTENTION`` a pure decode step of a few
    tokens runs as two kernels (K-split projection, attention that finishes the projection)."""
    T = x.shape[0]
    if (QKV_IN_ATTENTION and QKV_PARTIAL and ctx.decode_only and cache.write and rot is not None
            and rot.rotary_dim == hd and x.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
            and not FORCE_GENERIC_ATTENTION and tc_gemm_ok(x, qkv_w)
            and cache.k.is_contiguous() and cache.v.is_contiguous() and attention_bf16_supported(hd, nh, nkv)):
        ks = tc_ksplit(qkv_w.shape[0], qkv_w.shape[1], M=T)
        if ks > 1:
            key = ("rotary_table", rot.inv_freq.data_ptr())          # one table per step for all layers
            table = ctx.scratch.get(key)
            if table is None:
                table = ctx.scratch[key] = ctx.alloc((T, hd // 2, 2), torch.float32)
                rope_table(ctx.positions, rot.inv_freq, table)
            parts = ctx.alloc((ks, T, (nh + 2 * nkv) * hd), torch.float32)
            gemm_tc(x, qkv_w, None, parts, EPI_PARTIAL, ksplit=ks)
            nsplit, part_o, part_ml, items, starts = _decode_scratch(ctx, cache, T, nh, nkv, hd, window)
            attention_decode_qkv_bf16(parts, qkv_b, table, ctx.max_positions, out, cache.k, cache.v, cache.block_table,
                                      ctx.positions, ctx.tok_seg, cache.num_pages, nh, window, scale, nsplit,
                                      part_o, part_ml, ctx.err, items=items, starts=starts)
            return
    q = qkv_rotate_store(ctx, x, qkv_w, qkv_b, nh, nkv, hd, rot, cache)
    attention(ctx, q, out, cache, window, scale)


def feed_forward_swiglu(ctx, x: torch.Tensor, gate_up_w: torch.Tensor, down_w: torch.Tensor):
    """``down(silu(gate(x)) * up(x))`` with the fused gate/up weight."""
    M, I = x.shape[0], gate_up_w.shape[0] // 2
    if tc_gemm_ok(x, gate_up_w, TC_GEMM_MAX_M_SWIGLU):
        act = ctx.alloc((M, I), x.dtype)
        gemm_tc(x, gate_up_w, None, act, EPI_SWIGLU)       # gate/up product with the SwiGLU in its epilogue
        return linear_delta(act, down_w)
    if x.dtype == torch.bfloat16 and gate_up_w.dtype == torch.bfloat16 and M <= GEMV_MAX_M \
            and gemv_supported(M, I, x.shape[1]) and (M == 1 or x.stride(0) % 8 == 0):
        act = ctx.alloc((M, I), x.dtype)
        gemv(x, gate_up_w, None, act, EPI_SWIGLU)        # gate/up product with the SwiGLU in its epilogue
        return linear_delta(act, down_w)
    gu = linear(x, gate_up_w)
    act = ctx.alloc((x.shape[0], gate_up_w.shape[0] // 2), x.dtype)
    swiglu(gu, act)
    return linear_delta(act, down_w)
