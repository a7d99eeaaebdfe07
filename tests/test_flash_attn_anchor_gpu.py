"""The attention arithmetic against the call andre-fu/prism itself makes (GPU).

The reference computes attention and appends to its cache with one library
call, ``flash_attn_with_kvcache(q, k_cache, v_cache, k=, v=, cache_seqlens=,
block_table=, causal=True)`` (engine/executor.py:119-120 for prompts, :151-153
for decoding).  Everywhere else in this suite that call is stated, not run:
the plain model and the golden files carry this repository's reading of its
semantics (scale ``hd^-1/2``, causal mask aligned to the end of the keys,
q-head ``h`` on kv-head ``h // (nh/nkv)``, new keys appended at
``cache_seqlens``).  Here the library itself runs, exactly as the executor
calls it - pages of 256 tokens, bfloat16, the head counts of Qwen2.5-7B (28/4
of 128) and of Qwen2.5-0.5B (14/2 of 64) - for a whole prompt, for a
continuation after ``prefix_len`` cached tokens, and for one token appended at
``cache_seqlens``, and is compared with the plain attention function and with
this engine's kernels on the very cache the library filled.

flash-attn is library code and only a witness here: nothing of the product
imports it.  If the installed build has no kernels for this GPU the test is
skipped with the library's own message.  The sliding window is not covered:
the reference never passes one.
"""

import pytest
import torch

from helpers import P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
PAGE = 256


def _fa():
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as e:                                   # noqa: BLE001
        pytest.skip(f"flash_attn does not import: {type(e).__name__}: {e}")
    return flash_attn_with_kvcache


def _call(fa, *a, **k):
    """One library call; a build without kernels for this GPU raises here and skips the test."""
    try:
        out = fa(*a, **k)
        torch.cuda.synchronize()
        return out
    except RuntimeError as e:
        msg = " ".join(str(e).split())
        if any(w in msg for w in ("no kernel image", "not supported", "only supports", "Ampere", "invalid device function")):
            pytest.skip(f"flash_attn has no kernels for this GPU: {msg[:200]}")
        raise


def _ops():
    from prism_b200 import ops
    return ops


class Cache:
    """A paged cache as the reference lays it out (engine/kv_cache.py:36-46), pages in a scrambled order,
    unused slots NaN for this engine's kernels (the library call gets a zero-filled twin: it multiplies
    masked slots by zero, and NaN times zero would poison its output)."""

    def __init__(self, nkv, hd, total_tokens, seed):
        g = torch.Generator().manual_seed(seed)
        self.nblk = (total_tokens + PAGE - 1) // PAGE
        self.num_pages = self.nblk + 3
        perm = torch.randperm(self.num_pages, generator=g)[:self.nblk]
        self.bt = perm.to(torch.int32).view(1, self.nblk).to(DEV)
        self.k = torch.zeros(self.num_pages, PAGE, nkv, hd, dtype=torch.bfloat16, device=DEV)
        self.v = torch.zeros_like(self.k)

    def rows(self, n):
        idx = torch.arange(n, device=DEV)
        return self.bt[0][idx // PAGE].long() * PAGE + idx % PAGE


@pytest.mark.parametrize("nh,nkv,hd", [(28, 4, 128), (14, 2, 64)])
def test_the_reference_s_attention_call(nh, nkv, hd):
    fa, ops = _fa(), _ops()
    T, prefix, tail = 777, 300, 5                   # 777 tokens span four pages; the continuation starts inside the second
    g = torch.Generator().manual_seed(5)
    q = torch.randn(T, nh, hd, generator=g).to(torch.bfloat16)
    k = torch.randn(T, nkv, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(T, nkv, hd, generator=g).to(torch.bfloat16)
    # one key far back that stands out for one query of the continuation: a wrong mask or a wrong page shows
    k[7, :, :] = 4.0 * q[prefix + 40, ::nh // nkv, :]
    want = P.attention(q.float(), k.float(), v.float()).reshape(T, nh * hd)       # float32, whole sequence, no cache
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    scale = hd ** -0.5
    tol = dict(atol=2e-2, rtol=2e-2)

    def ours_on(cache, first, n):
        """This engine's kernels for tokens first .. first+n-1 over `cache`, which already holds their keys."""
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        ck, cv = cache.k.clone(), cache.v.clone()
        held = torch.zeros(cache.num_pages * PAGE, dtype=torch.bool, device=DEV)
        held[cache.rows(first + n)] = True
        ck.view(-1, nkv, hd)[~held] = float("nan")            # slots no request owns must never be read
        cv.view(-1, nkv, hd)[~held] = float("nan")
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        outs = {}
        qq = qd[first:first + n].contiguous()
        out = torch.full((n, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_bf16(qq, out, ck, cv, cache.bt, i32([0, n]), i32([first]), n, cache.num_pages, None, scale, err)
        outs["mma.sync portions"] = out
        out = torch.full((n, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_tc(qq, out, ck, cv, cache.bt, i32([0, n]), i32([first]), n, cache.num_pages, None, scale, err)
        outs["tcgen05 portions"] = out
        out = torch.full((n, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attention_generic(qq, out, ck, cv, cache.bt, i32(list(range(first, first + n))), i32([0] * n), cache.num_pages,
                              None, scale, err)
        outs["generic"] = out
        if n == 1:
            ns = 3
            out = torch.full((1, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
            ops.attention_decode_bf16(qq, out, ck, cv, cache.bt, i32([first]), i32([0]), cache.num_pages, None, scale, ns,
                                      torch.empty(1, nh, ns, hd, device=DEV), torch.empty(1, nh, ns, 2, device=DEV), err)
            outs["decode"] = out
        torch.cuda.synchronize()
        assert int(err) == 0
        return outs

    # ---- a whole prompt: cache_seqlens = 0, the call appends all keys and attends causally ----
    c = Cache(nkv, hd, T, seed=1)
    sl = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = _call(fa, qd[None], c.k, c.v, k=kd[None], v=vd[None], cache_seqlens=sl, block_table=c.bt, causal=True)
    got = got.reshape(T, nh * hd).float().cpu()
    assert torch.allclose(got, want, **tol), float((got - want).abs().max())
    # the append: token t's key sits at logical slot t of the request's pages
    assert torch.equal(c.k.view(-1, nkv, hd)[c.rows(T)].cpu(), k) and torch.equal(c.v.view(-1, nkv, hd)[c.rows(T)].cpu(), v)
    for name, o in ours_on(c, 0, T).items():
        assert torch.allclose(o.float().cpu(), got, **tol), (name, float((o.float().cpu() - got).abs().max()))

    # ---- a continuation after prefix_len cached tokens (executor.py:84-101 with prefix_len > 0) ----
    c = Cache(nkv, hd, T, seed=2)
    _call(fa, qd[None, :prefix], c.k, c.v, k=kd[None, :prefix], v=vd[None, :prefix],
          cache_seqlens=torch.zeros(1, dtype=torch.int32, device=DEV), block_table=c.bt, causal=True)
    n = T - tail - prefix
    sl = torch.full((1,), prefix, dtype=torch.int32, device=DEV)
    got = _call(fa, qd[None, prefix:prefix + n], c.k, c.v, k=kd[None, prefix:prefix + n], v=vd[None, prefix:prefix + n],
                cache_seqlens=sl, block_table=c.bt, causal=True).reshape(n, nh * hd).float().cpu()
    # the mask is aligned to the end of the keys: the row at position p sees keys 0 .. p, the far key among them
    assert torch.allclose(got, want[prefix:prefix + n], **tol), float((got - want[prefix:prefix + n]).abs().max())
    for name, o in ours_on(c, prefix, n).items():
        assert torch.allclose(o.float().cpu(), got, **tol), (name, float((o.float().cpu() - got).abs().max()))

    # ---- single tokens appended *at* cache_seqlens (what decoding means; the reference's decode entry points
    # pass cache_seqlens one too large, engine/executor.py:205-208, which this engine does not reproduce) ----
    for p in range(T - tail, T):
        sl = torch.full((1,), p, dtype=torch.int32, device=DEV)
        got = _call(fa, qd[None, p:p + 1], c.k, c.v, k=kd[None, p:p + 1], v=vd[None, p:p + 1], cache_seqlens=sl,
                    block_table=c.bt, causal=True).reshape(1, nh * hd).float().cpu()
        assert torch.allclose(got, want[p:p + 1], **tol), (p, float((got - want[p:p + 1]).abs().max()))
        for name, o in ours_on(c, p, 1).items():
            assert torch.allclose(o.float().cpu(), got, **tol), (name, p, float((o.float().cpu() - got).abs().max()))
    assert torch.equal(c.k.view(-1, nkv, hd)[c.rows(T)].cpu(), k)
