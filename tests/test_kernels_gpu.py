"""Each CUDA kernel alone against a plain PyTorch float32 reference of the same
op, at sizes other than the tiny engine configurations use (GPU)."""


import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from prism_b200 import ops
    return ops


def _err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


# --------------------------------------------------------------------------
# references
# --------------------------------------------------------------------------

def ref_rmsnorm(x, w, eps):
    x = x.float()
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()


def ref_rope(x, positions, inv_freq, rd):
    """x [T, heads, hd] float32; rotate-half pairing over the first rd dims."""
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., :rd // 2], x[..., rd // 2:rd]
    out = x.clone()
    out[..., :rd // 2] = x1 * cos - x2 * sin
    out[..., rd // 2:rd] = x2 * cos + x1 * sin
    return out


def ref_paged_attention(q, k_cache, v_cache, block_table, positions, tok_seg, window, scale):
    """q [T, nh, hd]; caches [pages, P, nkv, hd]; float32 math, one token at a time."""
    T, nh, hd = q.shape
    P, nkv = k_cache.shape[1], k_cache.shape[2]
    g = nh // nkv
    kf = k_cache.float().reshape(-1, nkv, hd)
    vf = v_cache.float().reshape(-1, nkv, hd)
    out = torch.empty(T, nh, hd, dtype=torch.float32, device=q.device)
    for t in range(T):
        pos, seg = int(positions[t]), int(tok_seg[t])
        lo = max(0, pos - window + 1) if window else 0
        idx = torch.arange(lo, pos + 1, device=q.device)
        rows = block_table[seg][idx // P].long() * P + idx % P
        K = kf[rows].repeat_interleave(g, dim=1)          # [n, nh, hd]
        V = vf[rows].repeat_interleave(g, dim=1)
        s = torch.einsum("hd,nhd->hn", q[t].float(), K) * scale
        p = torch.softmax(s, dim=-1)
        out[t] = torch.einsum("hn,nhd->hd", p, V)
    return out.reshape(T, nh * hd)


class PagedCase:
    """Random requests laid out in a paged cache whose unused slots hold NaN,
    so that a read of a slot that no request owns (a wrong page, an unmasked
    tail of a page) poisons the output."""

    def __init__(self, segs, nh, nkv, hd, P, dtype, seed, num_pages=None, table_width=None):
        # segs: list of (cached_len, q_len)
        g = torch.Generator().manual_seed(seed)
        self.S = len(segs)
        total_pages = sum((c + n + P - 1) // P for c, n in segs)
        self.num_pages = num_pages or total_pages + 3
        W = table_width or max((c + n + P - 1) // P for c, n in segs) + 2
        perm = torch.randperm(self.num_pages, generator=g).tolist()
        self.k = torch.full((self.num_pages, P, nkv, hd), float("nan"), dtype=dtype, device=DEV)
        self.v = torch.full((self.num_pages, P, nkv, hd), float("nan"), dtype=dtype, device=DEV)
        bt = torch.full((self.S, W), -7, dtype=torch.int32)
        pos, seg_of, seg_start, cached, qlens = [], [], [0], [], []
        for s, (c, n) in enumerate(segs):
            for i in range((c + n + P - 1) // P):
                bt[s, i] = perm.pop()
            L = c + n
            kk = (torch.randn(L, nkv, hd, generator=g)).to(dtype)
            vv = (torch.randn(L, nkv, hd, generator=g)).to(dtype)
            idx = torch.arange(L)
            rows = (bt[s][idx // P].long() * P + idx % P).to(DEV)
            self.k.view(-1, nkv, hd)[rows] = kk.to(DEV)
            self.v.view(-1, nkv, hd)[rows] = vv.to(DEV)
            pos += list(range(c, c + n))
            seg_of += [s] * n
            seg_start.append(seg_start[-1] + n)
            cached.append(c)
            qlens.append(n)
        self.T = len(pos)
        self.q = (torch.randn(self.T, nh, hd, generator=g)).to(dtype).to(DEV)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        self.bt = bt.to(DEV)
        self.positions, self.tok_seg = i32(pos), i32(seg_of)
        self.seg_start, self.cached_len = i32(seg_start), i32(cached)
        self.max_q = max(qlens)
        self.max_kv = max(c + n for c, n in segs)


# --------------------------------------------------------------------------
# elementwise / norm / rope / embed / gemm / sample
# --------------------------------------------------------------------------

@pytest.mark.parametrize("T,H,V", [(5, 200, 77), (33, 3584, 1000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(T, H, V, dtype):
    ops = _ops()
    table = _rand((V, H), dtype, 1)
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(2)).to(torch.int32).to(DEV)
    out = torch.empty(T, H, dtype=torch.float32, device=DEV)
    err = _err()
    ops.embed(ids, table, out, err)
    assert torch.equal(out, table[ids.long()].float()) and int(err) == 0
    ids[1] = V                                        # outside the vocabulary: flagged, row zeroed, no fault
    ops.embed(ids, table, out, err)
    assert int(err) == 1 and float(out[1].abs().max()) == 0.0


@pytest.mark.parametrize("T,H", [(3, 96), (17, 1000), (64, 3584), (2, 8192)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nsplit", [0, 1, 3])
def test_add_rmsnorm(T, H, dtype, nsplit):
    ops = _ops()
    eps = 3e-6
    res = _rand((T, H), torch.float32, 3)
    w = _rand((H,), dtype, 4) + 1
    ref_res = res.clone()
    delta = None
    if nsplit == 1:
        delta = _rand((T, H), dtype, 5)
        ref_res = ref_res + delta.float()
    elif nsplit > 1:
        delta = _rand((nsplit, T, H), torch.float32, 5)
        ref_res = ref_res + delta.sum(0)
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(res, delta, w, eps, out)
    ref = ref_rmsnorm(ref_res, w, eps)
    assert torch.allclose(res, ref_res, atol=1e-6, rtol=1e-6)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(out.float(), ref, atol=tol, rtol=tol)
    # rows: only the listed rows are normed
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(res, None, w, eps, out2, rows)
    assert torch.allclose(out2.float(), ref[[T - 1, 0]], atol=tol, rtol=tol)


@pytest.mark.parametrize("M,N,K", [(1, 100, 96), (7, 333, 224), (16, 64, 64), (65, 129, 100), (200, 520, 3584)])
def test_sgemm(M, N, K):
    ops = _ops()
    x, w, b = _rand((M, K), torch.float32, 6), _rand((N, K), torch.float32, 7, 0.05), _rand((N,), torch.float32, 8)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.sgemm(x, w, b, out)
    ref = (x.double() @ w.double().T + b.double()).float()
    assert torch.allclose(out, ref, atol=2e-5, rtol=1e-5)
    # a row's result does not depend on the batch it is in
    out1 = torch.empty(1, N, dtype=torch.float32, device=DEV)
    ops.sgemm(x[M // 2:M // 2 + 1].contiguous(), w, b, out1)
    assert torch.equal(out1[0], out[M // 2])


@pytest.mark.parametrize("M,N,K", [(1, 152, 96), (8, 4608, 3584), (300, 1000, 512)])
def test_linear_bf16(M, N, K):
    ops = _ops()
    x, w, b = _rand((M, K), torch.bfloat16, 6), _rand((N, K), torch.bfloat16, 7, 0.05), _rand((N,), torch.bfloat16, 8)
    ref = x.float() @ w.float().T + b.float()
    out = ops.linear(x, w, b)
    assert out.dtype == torch.bfloat16 and torch.allclose(out.float(), ref, atol=3e-2, rtol=2e-2)
    out32 = ops.linear(x, w, None, out_dtype=torch.float32)
    assert out32.dtype == torch.float32 and torch.allclose(out32, x.float() @ w.float().T, atol=2e-3, rtol=2e-3)
    # a weight the file stores in 32-bit stays so and goes through the float32 kernel
    out_mixed = ops.linear(x, w.float(), b)
    assert out_mixed.dtype == torch.bfloat16 and torch.allclose(out_mixed.float(), ref, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 23, 32])
@pytest.mark.parametrize("N,K", [(4608, 3584), (3584, 18944), (100, 96), (1000, 40), (17, 3000), (152064 // 16 + 3, 512)])
def test_gemv_bf16(M, N, K):
    """The weight-streaming small-M product alone: bf16 and float32 outputs with
    bias, and the paired-SwiGLU epilogue, against float32 references."""
    ops = _ops()
    x = _rand((M, K), torch.bfloat16, 30)
    w = _rand((N, K), torch.bfloat16, 31, 0.05)
    b = _rand((N,), torch.bfloat16, 32)
    ref = x.float() @ w.float().T + b.float()
    scale = float(ref.abs().max())
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemv(x, w, b, out, ops.EPI_BF16)
    assert torch.allclose(out.float(), ref, atol=8e-3 * scale, rtol=1e-2)
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemv(x, w, None, out32, ops.EPI_F32)
    assert torch.allclose(out32, ref - b.float(), atol=2e-3 * scale, rtol=2e-3)
    if N % 2 == 0:
        I = N // 2
        act = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemv(x, w, None, act, ops.EPI_SWIGLU)
        g, u = (ref - b.float())[:, :I], (ref - b.float())[:, I:]
        r = g * torch.sigmoid(g) * u
        assert torch.allclose(act.float(), r, atol=1e-2 * float(r.abs().max()) + 1e-3, rtol=2e-2)


@pytest.mark.parametrize("M", [1, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K", [(256, 128), (4608, 3584), (3584, 18944), (100, 96), (1000, 40), (130, 3000), (9507, 512)])
def test_gemm_tcgen05(M, N, K):
    """The tcgen05 + TMA weight-streaming product alone: every epilogue, K tails
    (K % 64 != 0), N tails (N % 128 != 0), token counts up to 64, K-splits."""
    ops = _ops()
    x = _rand((M, K), torch.bfloat16, 40)
    w = _rand((N, K), torch.bfloat16, 41, 0.05)
    b = _rand((N,), torch.bfloat16, 42)
    err = _err()
    ref = x.float() @ w.float().T
    scale = float(ref.abs().max())
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x, w, b, out, ops.EPI_BF16, err=err)
    assert int(err) == 0
    assert torch.allclose(out.float(), ref + b.float(), atol=8e-3 * scale + 8e-3, rtol=1e-2)
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tc(x, w, None, out32, ops.EPI_F32, err=err)
    assert torch.allclose(out32, ref, atol=2e-3 * scale, rtol=2e-3)
    for ks in (2, 5):
        part = torch.full((ks, M, N), float("nan"), dtype=torch.float32, device=DEV)
        ops.gemm_tc(x, w, None, part, ops.EPI_PARTIAL, ksplit=ks, err=err)
        assert torch.allclose(part.sum(0), ref, atol=2e-3 * scale, rtol=2e-3)
        # split K with the sum inside the kernel (the last CTA of a tile adds up): twice, same bits
        o1 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        o2 = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
        o3 = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
        ops.gemm_tc(x, w, b, o1, ops.EPI_BF16, ksplit=ks, err=err)
        ops.gemm_tc(x, w, b, o2, ops.EPI_F32, ksplit=ks, err=err)
        ops.gemm_tc(x, w, b, o3, ops.EPI_F32, ksplit=ks, err=err)
        assert torch.allclose(o1.float(), ref + b.float(), atol=8e-3 * scale + 8e-3, rtol=1e-2)
        assert torch.allclose(o2, ref + b.float(), atol=2e-3 * scale, rtol=2e-3) and torch.equal(o2, o3)
    if N % 2 == 0:
        I = N // 2
        act = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_tc(x, w, None, act, ops.EPI_SWIGLU, err=err)
        g, u = ref[:, :I], ref[:, I:]
        r = g * torch.sigmoid(g) * u
        assert torch.allclose(act.float(), r, atol=1e-2 * float(r.abs().max()) + 1e-3, rtol=2e-2)
    assert int(err) == 0


def test_split_k_workspace_outgrown_after_a_graph_was_captured():
    """A graph captured with the K-split product's workspace keeps replaying correctly after a later eager
    call has outgrown that workspace: the old one stays allocated, so nobody else's data can land where the
    graph still writes its partial sums and counts its arrivals."""
    ops = _ops()
    N, K, ks = 3584, 3584, 5
    w = _rand((N, K), torch.bfloat16, 70, 0.05)
    b = _rand((N,), torch.bfloat16, 71)
    x8, x64 = _rand((8, K), torch.bfloat16, 72), _rand((64, K), torch.bfloat16, 73)
    ref8 = x8.float() @ w.float().T + b.float()
    ops._tc_ws.clear()                                        # start from the initial size, as a fresh process does
    out8 = torch.empty(8, N, dtype=torch.float32, device=DEV)
    ops.gemm_tc(x8, w, b, out8, ops.EPI_F32, ksplit=ks)      # sizes the workspace (1 Mi floats) before capture
    first = ops._tc_ws[0][0]
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        ops.gemm_tc(x8, w, b, out8, ops.EPI_F32, ksplit=ks)
    torch.cuda.synchronize()
    out64 = torch.empty(64, N, dtype=torch.float32, device=DEV)
    ops.gemm_tc(x64, w, b, out64, ops.EPI_F32, ksplit=ks)    # 5 * 64 * 3584 floats: more than the first workspace
    assert ops._tc_ws[0][0].numel() > first.numel() and ops._tc_ws[0][0].data_ptr() != first.data_ptr()
    del first
    # whatever the allocator hands out now must not be the graph's workspace
    junk = [torch.full((1 << 20,), float("nan"), device=DEV) for _ in range(8)]
    out8.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    scale = float(ref8.abs().max())
    assert torch.allclose(out8, ref8, atol=2e-3 * scale, rtol=2e-3)
    assert all(bool(torch.isnan(j).all()) for j in junk), "the replay wrote into memory that was given away"
    assert torch.allclose(out64, x64.float() @ w.float().T + b.float(), atol=2e-3 * scale, rtol=2e-3)


@pytest.mark.parametrize("T,I", [(3, 100), (40, 18944)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(T, I, dtype):
    ops = _ops()
    gu = _rand((T, 2 * I), dtype, 9, 2.0)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    g, u = gu[:, :I].float(), gu[:, I:].float()
    ref = g * torch.sigmoid(g) * u
    tol = 1e-6 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.float(), ref, atol=tol, rtol=tol)


def test_rope_table_at_far_positions():
    """cos/sin of position x inverse frequency in float32 with full range reduction: angles of
    tens of thousands of radians (position 131,071, theta 1e6) still match the CPU's."""
    ops = _ops()
    hd, theta = 128, 1e6
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    pos = torch.tensor([0, 1, 77, 4095, 32767, 131071], dtype=torch.int32)
    table = torch.empty(pos.shape[0], hd // 2, 2, device=DEV)
    ops.rope_table(pos.to(DEV), inv.to(DEV), table)
    ang = torch.outer(pos.float(), inv)                       # float32 product, as andre-fu/prism forms it
    assert torch.allclose(table[..., 0].cpu(), torch.cos(ang), atol=2e-6, rtol=0)
    assert torch.allclose(table[..., 1].cpu(), torch.sin(ang), atol=2e-6, rtol=0)


@pytest.mark.parametrize("nh,nkv,hd,rd,P", [(5, 1, 48, 48, 8), (28, 4, 128, 128, 256), (6, 3, 80, 32, 16), (2, 2, 16, 0, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("use_table", [False, True])
def test_rope_kv_write(nh, nkv, hd, rd, P, dtype, use_table):
    ops = _ops()
    T, S, W = 23, 3, 40
    pages = S * W
    qkv = _rand((T, (nh + 2 * nkv) * hd), dtype, 10)
    before = qkv.clone()
    q = qkv[:, :nh * hd].view(T, nh, hd)
    k = qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
    g = torch.Generator().manual_seed(11)
    tok_seg = torch.sort(torch.randint(0, S, (T,), generator=g)).values.to(torch.int32)
    positions = torch.zeros(T, dtype=torch.int32)
    start = [0, 100, 7]
    for s in range(S):
        n = int((tok_seg == s).sum())
        positions[tok_seg == s] = torch.arange(start[s], start[s] + n, dtype=torch.int32)
    # the positions used below touch distinct pages per request
    bt = torch.arange(S * W, dtype=torch.int32).view(S, W) % pages
    kc = torch.zeros(pages, P, nkv, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    theta = 1e6
    inv = (1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))).to(DEV) if rd else None
    err = _err()
    table = None
    if use_table and rd:
        table = torch.empty(T, rd // 2, 2, dtype=torch.float32, device=DEV)
        ops.rope_table(positions.to(DEV), inv, table)
    ops.rope_kv_write(q, k, v, positions.to(DEV), tok_seg.to(DEV), inv, rd, kc, vc, bt.to(DEV), pages, 10 ** 6, err,
                      table=table)
    assert int(err) == 0
    bq = before[:, :nh * hd].view(T, nh, hd).float()
    bk = before[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd).float()
    bv = before[:, (nh + nkv) * hd:].view(T, nkv, hd)
    rq = ref_rope(bq, positions.to(DEV), inv, rd) if rd else bq
    rk = ref_rope(bk, positions.to(DEV), inv, rd) if rd else bk
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(q.float(), rq, atol=tol, rtol=tol)
    assert torch.allclose(k.float(), rk, atol=tol, rtol=tol)
    for t in range(T):
        s, p = int(tok_seg[t]), int(positions[t])
        page = int(bt[s, p // P])
        assert torch.equal(kc[page, p % P], k[t]) and torch.equal(vc[page, p % P], bv[t])
    assert int((kc != 0).any(dim=-1).any(dim=-1).sum()) <= T      # nothing else was written


@pytest.mark.parametrize("nh,nkv,hd,rd,P", [(28, 4, 128, 128, 256), (6, 3, 80, 32, 16), (5, 1, 48, 48, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_bias", [True, False])
def test_rope_kv_write_from_partial_sums(nh, nkv, hd, rd, P, dtype, with_bias):
    """q/k/v given as a stack of float32 partial sums plus bias: same q, same
    cache contents as summing first and using the in-place kernel."""
    ops = _ops()
    T, S, W, ks = 11, 2, 30, 3
    pages = S * W
    D = (nh + 2 * nkv) * hd
    parts = _rand((ks, T, D), torch.float32, 50)
    bias = _rand((D,), dtype, 51) if with_bias else None
    total = parts.sum(0) + (bias.float() if with_bias else 0)
    tok_seg = torch.tensor([0] * 6 + [1] * 5, dtype=torch.int32, device=DEV)
    positions = torch.tensor(list(range(40, 46)) + list(range(0, 5)), dtype=torch.int32, device=DEV)
    bt = (torch.arange(S * W, dtype=torch.int32).view(S, W)).to(DEV)
    theta = 1e4
    inv = (1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))).to(DEV)
    table = torch.empty(T, rd // 2, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(positions, inv, table)
    err = _err()
    kc = torch.zeros(pages, P, nkv, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    q = torch.empty(T, nh, hd, dtype=dtype, device=DEV)
    ops.rope_kv_write_partial(parts, bias, q, positions, tok_seg, table, rd, kc, vc, bt, pages, 1 << 20, nkv, err)
    # reference: float32 sum, float32 rotation, one rounding
    tq = total[:, :nh * hd].view(T, nh, hd)
    tk = total[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    tv = total[:, (nh + nkv) * hd:].view(T, nkv, hd)
    rq, rk = ref_rope(tq, positions, inv, rd), ref_rope(tk, positions, inv, rd)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert int(err) == 0 and torch.allclose(q.float(), rq, atol=tol, rtol=tol)
    for t in range(T):
        s_, p_ = int(tok_seg[t]), int(positions[t])
        page = int(bt[s_, p_ // P])
        assert torch.allclose(kc[page, p_ % P].float(), rk[t], atol=tol, rtol=tol)
        assert torch.allclose(vc[page, p_ % P].float(), tv[t], atol=tol, rtol=tol)


def test_sample_greedy_and_temperature():
    ops = _ops()
    R, V = 9, 152064 // 8 + 5
    logits = _rand((R, V), torch.float32, 12, 3.0)
    logits[3, 100] = logits[3, 7] = logits[3].max() + 1           # a tie: the lowest index wins
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample(logits, None, None, out)                       # V >= 8192: the many-blocks-per-row kernel
    ref = logits.argmax(-1)
    ref[3] = 7
    assert torch.equal(out.long(), ref)
    ops.sample(logits, None, None, out)                       # again: its counters reset themselves
    assert torch.equal(out.long(), ref)
    small = logits[:, :1000].contiguous()                     # small vocabulary: one block per row
    small[3, 7] = small[3, 100] = small[3].max() + 1
    ops.sample(small, None, None, out)
    rs = small.argmax(-1)
    rs[3] = 7
    assert torch.equal(out.long(), rs)
    temps = torch.tensor([0.7, 0.0, 1.3, 0.2, 1.0, 0.5, 2.0, 0.9, 1.1], device=DEV)
    us = torch.tensor([0.0, 0.5, 0.999999, 0.3, 0.25, 0.75, 0.5, 0.1, 0.9], device=DEV)
    ops.sample(logits, temps, us, out)
    for r in range(R):
        if temps[r] <= 0:
            assert int(out[r]) == int(ref[r])
            continue
        p = torch.softmax(logits[r].double() / float(temps[r]), -1)
        c = torch.cumsum(p, -1)
        tok = int(out[r])
        lo = float(c[tok - 1]) if tok > 0 else 0.0
        # the drawn token's cumulative interval contains u (to float32 rounding of the sums)
        assert lo - 1e-4 <= float(us[r]) <= float(c[tok]) + 1e-4, (r, tok, lo, float(us[r]), float(c[tok]))


# --------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------

GENERIC_CASES = [
    # nh, nkv, hd, P, window, segs (cached, q_len)
    (5, 1, 48, 8, None, [(0, 19), (37, 1), (5, 6)]),
    (6, 3, 80, 16, 11, [(0, 40), (30, 1), (16, 16)]),
    (28, 4, 128, 64, None, [(100, 3), (0, 70)]),
    (3, 3, 16, 4, 5, [(0, 9), (9, 2)]),
    (2, 1, 256, 32, None, [(50, 2)]),
]


@pytest.mark.parametrize("case", GENERIC_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_generic(case, dtype):
    ops = _ops()
    nh, nkv, hd, P, window, segs = case
    c = PagedCase(segs, nh, nkv, hd, P, dtype, seed=20)
    out = torch.empty(c.T, nh * hd, dtype=dtype, device=DEV)
    err = _err()
    scale = hd ** -0.5
    ops.attention_generic(c.q, out, c.k, c.v, c.bt, c.positions, c.tok_seg, c.num_pages, window, scale, err)
    ref = ref_paged_attention(c.q, c.k, c.v, c.bt, c.positions, c.tok_seg, window, scale)
    assert int(err) == 0 and not torch.isnan(out.float()).any()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.float(), ref, atol=tol, rtol=tol)


def test_attention_generic_rejects_big_head():
    ops = _ops()
    c = PagedCase([(0, 2)], 1, 1, 272, 16, torch.float32, seed=1)
    with pytest.raises(ops.KernelError):
        ops.attention_generic(c.q, torch.empty(2, 272, device=DEV), c.k, c.v, c.bt, c.positions, c.tok_seg,
                              c.num_pages, None, 1.0, _err())


def test_the_host_side_shape_rule_is_the_library_s():
    ops = _ops()
    for hd in (16, 32, 48, 64, 80, 96, 128, 256):
        for nh, nkv in ((4, 2), (28, 4), (40, 8), (32, 1), (16, 1), (17, 1), (3, 3), (6, 4)):
            assert ops.attention_bf16_shape_ok(hd, nh, nkv) == ops.attention_bf16_supported(hd, nh, nkv), (hd, nh, nkv)


DECODE_CASES = [
    # nh, nkv, hd, P, window, contexts (cached lens; one new token each), nsplit
    (28, 4, 128, 256, None, [2048, 1, 0, 255, 256, 257, 4000], 10),
    (28, 4, 128, 64, None, [63, 64, 65, 1000], 1),
    (8, 8, 64, 16, None, [5, 300, 129], 3),
    (28, 4, 128, 256, None, [2100, 2047, 1, 64, 700, 4095, 33, 1000], 8),
    (16, 1, 64, 32, 100, [99, 100, 101, 700, 3], 7),
    (14, 2, 128, 8, 64, [1500, 64, 63], 64),
    (40, 8, 128, 256, None, [3000], 33),
    (14, 2, 64, 256, None, [300, 17, 700, 64, 1] + [0] * 11, 9),        # a graph bucket of 16 with padded rows
    (14, 2, 64, 256, None, [300, 17, 700, 64, 1], 11),
    (12, 2, 128, 64, None, [129, 64, 1000, 0, 0, 0, 0, 0], 5),
    # every head size in steps of 16 (an odd number of 16-wide steps: 16, 48, 80, 112)
    (4, 2, 16, 16, None, [200, 15, 16, 0], 3),
    (3, 1, 32, 8, None, [77, 300], 2),
    (6, 3, 48, 16, 24, [23, 24, 25, 500], 4),
    (10, 2, 80, 32, None, [1000, 31], 6),
    (8, 8, 96, 64, None, [130, 64], 1),
    (16, 1, 112, 256, None, [700, 257, 3], 5),
]


@pytest.mark.parametrize("case", DECODE_CASES)
def test_attention_decode_bf16(case):
    ops = _ops()
    nh, nkv, hd, P, window, ctxs, nsplit = case
    c = PagedCase([(n, 1) for n in ctxs], nh, nkv, hd, P, torch.bfloat16, seed=21)
    out = torch.empty(c.T, nh * hd, dtype=torch.bfloat16, device=DEV)
    part_o = torch.full((c.T, nh, nsplit, hd), float("nan"), device=DEV)
    part_ml = torch.full((c.T, nh, nsplit, 2), float("nan"), device=DEV)
    err = _err()
    scale = hd ** -0.5
    ref = ref_paged_attention(c.q, c.k, c.v, c.bt, c.positions, c.tok_seg, window, scale)
    for _ in range(2):
        out.fill_(float("nan"))
        ops.attention_decode_bf16(c.q, out, c.k, c.v, c.bt, c.positions, c.tok_seg, c.num_pages, window, scale,
                                  nsplit, part_o, part_ml, err)
        assert int(err) == 0 and not torch.isnan(out.float()).any()
        assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), float((out.float() - ref).abs().max())


def _work_items(ops, ctxs, nkv, window, sms, places=None):
    """The host's work items for a step on the device; ``places``: a grid with more places than items."""
    items, starts, most = ops.decode_work_items(ctxs, nkv, window, sms=sms)
    if places:
        import numpy as np
        items = np.concatenate([items, np.full((places - len(items), 4), -1, dtype=np.int32)])
    return torch.from_numpy(items).to(DEV), torch.from_numpy(starts).to(DEV), most


@pytest.mark.parametrize("case", DECODE_CASES)
@pytest.mark.parametrize("sms", [1, 6, 40, 148, 2000])
def test_attention_decode_bf16_on_work_items(case, sms):
    """With work items every request is shared among the CTAs that the host chose from its own length (here for
    GPUs of 1 to 2,000 SMs, so from one CTA each to as many as three tiles allow); a grid with places to spare
    leaves them alone; partial results are NaN beforehand and positions and segments are not read."""
    ops = _ops()
    nh, nkv, hd, P, window, ctxs, _ = case
    c = PagedCase([(n, 1) for n in ctxs], nh, nkv, hd, P, torch.bfloat16, seed=22)
    scale, err = hd ** -0.5, _err()
    ref = ref_paged_attention(c.q, c.k, c.v, c.bt, c.positions, c.tok_seg, window, scale)
    junk = torch.full_like(c.positions, 1 << 20)
    for places in (None, 700):
        items, starts, most = _work_items(ops, ctxs, nkv, window, sms, places)
        n = items.shape[0]
        out = torch.full((c.T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        part_o = torch.full((n, nh, hd), float("nan"), device=DEV)
        part_ml = torch.full((n, nh, 2), float("nan"), device=DEV)
        ops.attention_decode_bf16(c.q, out, c.k, c.v, c.bt, junk, junk, c.num_pages, window, scale,
                                  most, part_o, part_ml, err, items=items, starts=starts)
        assert int(err) == 0 and not torch.isnan(out.float()).any()
        assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), float((out.float() - ref).abs().max())
        # a request with one item wrote its output itself; the others left one partial per item
        used = (starts >> 16).tolist()
        # (a token's slots: [head][split] from its first item on)
        written = (~torch.isnan(part_ml[:, :, 0])).sum(1).tolist()          # per item row: nh slots
        want = [nh if tok >= 0 and used[tok] > 1 else 0 for tok in items[:, 0].tolist()]
        assert written == want and sum(used) == (items[:, 0] >= 0).sum().item(), (used, written)


def test_attention_decode_qkv_on_work_items():
    """The decode kernel that finishes the projection takes the same work items."""
    ops = _ops()
    nh, nkv, hd, P, window, ctxs = 12, 2, 128, 64, None, [1300, 64, 200, 0, 5000]
    c = PagedCase([(n, 1) for n in ctxs], nh, nkv, hd, P, torch.bfloat16, seed=23)
    T, ks, D = c.T, 2, (nh + 2 * nkv) * hd
    parts = _rand((ks, T, D), torch.float32, 62, scale=0.5)
    inv = (1.0 / (1e4 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))).to(DEV)
    table = torch.empty(T, hd // 2, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(c.positions, inv, table)
    scale, err = hd ** -0.5, _err()
    outs = []
    for planned in (False, True):
        k, v = c.k.clone(), c.v.clone()
        got = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        if planned:
            items, starts, most = _work_items(ops, ctxs, nkv, window, 20, places=64)
            assert most > 1 and (starts >> 16).sum().item() > T
            po = torch.full((items.shape[0], nh, hd), float("nan"), device=DEV)
            pml = torch.full((items.shape[0], nh, 2), float("nan"), device=DEV)
        else:
            items, starts, most = None, None, 16
            po = torch.full((T, nh, most, hd), float("nan"), device=DEV)
            pml = torch.full((T, nh, most, 2), float("nan"), device=DEV)
        ops.attention_decode_qkv_bf16(parts, None, table, 1 << 20, got, k, v, c.bt, c.positions, c.tok_seg, c.num_pages,
                                      nh, window, scale, most, po, pml, err, items=items, starts=starts)
        assert int(err) == 0 and not torch.isnan(got.float()).any()
        outs.append((got.float(), k, v))
    assert torch.allclose(outs[0][0], outs[1][0], atol=4e-3, rtol=1e-2)
    for a, b in ((outs[0][1], outs[1][1]), (outs[0][2], outs[1][2])):       # the tokens' own keys and values were stored
        assert torch.equal(torch.isnan(a), torch.isnan(b)) and torch.equal(a.nan_to_num(), b.nan_to_num())


@pytest.mark.parametrize("case", DECODE_CASES + [(8, 2, 64, 16, 40, [100, 39, 40, 41, 0], 3)])     # head sizes 16 .. 128
@pytest.mark.parametrize("bias_dtype", [None, torch.bfloat16, torch.float32])
def test_attention_decode_finishes_the_qkv_projection(case, bias_dtype):
    """The decode kernel given the projection's partial sums instead of q and a filled cache: the same output
    and the same cache contents as the rotary + store kernel followed by the plain decode kernel.  The
    tokens' own cache rows hold NaN beforehand: they must be computed, not read."""
    ops = _ops()
    nh, nkv, hd, P, window, ctxs, nsplit = case
    c = PagedCase([(n, 1) for n in ctxs], nh, nkv, hd, P, torch.bfloat16, seed=27)
    T, ks, D = c.T, 3, (nh + 2 * nkv) * hd
    parts = _rand((ks, T, D), torch.float32, 60, scale=0.5)
    bias = None if bias_dtype is None else _rand((D,), bias_dtype, 61, scale=0.5)
    inv = (1.0 / (1e4 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))).to(DEV)
    table = torch.empty(T, hd // 2, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(c.positions, inv, table)
    scale, err = hd ** -0.5, _err()
    # two kernels
    k1, v1 = c.k.clone(), c.v.clone()
    q = torch.empty(T, nh, hd, dtype=torch.bfloat16, device=DEV)
    ops.rope_kv_write_partial(parts, bias, q, c.positions, c.tok_seg, table, hd, k1, v1, c.bt, c.num_pages, 1 << 20, nkv, err)
    want = torch.empty(T, nh * hd, dtype=torch.bfloat16, device=DEV)
    mk = lambda: (torch.full((T, nh, nsplit, hd), float("nan"), device=DEV), torch.full((T, nh, nsplit, 2), float("nan"), device=DEV))
    po, pml = mk()
    ops.attention_decode_bf16(q, want, k1, v1, c.bt, c.positions, c.tok_seg, c.num_pages, window, scale, nsplit, po, pml,
                              err)
    ref = ref_paged_attention(q, k1, v1, c.bt, c.positions, c.tok_seg, window, scale)
    assert int(err) == 0 and torch.allclose(want.float(), ref, atol=2e-2, rtol=2e-2)
    # one kernel
    k2, v2 = c.k.clone(), c.v.clone()
    for t, n in enumerate(ctxs):
        k2[int(c.bt[t, n // P]), n % P] = float("nan")
        v2[int(c.bt[t, n // P]), n % P] = float("nan")
    for _ in range(2):
        got = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        po, pml = mk()
        ops.attention_decode_qkv_bf16(parts, bias, table, 1 << 20, got, k2, v2, c.bt, c.positions, c.tok_seg, c.num_pages,
                                      nh, window, scale, nsplit, po, pml, err)
        assert int(err) == 0 and not torch.isnan(got.float()).any()
        assert torch.allclose(got.float(), want.float(), atol=4e-3, rtol=1e-2), float((got.float() - want.float()).abs().max())
    # the caches agree wherever a request owns the slot (both hold NaN elsewhere)
    assert torch.equal(torch.isnan(k2), torch.isnan(k1)) and torch.equal(torch.isnan(v2), torch.isnan(v1))
    assert torch.allclose(k2.float().nan_to_num(), k1.float().nan_to_num(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(v2.float().nan_to_num(), v1.float().nan_to_num(), atol=1e-2, rtol=1e-2)


def test_attention_decode_qkv_reports_a_position_out_of_range():
    ops = _ops()
    nh, nkv, hd, P = 4, 2, 64, 16
    c = PagedCase([(20, 1), (5, 1)], nh, nkv, hd, P, torch.bfloat16, seed=28)
    parts = _rand((2, c.T, (nh + 2 * nkv) * hd), torch.float32, 62)
    table = torch.zeros(c.T, hd // 2, 2, dtype=torch.float32, device=DEV)
    err = _err()
    ops.attention_decode_qkv_bf16(parts, None, table, 20, torch.empty(c.T, nh * hd, dtype=torch.bfloat16, device=DEV),
                                  c.k, c.v, c.bt, c.positions, c.tok_seg, c.num_pages, nh, None, hd ** -0.5, 2,
                                  torch.empty(c.T, nh, 2, hd, device=DEV), torch.empty(c.T, nh, 2, 2, device=DEV), err)
    torch.cuda.synchronize()
    assert int(err) != 0                     # position 20 with max_pos 20


PREFILL_CASES = [
    (28, 4, 128, 256, None, [(0, 200), (300, 1), (64, 64), (5, 63), (0, 1), (1000, 65)]),
    (8, 8, 64, 16, None, [(0, 130), (17, 2)]),
    (16, 1, 64, 32, 50, [(0, 180), (49, 3), (50, 1), (400, 70)]),
    (14, 2, 128, 8, 64, [(100, 129), (0, 64)]),
    (4, 2, 16, 16, None, [(0, 150), (20, 3)]),
    (3, 1, 32, 8, None, [(5, 70), (0, 1)]),
    (6, 3, 48, 16, 24, [(0, 100), (23, 2), (200, 65)]),
    (10, 2, 80, 32, None, [(64, 64), (0, 130)]),
    (8, 8, 96, 64, None, [(0, 200)]),
    (16, 1, 112, 256, 300, [(250, 80), (0, 17)]),
]


@pytest.mark.parametrize("case", PREFILL_CASES)
def test_attention_prefill_bf16(case):
    ops = _ops()
    nh, nkv, hd, P, window, segs = case
    c = PagedCase(segs, nh, nkv, hd, P, torch.bfloat16, seed=22)
    out = torch.full((c.T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = _err()
    scale = hd ** -0.5
    ops.attention_prefill_bf16(c.q, out, c.k, c.v, c.bt, c.seg_start, c.cached_len, c.max_q, c.num_pages,
                               window, scale, err)
    ref = ref_paged_attention(c.q, c.k, c.v, c.bt, c.positions, c.tok_seg, window, scale)
    assert int(err) == 0 and not torch.isnan(out.float()).any()
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), float((out.float() - ref).abs().max())


PREFILL_TC_CASES = [
    (28, 4, 128, 256, None, [(0, 200), (300, 1), (64, 64), (5, 63), (0, 1), (1000, 65)]),
    (8, 8, 64, 64, None, [(0, 130), (17, 2)]),
    (16, 1, 64, 64, 50, [(0, 180), (49, 3), (50, 1), (400, 70)]),
    (14, 2, 128, 128, 64, [(100, 129), (0, 64)]),
    (4, 2, 128, 64, None, [(0, 700)]),
    (6, 2, 128, 192, None, [(130, 300), (0, 127), (0, 128), (63, 129)]),
    (3, 1, 64, 64, 200, [(0, 517)]),
    (4, 2, 128, 256, None, [(0, 3000)]),                 # 47 key tiles: the lazy rescale and both S buffers many times over
    (2, 1, 64, 64, None, [(1000, 2100), (3000, 90)]),
]


@pytest.mark.parametrize("nsplit", [1, 2, 5, 16])
@pytest.mark.parametrize("case", PREFILL_TC_CASES)
def test_attention_prefill_tc(case, nsplit):
    """The tcgen05 kernel: 128-row query tiles, keys by TMA through the block table.  With nsplit > 1 the
    key tiles of a query tile are shared among that many CTAs and merged afterwards; with more splits than
    key tiles some CTAs leave an empty partial result, and a split may hold only keys that a row cannot see."""
    ops = _ops()
    nh, nkv, hd, P, window, segs = case
    c = PagedCase(segs, nh, nkv, hd, P, torch.bfloat16, seed=24)
    out = torch.full((c.T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = _err()
    scale = hd ** -0.5
    assert ops.attention_prefill_tc_supported(hd, nh, nkv, P)
    ref = ref_paged_attention(c.q, c.k, c.v, c.bt, c.positions, c.tok_seg, window, scale)
    for _ in range(2):
        out.fill_(float("nan"))
        ops.attention_prefill_tc(c.q, out, c.k, c.v, c.bt, c.seg_start, c.cached_len, c.max_q, c.num_pages,
                                 window, scale, err, nsplit=nsplit)
        assert int(err) == 0 and not torch.isnan(out.float()).any()
        assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), float((out.float() - ref).abs().max())


def test_attention_prefill_tc_split_after_decode_tokens():
    """Split portions behind single decoded tokens in one batch, as a step has them: the kernel gets the
    segments from ``first`` on, indexes the partial results by the token's place in the whole batch, and the
    merge writes only the portions' rows."""
    ops = _ops()
    nh, nkv, hd, P, first = 8, 2, 128, 64, 3
    c = PagedCase([(70, 1), (0, 1), (900, 1), (2000, 140), (500, 33)], nh, nkv, hd, P, torch.bfloat16, seed=26)
    scale = hd ** -0.5
    ref = ref_paged_attention(c.q, c.k, c.v, c.bt, c.positions, c.tok_seg, None, scale)
    out = torch.full((c.T, nh * hd), 9.0, dtype=torch.bfloat16, device=DEV)
    err = _err()
    ops.attention_prefill_tc(c.q, out, c.k, c.v, c.bt[first:], c.seg_start[first:], c.cached_len[first:], 140,
                             c.num_pages, None, scale, err, nsplit=4, first_token=first)
    assert int(err) == 0
    assert torch.equal(out[:first].float(), torch.full_like(out[:first].float(), 9.0))      # not this call's rows
    assert torch.allclose(out[first:].float(), ref[first:], atol=2e-2, rtol=2e-2)


def test_attention_prefill_tc_is_reproducible():
    """The same call gives the same bits every time.  (A wait on a barrier whose phases are told
    apart by one parity bit once passed two phases early when the tensor pipe was busy with the
    neighbouring CTA; it showed as a different result every twentieth call or so.)"""
    ops = _ops()
    nh, nkv, hd, P = 28, 4, 128, 256
    c = PagedCase([(0, 1100)], nh, nkv, hd, P, torch.bfloat16, seed=25)
    err = _err()
    outs = []
    res = torch.zeros(c.T, 3584, device=DEV)
    w = torch.ones(3584, dtype=torch.bfloat16, device=DEV)
    normed = torch.empty(c.T, 3584, dtype=torch.bfloat16, device=DEV)
    for _ in range(120):
        out = torch.empty((c.T, nh * hd), dtype=torch.bfloat16, device=DEV)
        # a short kernel before it, as in a layer: the attention CTAs become resident while it runs
        # (programmatic dependent launch) and are released together
        ops.add_rmsnorm(res, None, w, 1e-6, normed)
        ops.attention_prefill_tc(c.q, out, c.k, c.v, c.bt, c.seg_start, c.cached_len, c.max_q, c.num_pages,
                                 None, hd ** -0.5, err)
        outs.append(out)
    torch.cuda.synchronize()
    assert int(err) == 0
    differ = [i for i, o in enumerate(outs) if not torch.equal(o, outs[0])]
    assert not differ, differ


def test_attention_prefill_tc_refuses():
    ops = _ops()
    assert not ops.attention_prefill_tc_supported(48, 4, 2, 64)
    assert not ops.attention_prefill_tc_supported(128, 4, 2, 16)
    c = PagedCase([(0, 20)], 4, 2, 128, 16, torch.bfloat16, seed=1)
    with pytest.raises(ops.KernelError):
        ops.attention_prefill_tc(c.q, torch.empty(c.T, 4 * 128, dtype=torch.bfloat16, device=DEV), c.k, c.v, c.bt,
                                 c.seg_start, c.cached_len, c.max_q, c.num_pages, None, 1.0, _err())


@pytest.mark.parametrize("kind", ["generic32", "generic16", "decode", "prefill", "prefill_tc", "prefill_tc_split"])
def test_attention_finds_one_far_key(kind):
    """One key among thousands carries the whole softmax: the query and that
    key are scaled so that its score stands out, and its value is marked.  A
    kernel that drops a tile, a split or a page loses the mark."""
    ops = _ops()
    nh, nkv, hd, P = 8, 2, 64, (64 if kind.startswith("prefill_tc") else 16)
    dtype = torch.float32 if kind == "generic32" else torch.bfloat16
    ctx = 3000
    segs = [(ctx, 1)] if not kind.startswith("prefill") else [(ctx - 40, 41)]
    for far in (0, 17, 1234, 2047, 2048, ctx - 1, ctx):
        c = PagedCase(segs, nh, nkv, hd, P, dtype, seed=23)
        c.q[:] = 0
        c.q[-1, :, 0] = 30.0                      # the last query looks along dim 0
        page, off = int(c.bt[0, far // P]), far % P
        c.k[page, off, :, 0] = 30.0               # the far key answers: score 900 * scale
        c.v[page, off] = 5.0
        out = torch.empty(c.T, nh * hd, dtype=dtype, device=DEV)
        err = _err()
        scale = hd ** -0.5
        if kind.startswith("generic"):
            ops.attention_generic(c.q, out, c.k, c.v, c.bt, c.positions, c.tok_seg, c.num_pages, None, scale, err)
        elif kind == "decode":
            ns = 9
            ops.attention_decode_bf16(c.q, out, c.k, c.v, c.bt, c.positions, c.tok_seg, c.num_pages, None, scale, ns,
                                      torch.empty(c.T, nh, ns, hd, device=DEV), torch.empty(c.T, nh, ns, 2, device=DEV), err)
        elif kind.startswith("prefill_tc"):
            ops.attention_prefill_tc(c.q, out, c.k, c.v, c.bt, c.seg_start, c.cached_len, c.max_q, c.num_pages,
                                     None, scale, err, nsplit=7 if kind.endswith("split") else 1)
        else:
            ops.attention_prefill_bf16(c.q, out, c.k, c.v, c.bt, c.seg_start, c.cached_len, c.max_q, c.num_pages,
                                       None, scale, err)
        assert int(err) == 0
        assert torch.allclose(out[-1].float(), torch.full_like(out[-1].float(), 5.0), atol=0.05), (kind, far, out[-1][:4])


@pytest.mark.parametrize("kind", ["generic32", "generic16", "decode", "prefill", "prefill_tc", "prefill_tc_split"])
def test_attention_window_edge(kind):
    """A sliding window's edge, made visible: the key just outside the window
    carries an enormous score and a marked value and must not be seen; the key
    just inside must be (move the mark there and it dominates)."""
    ops = _ops()
    nh, nkv, hd, P, window = 4, 2, 64, (64 if kind.startswith("prefill_tc") else 16), 37
    dtype = torch.float32 if kind == "generic32" else torch.bfloat16
    for ctx in (36, 37, 64, 100, 129, 500):                        # the query sits at position ctx
        segs = [(ctx, 1)] if not kind.startswith("prefill") else [(max(0, ctx - 5), ctx - max(0, ctx - 5) + 1)]
        for inside in (False, True):
            key = ctx - window + (1 if inside else 0)               # first key inside / last key outside
            if key < 0:
                continue
            c = PagedCase(segs, nh, nkv, hd, P, dtype, seed=31)
            c.q[-1] = 0
            c.q[-1, :, 1] = 25.0
            page, off = int(c.bt[0, key // P]), key % P
            c.k[page, off, :, 1] = 25.0
            c.v[page, off] = 7.0
            out = torch.empty(c.T, nh * hd, dtype=dtype, device=DEV)
            err = _err()
            scale = hd ** -0.5
            if kind.startswith("generic"):
                ops.attention_generic(c.q, out, c.k, c.v, c.bt, c.positions, c.tok_seg, c.num_pages, window, scale, err)
            elif kind == "decode":
                ns = 3
                ops.attention_decode_bf16(c.q, out, c.k, c.v, c.bt, c.positions, c.tok_seg, c.num_pages, window, scale, ns,
                                          torch.empty(c.T, nh, ns, hd, device=DEV), torch.empty(c.T, nh, ns, 2, device=DEV), err)
            elif kind.startswith("prefill_tc"):
                ops.attention_prefill_tc(c.q, out, c.k, c.v, c.bt, c.seg_start, c.cached_len, c.max_q, c.num_pages,
                                         window, scale, err, nsplit=3 if kind.endswith("split") else 1)
            else:
                ops.attention_prefill_bf16(c.q, out, c.k, c.v, c.bt, c.seg_start, c.cached_len, c.max_q, c.num_pages,
                                           window, scale, err)
            last = out[-1].float()
            assert int(err) == 0
            if inside:
                assert torch.allclose(last, torch.full_like(last, 7.0), atol=0.05), (kind, ctx, "inside key not found")
            else:
                assert float(last.abs().max()) < 3.0, (kind, ctx, "key outside the window was seen", float(last.abs().max()))
