"""Times single kernels of prism_b200 on Qwen2.5-7B shapes with CUDA events,
flushing L2 between timed launches, and prints achieved bandwidth or FLOP/s.

    python benchmarks/kernel_bench.py gemv  [--m 8]
    python benchmarks/kernel_bench.py gemm_tc [--m 8]
    python benchmarks/kernel_bench.py attn_decode [--batch 8 --ctx 4096] [--ragged] [--splits N]
    python benchmarks/kernel_bench.py attn_prefill [--tokens 2048] [--mma-sync]
    python benchmarks/kernel_bench.py small [--m 8]       (norm, rope, swiglu, embed, sample)

With --once a case is launched a few times without timing (for ncu).
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from prism_b200 import ops  # noqa: E402

DEV = "cuda:0"
H, I, V, NH, NKV, HD = 3584, 18944, 152064, 28, 4, 128


def timeit(fn, reps=20, flush=True):
    junk = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=DEV) if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(reps):
        if flush:
            junk.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / reps * 1e3     # microseconds


def bench_gemv(args):
    M = args.m
    shapes = [("qkv", 4608, H, ops.EPI_BF16), ("o", H, H, ops.EPI_BF16), ("gate_up+swiglu", I, H, ops.EPI_SWIGLU),
              ("down", H, I, ops.EPI_BF16), ("lm_head", V, H, ops.EPI_F32)]
    for name, N, K, epi in shapes:
        rows = 2 * N if epi == ops.EPI_SWIGLU else N
        w = torch.randn(rows, K, device=DEV, dtype=torch.bfloat16) * 0.02
        x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
        out = torch.empty(M, N, device=DEV, dtype=torch.float32 if epi == ops.EPI_F32 else torch.bfloat16)
        if args.once:
            for _ in range(3):
                ops.gemv(x, w, None, out, epi)
            torch.cuda.synchronize()
            continue
        t = timeit(lambda: ops.gemv(x, w, None, out, epi))
        t_lib = timeit(lambda: torch.mm(x, w.t()))
        gb = rows * K * 2 / 1e9
        print(f"gemv {name:16s} M={M:3d} N={N:6d} K={K:6d}: {t:8.1f} us  {gb / t * 1e6:7.0f} GB/s   "
              f"(library mm: {t_lib:8.1f} us {gb / t_lib * 1e6:7.0f} GB/s)")


def bench_gemm_tc(args):
    M = args.m
    shapes = [("qkv", 4608, H, ops.EPI_BF16, 1), ("qkv split4", 4608, H, ops.EPI_PARTIAL, 4),
              ("o", H, H, ops.EPI_BF16, 1), ("o split5", H, H, ops.EPI_PARTIAL, 5), ("o split10", H, H, ops.EPI_PARTIAL, 10),
              ("gate_up+swiglu", I, H, ops.EPI_SWIGLU, 1), ("gate_up", 2 * I, H, ops.EPI_BF16, 1),
              ("down", H, I, ops.EPI_BF16, 1), ("down split5", H, I, ops.EPI_PARTIAL, 5),
              ("down split10", H, I, ops.EPI_PARTIAL, 10), ("lm_head", V, H, ops.EPI_F32, 1)]
    for name, N, K, epi, ks in shapes:
        rows = 2 * N if epi == ops.EPI_SWIGLU else N
        w = torch.randn(rows, K, device=DEV, dtype=torch.bfloat16) * 0.02
        x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
        if epi == ops.EPI_PARTIAL:
            out = torch.empty(ks, M, N, device=DEV, dtype=torch.float32)
        else:
            out = torch.empty(M, N, device=DEV, dtype=torch.float32 if epi == ops.EPI_F32 else torch.bfloat16)
        fn = lambda: ops.gemm_tc(x, w, None, out, epi, ksplit=ks)
        if args.once:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            continue
        t = timeit(fn)
        t_lib = timeit(lambda: torch.mm(x, w.t()))
        gb = rows * K * 2 / 1e9
        print(f"gemm_tc {name:16s} M={M:3d} N={N:6d} K={K:6d}: {t:8.1f} us  {gb / t * 1e6:7.0f} GB/s   "
              f"(library mm: {t_lib:8.1f} us {gb / t_lib * 1e6:7.0f} GB/s)")


def paged_case(batch, ctx, q_len, page=256):
    pages_per = (ctx + q_len + page - 1) // page
    n_pages = batch * pages_per + 1
    kc = torch.randn(n_pages, page, NKV, HD, device=DEV, dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.arange(batch * pages_per, dtype=torch.int32, device=DEV).view(batch, pages_per)
    T = batch * q_len
    q = torch.randn(T, NH, HD, device=DEV, dtype=torch.bfloat16)
    pos = torch.cat([torch.arange(ctx, ctx + q_len) for _ in range(batch)]).to(torch.int32).to(DEV)
    seg = torch.arange(batch).repeat_interleave(q_len).to(torch.int32).to(DEV)
    seg_start = (torch.arange(batch + 1) * q_len).to(torch.int32).to(DEV)
    cached = torch.full((batch,), ctx, dtype=torch.int32, device=DEV)
    return kc, vc, bt, q, pos, seg, seg_start, cached, n_pages


def bench_attn_decode(args):
    B, ctx = args.batch, args.ctx
    kc, vc, bt, q, pos, seg, _, _, n_pages = paged_case(B, ctx - 1, 1)
    if args.ragged:
        g = torch.Generator().manual_seed(0)
        pos = torch.randint(ctx // 32, ctx, (B,), generator=g).to(torch.int32).to(DEV)
        pos[0] = ctx - 1
    out = torch.empty(B, NH * HD, device=DEV, dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    if args.splits or args.bound:
        # equal splits for every request, as a caller without work items gets them
        ns = args.splits or ops.decode_splits(B, NKV, args.bound or ctx, None)
        po = torch.empty(B, NH, ns, HD, device=DEV)
        pml = torch.empty(B, NH, ns, 2, device=DEV)
        fn = lambda: ops.attention_decode_bf16(q, out, kc, vc, bt, pos, seg, n_pages, None, HD ** -0.5, ns, po, pml, err)
    else:
        # the engine's way: work items from the requests' contexts (--ragged: contexts from ctx/32 to ctx)
        items, starts, ns = ops.decode_work_items(pos.tolist(), NKV, None)
        items, starts = torch.from_numpy(items).to(DEV), torch.from_numpy(starts).to(DEV)
        po = torch.empty(items.shape[0], NH, HD, device=DEV)
        pml = torch.empty(items.shape[0], NH, 2, device=DEV)
        fn = lambda: ops.attention_decode_bf16(q, out, kc, vc, bt, pos, seg, n_pages, None, HD ** -0.5, ns, po, pml, err,
                                               items=items, starts=starts)
    if args.once:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        return
    t = timeit(fn)
    gb = int(pos.sum() + B) * NKV * HD * 2 * 2 / 1e9
    print(f"attn_decode B={B} ctx={'<=' if args.ragged else ''}{ctx} splits<={ns}: {t:8.1f} us  {gb / t * 1e6:7.0f} GB/s of K/V")


def bench_attn_prefill(args):
    Tn = args.tokens
    kc, vc, bt, q, pos, seg, seg_start, cached, n_pages = paged_case(1, args.cached, Tn)
    out = torch.empty(Tn, NH * HD, device=DEV, dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    if args.mma_sync:
        fn = lambda: ops.attention_prefill_bf16(q, out, kc, vc, bt, seg_start, cached, Tn, n_pages, None, HD ** -0.5, err)
    else:
        ns = args.splits or ops.prefill_splits(1, Tn, NH, args.cached + Tn, None)     # as the engine chooses
        fn = lambda: ops.attention_prefill_tc(q, out, kc, vc, bt, seg_start, cached, Tn, n_pages, None, HD ** -0.5, err,
                                              nsplit=ns)
    if args.once:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        return
    t = timeit(fn)
    fl = 4 * NH * HD * (Tn * (Tn + 1) / 2 + Tn * args.cached)
    print(f"attn_prefill ({'mma.sync' if args.mma_sync else f'tcgen05, {ns} split(s)'}) T={Tn} cached={args.cached}: {t:8.1f} us  {fl / t / 1e6:7.1f} TFLOP/s (causal flops)")


def bench_small(args):
    M = args.m
    res = torch.randn(M, H, device=DEV)
    delta = torch.randn(M, H, device=DEV, dtype=torch.bfloat16)
    w = torch.ones(H, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(M, H, device=DEV, dtype=torch.bfloat16)
    print(f"add_rmsnorm M={M}: {timeit(lambda: ops.add_rmsnorm(res, delta, w, 1e-6, out)):8.1f} us")
    gu = torch.randn(M, 2 * I, device=DEV, dtype=torch.bfloat16)
    act = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    print(f"swiglu M={M}: {timeit(lambda: ops.swiglu(gu, act)):8.1f} us")
    logits = torch.randn(M, V, device=DEV)
    tok = torch.empty(M, dtype=torch.int32, device=DEV)
    print(f"sample(argmax) M={M}: {timeit(lambda: ops.sample(logits, None, None, tok)):8.1f} us")
    kc, vc, bt, q, pos, seg, _, _, n_pages = paged_case(M, 2047, 1)
    qkv = torch.randn(M, (NH + 2 * NKV) * HD, device=DEV, dtype=torch.bfloat16)
    qq, kk, vv = qkv[:, :NH * HD].view(M, NH, HD), qkv[:, NH * HD:(NH + NKV) * HD].view(M, NKV, HD), \
        qkv[:, (NH + NKV) * HD:].view(M, NKV, HD)
    inv = (1.0 / (1e6 ** (torch.arange(0, HD, 2, dtype=torch.float32) / HD))).to(DEV)
    table = torch.empty(M, HD // 2, 2, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rope_table(pos, inv, table)
    print(f"rope_kv_write M={M}: "
          f"{timeit(lambda: ops.rope_kv_write(qq, kk, vv, pos, seg, inv, HD, kc, vc, bt, n_pages, 1 << 20, err, table=table)):8.1f} us")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv", "gemm_tc", "attn_decode", "attn_prefill", "small"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--bound", type=int, default=0, help="context bound used to choose the splits")
    ap.add_argument("--splits", type=int, default=0, help="attn_decode: CTAs per (token, kv head); attn_prefill: CTAs that share a query tile's keys; 0 = the engine's choice")
    ap.add_argument("--ragged", action="store_true", help="attn_decode: contexts drawn from ctx/32 .. ctx, one of them ctx")
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--cached", type=int, default=0, help="attn_prefill: tokens already in the cache before the portion")
    ap.add_argument("--mma-sync", action="store_true", help="attn_prefill: the mma.sync kernel instead of the tcgen05 one")
    ap.add_argument("--once", action="store_true")
    a = ap.parse_args()
    {"gemv": bench_gemv, "gemm_tc": bench_gemm_tc, "attn_decode": bench_attn_decode, "attn_prefill": bench_attn_prefill,
     "small": bench_small}[a.what](a)
