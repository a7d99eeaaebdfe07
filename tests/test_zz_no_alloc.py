"""The allocation-free decode-attention entry point, called through its
exported C symbol.

Some users of this library cannot allocate device memory when they need
attention (another component owns the memory budget, or they run where the
driver's allocator must not be entered), so they cannot hand the split-KV
kernel its scratch buffers.  ``prism_attention_decode_bf16_noalloc`` keeps
that scratch in a fixed array inside the library.  This test checks that it
gives what the ordinary entry point gives, twice in a row with different
shapes (the array keeps the first call's contents), and that it refuses a call
that would not fit.  The file is named so that pytest collects it last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _symbol():
    from prism_b200.csrc import build
    lib = ctypes.CDLL(build.build(verbose=False))            # the shared library itself, not the Python wrappers
    fn = lib.prism_attention_decode_bf16_noalloc
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.restype = i
    fn.argtypes = [p, i, p, i, p, p, p, i, p, p, i, i, i, i, i, i, i, f, i, p, p]
    lib.prism_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _call(fn, c, out, nh, nkv, hd, window, scale, nsplit, err):
    return fn(c.q.data_ptr(), c.q.stride(0), out.data_ptr(), out.stride(0), c.k.data_ptr(), c.v.data_ptr(),
              c.bt.data_ptr(), c.bt.shape[1], c.positions.data_ptr(), c.tok_seg.data_ptr(), c.T, nh, nkv, hd,
              c.k.shape[1], c.num_pages, int(window or 0), scale, nsplit, err.data_ptr(),
              torch.cuda.current_stream().cuda_stream)


def test_no_alloc_entry_point_matches_the_allocating_one():
    from prism_b200 import ops
    from test_kernels_gpu import PagedCase, ref_paged_attention
    lib, fn = _symbol()
    cases = [  # nh, nkv, hd, page, window, contexts, nsplit
        (28, 4, 128, 64, None, [700, 64, 1, 2049], 9),
        (8, 2, 64, 16, 40, [300, 5], 3),
    ]
    for nh, nkv, hd, P, window, ctxs, nsplit in cases:       # two calls in a row on the shared array
        c = PagedCase([(n, 1) for n in ctxs], nh, nkv, hd, P, torch.bfloat16, seed=77)
        scale = hd ** -0.5
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        want = torch.empty(c.T, nh * hd, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode_bf16(c.q, want, c.k, c.v, c.bt, c.positions, c.tok_seg, c.num_pages, window, scale,
                                  nsplit, torch.empty(c.T, nh, nsplit, hd, device=DEV),
                                  torch.empty(c.T, nh, nsplit, 2, device=DEV), err)
        got = torch.full_like(want, float("nan"))
        # the first call on a device looks up the array's address (and the driver may load the kernel then);
        # the claim is about the calls after it
        rc = _call(fn, c, got, nh, nkv, hd, window, scale, nsplit, err)
        torch.cuda.synchronize()
        assert rc == 0, lib.prism_noalloc_last_error()
        got.fill_(float("nan"))
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]           # the driver's own count: sees a cudaMalloc that torch's cannot
        rc = _call(fn, c, got, nh, nkv, hd, window, scale, nsplit, err)
        torch.cuda.synchronize()
        assert rc == 0, lib.prism_noalloc_last_error()
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated or freed inside the call"
        assert torch.cuda.memory_allocated() == before and int(err) == 0
        ref = ref_paged_attention(c.q, c.k, c.v, c.bt, c.positions, c.tok_seg, window, scale)
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.allclose(got.float(), ref, atol=2e-2, rtol=2e-2)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from test_kernels_gpu import PagedCase
    lib, fn = _symbol()
    nh, nkv, hd = 28, 4, 128
    c = PagedCase([(10, 1)] * 40, nh, nkv, hd, 16, torch.bfloat16, seed=1)
    out = torch.zeros(c.T, nh * hd, dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = _call(fn, c, out, nh, nkv, hd, None, 1.0, 64, err)           # 40*28*64*130 floats > 4 MiB
    assert rc == 1 and b"scratch" in lib.prism_noalloc_last_error()
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0                              # nothing ran
    rc = _call(fn, c, out, nh, nkv, 96, None, 1.0, 1, err)
    assert rc == 1 and b"head_dim" in lib.prism_noalloc_last_error()
