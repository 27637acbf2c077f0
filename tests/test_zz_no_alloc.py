"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of the kernel library cannot call cudaMalloc (they run inside a fixed memory budget,
or at a moment when an allocation's implicit synchronisation is not allowed), so they cannot hand
the split-key attention the scratch buffer it needs.  ``hfee_attention_decode_noalloc`` keeps that
scratch in a fixed array inside the library.  This test calls it directly with ctypes, twice in a
row on different inputs (the array keeps the first call's content; the second result must not
care), and compares each output with the regular entry point's, which gets scratch from the
caller.  It is collected last so that a run stopping at the first failure has run everything else.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
SCRATCH_FLOATS = 1 << 20        # HFEE_NOALLOC_SCRATCH_FLOATS in csrc/no_alloc.h


def _symbol():
    from hfee_b200.kernels import build
    lib = ctypes.CDLL(build.build())
    fn = lib.hfee_attention_decode_noalloc
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, I, P, P, P, I, I, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P]
    fn.restype = I
    lib.hfee_last_error.restype = ctypes.c_char_p
    return lib, fn


def _call(fn, b, out, heads, kv, hd, page, splits):
    return fn(b.q.data_ptr(), b.q.stride(0), b.kp.data_ptr(), b.vp.data_ptr(), b.table.data_ptr(),
              b.table.shape[1], page, b.cu_tokens.data_ptr(), b.slots.data_ptr(), b.context_before.data_ptr(),
              out.data_ptr(), out.stride(0), b.n, b.r, 1, heads, kv, hd, 1 / math.sqrt(hd), 0, splits,
              torch.cuda.current_stream().cuda_stream)


def test_no_alloc_entry_point_matches_regular_one_twice():
    from hfee_b200.kernels import ops
    from test_gpu_attention import Batch, _err
    lib, fn = _symbol()
    heads, kv, hd, page = 8, 2, 64, 16
    for call, (before, splits, seed) in enumerate([([0, 63, 64, 700, 255], 6, 11), ([1499, 5, 300], 9, 12)]):
        b = Batch(torch.bfloat16, heads, kv, hd, page, before, [1] * len(before), seed=seed)
        scale = 1 / math.sqrt(hd)
        want = torch.full_like(b.q, float("nan"))
        scratch = torch.empty(b.n * heads * splits * (hd + 2), dtype=torch.float32, device=DEV)
        ops.attention_mma(b.q, b.kp, b.vp, b.table, page, b.cu_tokens, b.slots, b.context_before, want, b.n, b.r, 1,
                          heads, kv, hd, scale, 0, splits, scratch)
        got = torch.full_like(b.q, float("nan"))
        if call == 0:                               # the first call on a device looks the array's address up
            assert _call(fn, b, got, heads, kv, hd, page, splits) == 0, lib.hfee_last_error().decode()
            got.fill_(float("nan"))
        torch.cuda.synchronize()
        # what the driver itself reports as free: an allocation inside the library, by whatever
        # route, would show here (torch's own counters only see torch's allocator)
        taken = []
        for _ in range(3):          # a memory-taking call would take some every time; another tenant of the GPU would not
            free_before, _ = torch.cuda.mem_get_info()
            rc = _call(fn, b, got, heads, kv, hd, page, splits)
            assert rc == 0, lib.hfee_last_error().decode()
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
            taken.append(free_before - free_after)
        assert min(taken) <= 0, f"call {call}: device memory was taken by every call: {taken} bytes"
        assert not torch.isnan(got.float()).any(), f"call {call}: output not fully written"
        # the same kernels ran on the same inputs in the same order: the same bits
        assert torch.equal(got, want), f"call {call}"
        assert _err(got, b.reference(scale)) < 1e-2, f"call {call}"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from test_gpu_attention import Batch
    lib, fn = _symbol()
    heads, kv, hd, page = 32, 8, 128, 16
    b = Batch(torch.bfloat16, heads, kv, hd, page, [10] * 9, [1] * 9, seed=1)
    out = torch.zeros_like(b.q)
    splits = 32                                   # 9 * 32 * 32 * 130 floats > 2^20
    assert b.n * heads * splits * (hd + 2) > SCRATCH_FLOATS
    rc = _call(fn, b, out, heads, kv, hd, page, splits)
    assert rc != 0
    assert "exceed the built-in scratch" in lib.hfee_last_error().decode()
    assert float(out.float().abs().max()) == 0.0          # nothing was launched
