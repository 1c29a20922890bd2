"""The allocation-free decode-attention entry point.

Some users of the kernel library may not allocate device memory (their memory is
a fixed arena owned by another runtime, or their allocator is frozen), so they
cannot hand the split-KV kernel its temporary buffer.  For them the library
exports ``us_paged_decode_attention_noalloc``, which keeps that buffer in an
array built into the library.  This test calls it through its exported C symbol
and checks it against the regular entry point, twice in a row with different
inputs, because the built-in buffer keeps the previous call's contents.

The file sorts last on purpose: if it fails, a run that stops at the first
failure has already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

VP, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _lib():
    from uniserve_v1_b200.ops import native
    lib = native.kernels()
    fn = lib.us_paged_decode_attention_noalloc
    fn.restype = I
    fn.argtypes = [VP, VP, VP, VP, VP, VP, I, I, I, I, I, I, I, I, F, LL, LL, VP]
    ref = lib.us_paged_decode_attention
    ref.restype = I
    ref.argtypes = [VP, VP, VP, VP, VP, VP, VP, I, I, I, I, I, I, I, I, F, LL, LL, VP]
    return lib, fn, ref


def _case(seed, B, Hq, Hkv, D, page, pages, lens):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g, device="cuda").to(torch.bfloat16)
    q = mk(B, Hq, D)
    kc, vc = mk(pages, page, Hkv, D), mk(pages, page, Hkv, D)
    per = (max(lens) + page - 1) // page
    pt = (torch.randperm(pages - 1, generator=g, device="cuda")[:B * per].view(B, per) + 1).to(torch.int32)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    return q, kc, vc, pt, sl


def _run(fn, ref, q, kc, vc, pt, sl, splits):
    B, Hq, D = q.shape
    pages, page, Hkv, _ = kc.shape
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = 1.0 / math.sqrt(D)
    out_a = torch.empty_like(q)
    out_b = torch.empty_like(q)
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pt.data_ptr(), sl.data_ptr(),
            out_a.data_ptr(), B, Hq, Hkv, D, pt.shape[1], page, splits, 0, scale, q.stride(0),
            out_a.stride(0), st)
    assert rc == 0
    scratch = torch.empty(B * Hq * splits * (D + 1) * 4, dtype=torch.uint8, device="cuda")
    rc = ref(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pt.data_ptr(), sl.data_ptr(),
             out_b.data_ptr(), scratch.data_ptr(), B, Hq, Hkv, D, pt.shape[1], page, splits, 0,
             scale, q.stride(0), out_b.stride(0), st)
    assert rc == 0
    torch.cuda.synchronize()
    return out_a, out_b


def test_noalloc_matches_regular_entry_point_twice():
    lib, fn, ref = _lib()
    # first call: also performs the one-time symbol look-up on this device
    a, b = _run(fn, ref, *_case(1, 6, 32, 4, 128, 16, 260, [1, 40, 300, 129, 512, 77]), splits=4)
    torch.testing.assert_close(a.float(), b.float(), atol=2e-2, rtol=2e-2)
    # second call, other shapes and data: the built-in buffer still holds call one's partials
    a, b = _run(fn, ref, *_case(2, 3, 8, 2, 64, 16, 80, [200, 5, 333]), splits=3)
    torch.testing.assert_close(a.float(), b.float(), atol=2e-2, rtol=2e-2)
    # the result is also right in absolute terms
    from uniserve_v1_b200.ops import reference as R
    q, kc, vc, pt, sl = _case(2, 3, 8, 2, 64, 16, 80, [200, 5, 333])
    want = R.paged_decode_attention(q, kc, vc, pt, sl, 1.0 / math.sqrt(64))
    torch.testing.assert_close(a.float(), want.float(), atol=2e-2, rtol=2e-2)


def test_noalloc_rejects_oversized_request():
    lib, fn, _ = _lib()
    q, kc, vc, pt, sl = _case(3, 2, 8, 2, 64, 16, 32, [10, 20])
    out = torch.empty_like(q)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # claim a batch whose partials cannot fit in the built-in buffer; the check
    # fires before anything is launched
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pt.data_ptr(), sl.data_ptr(),
            out.data_ptr(), 4096, 64, 2, 128, pt.shape[1], 16, 32, 0, 0.1, q.stride(0),
            out.stride(0), st)
    assert rc == 5
    lib.us_last_error.restype = ctypes.c_char_p
    assert b"exceeds the built-in scratch" in lib.us_last_error()
