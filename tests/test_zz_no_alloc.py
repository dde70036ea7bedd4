"""The library's entry point that allocates nothing, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory: a host without torch's
allocator, a process that has given all device memory to its own pool, a loop that must
not enter cudaMalloc.  For them the split-KV decode attention exists once more with its
scratch in a fixed device array inside the library (csrc/no_alloc.h).  This test calls
that symbol with raw pointers, twice in a row with different shapes (the array keeps what
the first call left), and compares each result with the ordinary entry point's and with
the float32 reference of the kernel tests, within their bfloat16 tolerance.  It stands in a file of its own that pytest
collects last.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, lens, NH, NKV, D, page, n_splits):
    from acvram_b200.kernels import ops
    lib = ops.library()
    fn = lib.acv_attention_decode_static
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, I, P, I, P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, I, P]
    fn.restype = I

    g = torch.Generator(device="cuda").manual_seed(seed)
    B = len(lens)
    n_pages = sum((l + page - 1) // page for l in lens) + 2
    width = max((l + page - 1) // page for l in lens)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed))
    table = torch.full((B, width), -1, dtype=torch.int32)
    used = 0
    for b, l in enumerate(lens):
        n = (l + page - 1) // page
        table[b, :n] = perm[used:used + n].to(torch.int32)
        used += n
    table = table.cuda()
    kp = (torch.randn(n_pages, NKV, page, D, device="cuda", generator=g)).to(torch.bfloat16)
    vp = (torch.randn(n_pages, NKV, page, D, device="cuda", generator=g)).to(torch.bfloat16)
    q = torch.randn(B, (NH + 2 * NKV) * D, device="cuda", generator=g).to(torch.bfloat16)
    kv_len = torch.tensor(lens, dtype=torch.int32, device="cuda")
    rows = torch.arange(B, dtype=torch.int32, device="cuda")
    scale = D ** -0.5

    want = torch.zeros(B, NH * D, device="cuda", dtype=torch.bfloat16)
    ops.attention_decode(q, want, kp, vp, rows, rows, B, kv_len, table, NH, NKV, D, scale, 0, n_splits, max(lens))

    got = torch.full_like(want, 5.0)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), kp.data_ptr(), vp.data_ptr(), rows.data_ptr(),
            rows.data_ptr(), B, kv_len.data_ptr(), table.data_ptr(), table.stride(0), NH, NKV, D, page, n_pages, scale,
            0, n_splits, max(lens), stream)
    assert rc == 0, f"acv_attention_decode_static returned {rc}"
    torch.cuda.synchronize()
    torch.testing.assert_close(got, want, rtol=1.6e-2, atol=1.6e-2)
    # and against the plain float32 reference, so that a fault shared by both entry points would show too
    import kernel_refs
    plain = torch.zeros_like(want)
    kernel_refs.attention_generic(q, plain, kp, vp, kv_len - 1, rows, table, NH, NKV, D, scale, 0)
    torch.testing.assert_close(got, plain, rtol=1.6e-2, atol=1.6e-2)
    return lib


def test_static_scratch_entry_point_twice_in_a_row():
    lib = _case(1, [700, 64, 333], NH=8, NKV=2, D=128, page=16, n_splits=4)
    _case(2, [90, 1500, 17, 256, 129], NH=6, NKV=2, D=64, page=8, n_splits=3)
    _case(3, [40, 50], NH=4, NKV=4, D=128, page=16, n_splits=1)
    lib.acv_attention_decode_static_capacity.restype = ctypes.c_longlong
    assert lib.acv_attention_decode_static_capacity() == 1 << 20


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from acvram_b200.kernels import ops
    lib = ops.library()
    fn = lib.acv_attention_decode_static
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, I, P, I, P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, I, P]
    fn.restype = I
    z = torch.zeros(16, dtype=torch.int32, device="cuda")
    # 4096 requests x 8 kv-heads x 16 splits x 4 x (128 + 2) floats is far beyond 2^20: refused, nothing launched
    rc = fn(z.data_ptr(), 6144, z.data_ptr(), 4096, z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), 4096,
            z.data_ptr(), z.data_ptr(), 8, 32, 8, 128, 16, 1, 0.1, 0, 16, 4096, torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    torch.cuda.synchronize()
