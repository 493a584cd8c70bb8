"""The allocation-free column sum (csrc/abi/no_alloc.h), called through its exported C symbol.

Some callers cannot allocate GPU memory while they work: code inside a CUDA-graph capture, a
callback that must stay off the allocator's locks, or an FFI host with no allocator to lend a
workspace.  For them the library keeps a fixed 4 MiB scratch array of its own.  This test
calls the symbol with ctypes on buffers it allocated beforehand, twice in a row (the second
call reuses the scratch the first one dirtied), and compares with the regular, allocating
column-sum entry point."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "luatorch_b200",
                   "lib", "libluatorch.so")


def _lib():
    assert os.path.exists(LIB), "libluatorch.so is not built: run python -m luatorch_b200.build"
    lib = ctypes.CDLL(LIB)
    lib.lt_column_sum_f32_noalloc.restype = ctypes.c_int
    lib.lt_column_sum_f32_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                              ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    lib.lt_column_sum_noalloc_scratch_floats.restype = ctypes.c_int64
    lib.lt_column_sum_noalloc_scratch_floats.argtypes = [ctypes.c_int64, ctypes.c_int64]
    return lib


def test_no_alloc_column_sum_matches_allocating_entry_point():
    from luatorch_b200 import _C
    lib = _lib()
    torch.cuda.init()
    gen = torch.Generator().manual_seed(77)
    stream = torch.cuda.current_stream().cuda_stream
    for rows, cols in [(1000, 300), (4097, 72)]:
        x = torch.randn(rows, cols, generator=gen).cuda()
        out = torch.full((cols,), 123.0, device="cuda")
        ref = _C.column_sum(x, None, False)
        for _ in range(2):                      # second call sees the first call's scratch
            out.fill_(123.0)
            rc = lib.lt_column_sum_f32_noalloc(x.data_ptr(), rows, cols, cols, out.data_ptr(), stream)
            assert rc == 0
            torch.cuda.synchronize()
            torch.testing.assert_close(out, ref, atol=1e-4, rtol=1e-5)
            torch.testing.assert_close(out, x.sum(0), atol=1e-3, rtol=1e-4)
    # strided input (ld > cols)
    wide = torch.randn(500, 128, generator=gen).cuda()
    out = torch.empty(100, device="cuda")
    assert lib.lt_column_sum_f32_noalloc(wide.data_ptr(), 500, 100, 128, out.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    torch.testing.assert_close(out, wide[:, :100].sum(0), atol=1e-3, rtol=1e-4)


def test_no_alloc_column_sum_rejects_oversized_and_bad_arguments():
    lib = _lib()
    rows, cols = 1 << 20, 4096                  # needs 8192 * 4096 floats of scratch: too many
    assert lib.lt_column_sum_noalloc_scratch_floats(rows, cols) > (1 << 20)
    dummy = torch.zeros(8, device="cuda")
    assert lib.lt_column_sum_f32_noalloc(dummy.data_ptr(), rows, cols, cols, dummy.data_ptr(), None) == 2
    # more 128-row slabs than a launch grid can hold: refused as too large, not a launch error
    assert lib.lt_column_sum_f32_noalloc(dummy.data_ptr(), 128 * 65536, 1, 1, dummy.data_ptr(), None) == 2
    # no rows: zeros, whatever the column count, and no scratch is touched
    out = torch.full((3000,), 5.0, device="cuda")
    assert lib.lt_column_sum_f32_noalloc(dummy.data_ptr(), 0, 3000, 3000, out.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert torch.all(out == 0)
    assert lib.lt_column_sum_f32_noalloc(None, 4, 2, 2, dummy.data_ptr(), None) == 1
    assert lib.lt_column_sum_f32_noalloc(dummy.data_ptr(), 4, 2, 1, dummy.data_ptr(), None) == 1
