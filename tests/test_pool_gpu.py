"""The caching device-memory pool behind the pool_* ABI (csrc/abi/memory_pool.cpp), through
ctypes in a process of its own so its counters start from zero.  Semantics follow the
reference's pool (csrc/cuda/memory_pool.cu:32-176): 512-byte minimum and power-of-two size
classes, reuse of a cached block at most twice the request, pool_clear returns the cache to
the driver, the two byte counters; plus this pool's additions: stream-ordered release,
per-device free lists and the debug canaries that report a write past the end of a block."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PRELUDE = """
import ctypes as C, os, sys
sys.path.insert(0, %r)
import torch
L = C.CDLL(os.path.join(%r, "luatorch_b200", "lib", "libluatorch.so"))
L.pool_alloc.restype = C.c_void_p; L.pool_alloc.argtypes = [C.c_size_t]
L.pool_free.argtypes = [C.c_void_p]
L.pool_free_async.argtypes = [C.c_void_p, C.c_void_p]
for n in ("pool_allocated_bytes", "pool_cached_bytes", "cuda_memory_allocated", "cuda_memory_cached", "pool_overruns_seen"):
    getattr(L, n).restype = C.c_size_t
L.pool_check_canaries.restype = C.c_int
torch.cuda.init(); torch.zeros(1, device="cuda")
L.pool_init()
MiB = 1 << 20
""" % (ROOT, ROOT)


def _run(body):
    r = subprocess.run([sys.executable, "-c", PRELUDE + textwrap.dedent(body)], capture_output=True,
                       text=True, timeout=180)
    assert r.returncode == 0 and "CASE_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])
    return r


def test_counters_size_classes_reuse_and_clear():
    _run("""
    assert L.pool_allocated_bytes() == 0 and L.pool_cached_bytes() == 0
    a = L.pool_alloc(100)                       # 512-byte minimum
    assert a and L.pool_allocated_bytes() == 512 and L.pool_cached_bytes() == 0
    b = L.pool_alloc(5000)                      # next power of two
    assert L.pool_allocated_bytes() == 512 + 8192
    L.pool_free(b)
    assert L.pool_cached_bytes() == 8192 and L.pool_allocated_bytes() == 512 + 8192
    assert L.cuda_memory_allocated() == L.pool_allocated_bytes() and L.cuda_memory_cached() == 8192
    c = L.pool_alloc(8000)                      # same class: the cached block comes back
    assert c == b and L.pool_cached_bytes() == 0 and L.pool_allocated_bytes() == 512 + 8192
    L.pool_free(c)
    d = L.pool_alloc(4096)                      # 8192 <= 2 x 4096: reused
    assert d == b
    L.pool_free(d)
    e = L.pool_alloc(2048)                      # 8192 > 2 x 2048: a new block
    assert e != b and L.pool_allocated_bytes() == 512 + 8192 + 2048
    big = L.pool_alloc(3 * MiB)                 # above 1 MiB: rounded to 2 MiB multiples
    assert L.pool_allocated_bytes() == 512 + 8192 + 2048 + 4 * MiB
    L.pool_free(big)
    again = L.pool_alloc(4 * MiB)
    assert again == big
    L.pool_free(again)
    small = L.pool_alloc(1 * MiB)               # 4 MiB > 2 x 1 MiB: not served from the big block
    assert small != big
    for p in (a, e, small): L.pool_free(p)
    cached = L.pool_cached_bytes()
    assert cached == L.pool_allocated_bytes() > 0
    L.pool_clear()                              # everything cached goes back to the driver
    assert L.pool_cached_bytes() == 0 and L.pool_allocated_bytes() == 0
    # a pointer the pool does not know is handed to cudaFree, as in the reference (no crash)
    print("CASE_OK")
    """)


def test_stream_ordered_release_is_not_reused_before_its_event():
    _run("""
    side = torch.cuda.Stream()
    p = L.pool_alloc(4 * MiB)
    x = torch.randn(8192, 8192, device="cuda")
    with torch.cuda.stream(side):
        for _ in range(30):                      # tens of milliseconds of work on the side stream
            x = (x @ x).clamp_(-1, 1)
    L.pool_free_async(p, C.c_void_p(side.cuda_stream))
    assert L.pool_cached_bytes() == 4 * MiB
    q = L.pool_alloc(4 * MiB)                    # the side stream may still use p: not handed out
    assert q != p
    side.synchronize()
    r = L.pool_alloc(4 * MiB)                    # the event has completed: p is reusable
    assert r == p
    L.pool_free(q); L.pool_free(r); L.pool_clear()
    assert L.pool_allocated_bytes() == 0
    print("CASE_OK")
    """)


def test_debug_canaries_report_a_write_past_the_end():
    _run("""
    L.pool_set_debug(1)
    p = L.pool_alloc(1000)
    q = L.pool_alloc(1000)
    assert L.pool_check_canaries() == 0
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemset.argtypes = [C.c_void_p, C.c_int, C.c_size_t]
    # 8 bytes past the end of q: still inside the pool's own block (the canary), so nothing
    # faults, and exactly what a kernel with an off-by-a-few index would do
    assert rt.cudaMemset(C.c_void_p(q + 1000), 0, 8) == 0
    assert L.pool_check_canaries() == 1
    L.pool_free(p)
    assert L.pool_overruns_seen() == 0
    L.pool_free(q)
    assert L.pool_overruns_seen() == 1
    L.pool_set_debug(0)
    L.pool_clear()
    print("CASE_OK")
    """)


def test_free_lists_are_per_device():
    _run("""
    if torch.cuda.device_count() < 2:
        print("CASE_OK (one device)"); raise SystemExit(0)
    rt = C.CDLL("libcudart.so.12")
    rt.cudaSetDevice(0)
    a = L.pool_alloc(64 * 1024)
    L.pool_free(a)
    rt.cudaSetDevice(1)
    b = L.pool_alloc(64 * 1024)                  # the reference would hand out device 0's block here
    assert b != a
    attr = torch.cuda.current_device()
    L.pool_free(b)
    rt.cudaSetDevice(0)
    c = L.pool_alloc(64 * 1024)
    assert c == a
    L.pool_free(c); L.pool_clear()
    assert L.pool_allocated_bytes() == 0
    print("CASE_OK")
    """)
