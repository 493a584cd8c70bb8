"""Debug mode: the checks a memory sanitizer would make, done by the framework itself.

`compute-sanitizer` cannot run everywhere, so the kernels never trap on bad input: an
out-of-range token id or label, or a wait that ran out, is recorded in a device status word
({flag, position, offending value}) and the kernel carries on with a safe value.  Normally
nobody reads those words on the hot path (that would cost a host synchronisation per call).
`enable()` turns that reading on:

  * after every embedding lookup and cross-entropy call the status word is read back and an
    IndexError names the first offending position and value;
  * after every tensor-core GEMM / attention call the kernels' error words (expired barrier
    waits, misaligned shared memory) are read and raised as RuntimeError;
  * the C ABI's memory pool pads every block with a 256-byte canary that `pool_free` and
    `pool_check_canaries()` verify (`pool_set_debug`, csrc/abi/memory_pool.cpp).

Slow (a device synchronisation per checked call): for chasing a fault, not for training runs.
LT_DEBUG_CHECKS=1 in the environment enables it at import.  The reference has only bounds
checks in tensor_get / tensor_set (csrc/tensor.c:236-258)."""
from __future__ import annotations

import os

_on = os.environ.get("LT_DEBUG_CHECKS", "0") == "1"
checked = 0        # status words read so far (tests look at this)


def enable(flag: bool = True) -> None:
    global _on
    _on = bool(flag)


def enabled() -> bool:
    return _on


def check_index_word(err, what: str) -> None:
    """`err`: int32[4] device tensor {flag, position, value, -}.  Raises IndexError in debug mode."""
    global checked
    if not _on or err is None:
        return
    checked += 1
    rec = err.tolist()
    if rec[0]:
        raise IndexError("%s: position %d holds %d, outside the valid range" % (what, rec[1], rec[2]))


def check_kernels(ext) -> None:
    """Raise if a tensor-core kernel recorded an error (expired wait, bad alignment)."""
    global checked
    if not _on:
        return
    checked += 1
    g, a = int(ext.gemm_device_error()), int(ext.attention_device_error())
    if g or a:
        raise RuntimeError("luatorch_b200 kernel error word: gemm=%d attention=%d" % (g, a))
