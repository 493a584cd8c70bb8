"""In-tree native build: compiles every CUDA source for sm_100a with nvcc and links

  luatorch_b200/_C.so            PyTorch-facing binding of the kernels
  luatorch_b200/lib/libluatorch.so   the C ABI library the LuaJIT FFI front end binds
                                 (same symbol list as the reference's library,
                                 lua/luatorch/tensor.lua:33-178)

Objects live under build/ (ignored by git); the shared objects are written next to the Python
package so a snapshot of the tree carries them.  Incremental: a source is recompiled when it
or any header is newer than its object.  `python -m luatorch_b200.build [--force] [--verbose]`.

The reference builds one library with CMake for sm_75..90 only (CMakeLists.txt:9-20).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"
PKG = ROOT / "luatorch_b200"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177",
]

KERNEL_SOURCES = [
    "kernels/gemm_tcgen05.cu", "kernels/elementwise.cu", "kernels/reduce.cu",
    "kernels/softmax_ce.cu", "kernels/layernorm.cu", "kernels/embedding.cu", "kernels/conv.cu",
    "kernels/optim.cu", "kernels/attention_fwd.cu", "kernels/attention_bwd.cu",
    "comm/comm_kernels.cu",
]
ABI_SOURCES = [
    "abi/tensor_core.cpp", "abi/cpu_ops.cpp", "abi/cuda_ops.cu", "abi/memory_pool.cpp",
    "abi/nccl_shim.cpp", "abi/no_alloc.cu",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _headers_mtime() -> float:
    newest = 0.0
    for pat in ("*.h", "*.cuh", "*.hpp"):
        for p in CSRC.rglob(pat):
            newest = max(newest, p.stat().st_mtime)
    return newest


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build command failed:\n%s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr)


def _stale(src: Path, obj: Path, hdr_mtime: float, force: bool) -> bool:
    if force or not obj.exists():
        return True
    t = obj.stat().st_mtime
    return src.stat().st_mtime > t or hdr_mtime > t


def _compile_cu(src: Path, obj: Path, verbose: bool, extra=()):
    obj.parent.mkdir(parents=True, exist_ok=True)
    _run([_nvcc(), *NVCC_FLAGS, *extra, "-I", CSRC, "-c", src, "-o", obj], verbose)


def _compile_cpp(src: Path, obj: Path, verbose: bool, extra=()):
    obj.parent.mkdir(parents=True, exist_ok=True)
    _run(["g++", "-O2", "-std=c++17", "-fPIC", "-I", CSRC, "-I", "/usr/local/cuda/include", *extra,
          "-c", src, "-o", obj], verbose)


def build_all(force: bool = False, verbose: bool = False, abi: bool = True) -> None:
    hdr = _headers_mtime()
    jobs = []
    kernel_objs = []
    for rel in KERNEL_SOURCES:
        src = CSRC / rel
        obj = BUILD / (rel.replace("/", "_") + ".o")
        kernel_objs.append(obj)
        if _stale(src, obj, hdr, force):
            jobs.append((_compile_cu, (src, obj, verbose)))

    # ---- torch binding
    import torch  # noqa: F401  (import cost is paid once; needed for include / library paths)
    from torch.utils import cpp_extension as ce
    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    import sysconfig
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    bind_src = CSRC / "binding" / "torch_binding.cpp"
    bind_obj = BUILD / "binding_torch_binding.o"
    if _stale(bind_src, bind_obj, hdr, force):
        jobs.append((_compile_cpp, (bind_src, bind_obj, verbose,
                                    ["-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                                     "-D_GLIBCXX_USE_CXX11_ABI=1", *inc])))

    abi_objs = []
    if abi:
        for rel in ABI_SOURCES:
            src = CSRC / rel
            if not src.exists():
                continue
            obj = BUILD / (rel.replace("/", "_") + ".o")
            abi_objs.append(obj)
            if _stale(src, obj, hdr, force):
                fn = _compile_cu if src.suffix == ".cu" else _compile_cpp
                jobs.append((fn, (src, obj, verbose)))

    if jobs:
        workers = max(1, min(len(jobs), os.cpu_count() or 4))
        with ThreadPoolExecutor(workers) as ex:
            futs = [ex.submit(fn, *args) for fn, args in jobs]
            for f in futs:
                f.result()

    # ---- link _C.so
    out = PKG / "_C.so"
    deps = kernel_objs + [bind_obj]
    if force or jobs or not out.exists() or any(o.stat().st_mtime > out.stat().st_mtime for o in deps):
        libdirs = []
        for p in ce.library_paths(device_type="cuda"):
            libdirs += ["-L", p, "-Wl,-rpath," + p]
        _run(["g++", "-shared", "-o", out, *deps, *libdirs, "-lc10", "-lc10_cuda", "-ltorch_cpu",
              "-ltorch_cuda", "-ltorch", "-ltorch_python", "-L", "/usr/local/cuda/lib64",
              "-lcudart"], verbose)

    # ---- link libluatorch.so (no PyTorch dependency)
    if abi and abi_objs:
        lib = PKG / "lib" / "libluatorch.so"
        lib.parent.mkdir(parents=True, exist_ok=True)
        deps = kernel_objs + abi_objs
        if force or jobs or not lib.exists() or any(o.stat().st_mtime > lib.stat().st_mtime for o in deps):
            _run(["g++", "-shared", "-o", lib, *deps, "-L", "/usr/local/cuda/lib64",
                  "-Wl,-rpath,/usr/local/cuda/lib64", "-lcudart", "-lpthread", "-ldl", "-lm"], verbose)


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    build_all(force="--force" in argv, verbose="--verbose" in argv)
    print("built", PKG / "_C.so")


if __name__ == "__main__":
    main()
