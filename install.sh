#!/usr/bin/env bash
# Builds luatorch_b200 in place and runs a smoke test.
#   ./install.sh            build + XOR smoke test on the CPU (+ a tiny GPT step if a B200 is visible)
#   ./install.sh --tests    additionally run the CPU test suite
# Nothing is downloaded: python with torch, nvcc (CUDA >= 12.8, sm_100a) and g++ must be present.
# (Counterpart of the reference's tools/install.sh, which checks luajit / cmake / nvcc, builds
# libluatorch with CMake and runs examples/xor.lua.)
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")"

PY=${PYTHON:-python}
fail() { echo "ERROR: $*" >&2; exit 1; }

command -v "$PY" >/dev/null || fail "python not found (set PYTHON=/path/to/python)"
"$PY" - <<'PYEOF' || fail "python >= 3.10 with torch >= 2.6 is required"
import sys
assert sys.version_info >= (3, 10), sys.version
import torch
major, minor = (int(x) for x in torch.__version__.split("+")[0].split(".")[:2])
assert (major, minor) >= (2, 6), torch.__version__
print("found python %d.%d, torch %s" % (sys.version_info[0], sys.version_info[1], torch.__version__))
PYEOF

command -v nvcc >/dev/null || fail "nvcc not found: the kernels are compiled for sm_100a with the CUDA toolkit (>= 12.8)"
NVCC_REL=$(nvcc --version | sed -n 's/.*release \([0-9]*\)\.\([0-9]*\).*/\1 \2/p')
read -r NV_MAJ NV_MIN <<<"$NVCC_REL"
if [ "$NV_MAJ" -lt 12 ] || { [ "$NV_MAJ" -eq 12 ] && [ "$NV_MIN" -lt 8 ]; }; then
  fail "nvcc $NV_MAJ.$NV_MIN cannot target sm_100a (needs >= 12.8)"
fi
echo "found nvcc $NV_MAJ.$NV_MIN"
command -v g++ >/dev/null || fail "g++ not found"

GPU_OK=0
if command -v nvidia-smi >/dev/null; then
  CC=$(nvidia-smi --query-gpu=compute_cap --format=csv,noheader 2>/dev/null | head -1 || true)
  if [ "$CC" = "10.0" ]; then
    GPU_OK=1
    echo "found $(nvidia-smi --query-gpu=name --format=csv,noheader | head -1) (compute capability 10.0)"
  elif [ -n "$CC" ]; then
    echo "note: visible GPU has compute capability $CC; the kernels run on 10.0 (B200) only - CPU paths still work"
  fi
else
  echo "no GPU visible: building anyway (nvcc cross-compiles), CPU paths will be tested"
fi

echo
echo "building (nvcc -gencode arch=compute_100a,code=sm_100a) ..."
"$PY" -m luatorch_b200.build
[ -f luatorch_b200/_C.so ] || fail "build produced no luatorch_b200/_C.so"
[ -f luatorch_b200/lib/libluatorch.so ] || fail "build produced no luatorch_b200/lib/libluatorch.so"

echo
echo "smoke test: XOR on the CPU ..."
"$PY" -m luatorch_b200.train.xor --steps 1500 | tail -6
if [ "$GPU_OK" = 1 ]; then
  echo
  echo "smoke test: one tiny GPT forward + backward on cuda:0 ..."
  "$PY" -c "import __graft_entry__ as g; g.smoke(); print('gpu smoke ok')"
fi
if [ "${1:-}" = "--tests" ]; then
  echo
  "$PY" -m pytest tests -q -m "not gpu"
fi

cat <<'MSG'

luatorch_b200 is built.  Next steps:
  python -m luatorch_b200.train.mlp                     # MLP classifier (add --graph on a GPU)
  python -m luatorch_b200.train.gpt --preset small      # small GPT on synthetic tokens
  python -m luatorch_b200.tools.benchmark               # per-kernel roofline table (B200)
  python bench.py --gpus 1                              # GPT-124M-config training tokens/s
  LuaJIT front end: ffi.load("luatorch_b200/lib/libluatorch.so") exports the reference's C ABI
MSG
