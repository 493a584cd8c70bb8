// Allocation-free column sum (declaration and contract in no_alloc.h).
#include "no_alloc.h"

#include <cuda_runtime.h>
#include <stdio.h>
#include <mutex>

#include "../kernels/ops.h"

namespace {

// The scratch lives in the library image: one copy per GPU that loads it, held until exit.
static __device__ __align__(256) float g_noalloc_scratch[LT_NOALLOC_MAX_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device pointer;
// the real address is looked up once per device and cached here.
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;   // two host threads may make a device's first call together

int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fprintf(stderr, "luatorch error: no_alloc column sum: cannot identify the current device (%s)\n",
            cudaGetErrorString(e));
    return LT_NOALLOC_CUDA_ERROR;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "luatorch error: no_alloc column sum: cudaGetSymbolAddress failed (%s)\n",
              cudaGetErrorString(e));
      return LT_NOALLOC_CUDA_ERROR;
    }
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_addr[dev];
  return LT_NOALLOC_OK;
}

}  // namespace

extern "C" int64_t lt_column_sum_noalloc_scratch_floats(int64_t rows, int64_t cols) {
  return lt::column_sum_scratch_floats(rows, cols);
}

extern "C" int lt_column_sum_f32_noalloc(const float* in, int64_t rows, int64_t cols, int64_t ld,
                                         float* out, void* stream) {
  if (in == nullptr || out == nullptr || rows < 0 || cols <= 0 || ld < cols) {
    fprintf(stderr, "luatorch error: no_alloc column sum: bad argument\n");
    return LT_NOALLOC_BAD_ARGUMENT;
  }
  if (rows == 0) {
    // the sum over no rows is zero; nothing touches the scratch (cudaMemsetAsync allocates nothing)
    const cudaError_t e = cudaMemsetAsync(out, 0, sizeof(float) * (size_t)cols,
                                          static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LT_NOALLOC_OK : LT_NOALLOC_CUDA_ERROR;
  }
  const int64_t need = lt::column_sum_scratch_floats(rows, cols);
  // 65535 is the largest grid.y: the two-stage path launches one block row per 128 input rows
  if (need > LT_NOALLOC_MAX_SCRATCH_FLOATS || (rows + 127) / 128 > 65535) {
    fprintf(stderr,
            "luatorch error: no_alloc column sum: [%lld x %lld] needs %lld scratch floats, the "
            "built-in scratch holds %d; use the allocating entry point\n",
            (long long)rows, (long long)cols, (long long)need, LT_NOALLOC_MAX_SCRATCH_FLOATS);
    return LT_NOALLOC_TOO_LARGE;
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != LT_NOALLOC_OK) return rc;
  const cudaError_t e = lt::column_sum(lt::DT_F32, in, ld, out, lt::DT_F32, /*accumulate=*/0, rows,
                                       cols, scratch, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    fprintf(stderr, "luatorch error: no_alloc column sum: launch failed (%s)\n",
            cudaGetErrorString(e));
    return LT_NOALLOC_CUDA_ERROR;
  }
  return LT_NOALLOC_OK;
}
