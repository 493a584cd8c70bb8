// Whole-tensor reductions in ONE launch with the result left on the device: per-thread
// grid-stride accumulation, warp-shuffle + shared-memory block reduction, per-block partial
// to a scratch array, and the last block to finish (atomic ticket) folds the partials in a
// fixed order, so results are bitwise reproducible.
//
// The reference does the same job in two steps with a cudaMalloc + device-to-host copy +
// host loop + cudaFree per call (csrc/cuda/ops/arithmetic.cu:339-448) and uses cublasSdot
// for dot (csrc/cuda/ops/matmul.cu:232-256).  The inf/nan check replaces
// csrc/cuda/ops/cast.cu:67-99 (per-call cudaMalloc + copy) with a device-resident flag and
// fuses the unscale multiply of csrc/cuda/ops/cast.cu:101-115.
#include "ops.h"
#include "common.cuh"

namespace lt {
namespace {

constexpr int THREADS = 256;
constexpr int MAX_PARTIALS = 2048;

struct Scratch {
  float partial[MAX_PARTIALS];
  unsigned int ticket;
};

template <int OP> __device__ __forceinline__ float red_identity() {
  return OP == RED_SUM ? 0.0f : (OP == RED_MAX ? -INFINITY : INFINITY);
}
template <int OP> __device__ __forceinline__ float red_combine(float a, float b) {
  return OP == RED_SUM ? a + b : (OP == RED_MAX ? fmaxf(a, b) : fminf(a, b));
}
template <int OP> __device__ __forceinline__ float red_block(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = red_combine<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = lane < (THREADS / 32) ? sh[lane] : red_identity<OP>();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = red_combine<OP>(r, __shfl_xor_sync(0xffffffffu, r, o));
  return r;
}

// PAIR 0: reduce a;  1: a*b (dot);  2: (a-b)^2 (mse);  3: |a-b| (mae)
template <int PAIR> __device__ __forceinline__ float pair_fn(float x, float y) {
  if (PAIR == 1) return x * y;
  if (PAIR == 2) return (x - y) * (x - y);
  if (PAIR == 3) return fabsf(x - y);
  return x;
}
template <typename T, int OP, int PAIR>
__global__ void __launch_bounds__(THREADS)
reduce_kernel(const T* __restrict__ a, const T* __restrict__ b, int64_t n, float scale,
              float* __restrict__ out, Scratch* scratch, int vec_ok) {
  __shared__ float sh[32];
  __shared__ bool is_last;
  constexpr int V = VecIO<T>::N;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  float acc = red_identity<OP>();
  int64_t done = 0;
  if (vec_ok) {
    const int64_t nvec = n / V;
    for (int64_t i = tid; i < nvec; i += nthreads) {
      float x[V];
      VecIO<T>::load(a + i * V, x);
      if (PAIR) {
        float y[V];
        VecIO<T>::load(b + i * V, y);
#pragma unroll
        for (int j = 0; j < V; ++j) x[j] = pair_fn<PAIR>(x[j], y[j]);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) acc = red_combine<OP>(acc, x[j]);
    }
    done = nvec * V;
  }
  for (int64_t i = done + tid; i < n; i += nthreads) {
    float x = VecIO<T>::ld(a + i);
    if (PAIR) x = pair_fn<PAIR>(x, VecIO<T>::ld(b + i));
    acc = red_combine<OP>(acc, x);
  }
  acc = red_block<OP>(acc, sh);
  if (threadIdx.x == 0) {
    scratch->partial[blockIdx.x] = acc;
    __threadfence();
    unsigned int t = atomicAdd(&scratch->ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    float r = red_identity<OP>();
    for (int i = threadIdx.x; i < (int)gridDim.x; i += THREADS)
      r = red_combine<OP>(r, ((volatile float*)scratch->partial)[i]);
    r = red_block<OP>(r, sh);
    if (threadIdx.x == 0) {
      *out = r * scale;
      scratch->ticket = 0;  // ready for the next call on this stream
    }
  }
}

template <typename T, int OP, int PAIR>
cudaError_t launch_reduce(const void* a, const void* b, int64_t n, float scale, float* out,
                          void* scratch, cudaStream_t s) {
  int grid = stream_grid((n + VecIO<T>::N - 1) / VecIO<T>::N, THREADS);
  if (grid > MAX_PARTIALS) grid = MAX_PARTIALS;
  const int vec_ok = is_aligned16(a) && (!b || is_aligned16(b));
  reduce_kernel<T, OP, PAIR><<<grid, THREADS, 0, s>>>((const T*)a, (const T*)b, n, scale, out,
                                                (Scratch*)scratch, vec_ok);
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
finite_scale_kernel(T* a, int64_t n, float scale, int write_back, int* flag) {
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  bool bad = false;
  for (int64_t i = tid; i < n; i += nthreads) {
    float x = VecIO<T>::ld(a + i) * scale;
    if (!isfinite(x)) bad = true;
    if (write_back) VecIO<T>::st(a + i, x);
  }
  bad = __any_sync(0xffffffffu, bad);
  if (bad && (threadIdx.x & 31) == 0) atomicOr(flag, 1);
}

}  // namespace

size_t reduce_scratch_bytes() { return sizeof(Scratch); }

cudaError_t reduce_all(int op, int dtype, const void* a, int64_t n, float scale, float* out,
                       void* scratch, cudaStream_t s) {
  if (n <= 0) return cudaErrorInvalidValue;
  LT_DISPATCH_DTYPE(dtype, T, switch (op) {
    case RED_SUM: return launch_reduce<T, RED_SUM, 0>(a, nullptr, n, scale, out, scratch, s);
    case RED_MAX: return launch_reduce<T, RED_MAX, 0>(a, nullptr, n, scale, out, scratch, s);
    case RED_MIN: return launch_reduce<T, RED_MIN, 0>(a, nullptr, n, scale, out, scratch, s);
    default: return cudaErrorInvalidValue;
  })
  return cudaErrorInvalidValue;
}

cudaError_t dot_all(int dtype, const void* a, const void* b, int64_t n, float* out, void* scratch,
                    cudaStream_t s) {
  if (n <= 0) return cudaErrorInvalidValue;
  LT_DISPATCH_DTYPE(dtype, T, return launch_reduce<T, RED_SUM, 1>(a, b, n, 1.0f, out, scratch, s))
  return cudaErrorInvalidValue;
}

cudaError_t pointwise_loss(int mode, int dtype, const void* pred, const void* target, int64_t n,
                           float* loss_out, void* scratch, cudaStream_t s) {
  if (n <= 0) return cudaErrorInvalidValue;
  const float scale = 1.0f / (float)n;
  LT_DISPATCH_DTYPE(dtype, T, {
    if (mode == 0) return launch_reduce<T, RED_SUM, 2>(pred, target, n, scale, loss_out, scratch, s);
    return launch_reduce<T, RED_SUM, 3>(pred, target, n, scale, loss_out, scratch, s);
  })
  return cudaErrorInvalidValue;
}

cudaError_t check_finite_scale(int dtype, void* a, int64_t n, float scale, int write_back,
                               int* flag, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    finite_scale_kernel<T><<<stream_grid(n, THREADS), THREADS, 0, s>>>((T*)a, n, scale, write_back,
                                                                      flag);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

}  // namespace lt
