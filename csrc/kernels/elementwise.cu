// Elementwise family: one templated, 16-byte-vectorised grid-stride kernel shape for all
// binary / scalar / unary ops, their activation backward forms, casts, RNG fills and
// dropout, plus bias broadcast, deterministic column sums, 2-d transpose and the bf16
// hi/lo split that feeds the fp32-accurate tensor-core matmul.
//
// Covers the reference kernels K1-K22, K27-K33, K46 and K48 (csrc/cuda/ops/arithmetic.cu,
// activation.cu, cast.cu, matmul.cu:199-206), which are scalar one-thread-per-element
// launches of 256-thread blocks there.
#include <stdlib.h>
#include "ops.h"
#include "common.cuh"

namespace lt {

std::atomic<uint64_t> g_ops_launches{0};
uint64_t ops_launch_count() { return g_ops_launches.load(); }
int g_pdl_override = -1;
int g_late_chain = 0;
int g_late_side = 0;
unsigned long long g_pdl_seq = 0, g_side_mark = 0;
void set_pdl_override(int v) { g_pdl_override = v < 0 ? -1 : (v != 0); }

namespace {

constexpr int THREADS = 256;

// out[i] = f(a[i], b[i]) ; b may be null for unary functors.
template <typename T, typename F>
__global__ void __launch_bounds__(THREADS)
map_kernel(const T* a, const T* b, T* out, int64_t n,  // a/b may alias out (in-place ops)
           int vec_ok, F f) {
  constexpr int V = VecIO<T>::N;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  int64_t done = 0;
  if (vec_ok) {
    const int64_t nvec = n / V;
    for (int64_t i = tid; i < nvec; i += nthreads) {
      float x[V], y[V], o[V];
      VecIO<T>::load(a + i * V, x);
      if (b) VecIO<T>::load(b + i * V, y);
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = f(x[j], b ? y[j] : 0.0f);
      VecIO<T>::store(out + i * V, o);
    }
    done = nvec * V;
  }
  for (int64_t i = done + tid; i < n; i += nthreads) {
    float x = VecIO<T>::ld(a + i);
    float y = b ? VecIO<T>::ld(b + i) : 0.0f;
    VecIO<T>::st(out + i, f(x, y));
  }
}

template <typename T, typename F>
cudaError_t launch_map(const void* a, const void* b, void* out, int64_t n, F f, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int vec_ok = is_aligned16(a) && is_aligned16(out) && (!b || is_aligned16(b));
  const int grid = stream_grid((n + VecIO<T>::N - 1) / VecIO<T>::N, THREADS);
  map_kernel<T, F><<<grid, THREADS, 0, s>>>((const T*)a, (const T*)b, (T*)out, n, vec_ok, f);
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

template <int OP> struct BinF {
  __device__ __forceinline__ float operator()(float x, float y) const {
    if (OP == BIN_ADD) return x + y;
    if (OP == BIN_SUB) return x - y;
    if (OP == BIN_MUL) return x * y;
    return y == 0.0f ? 0.0f : x / y;  // division by zero yields 0, as the CPU op does
  }
};
template <int OP> struct ScalarF {
  float s;
  __device__ __forceinline__ float operator()(float x, float) const {
    if (OP == SC_ADD) return x + s;
    if (OP == SC_MUL) return x * s;
    if (OP == SC_DIV) return x / s;
    if (OP == SC_POW) return powf(x, s);
    return x > s ? 1.0f : 0.0f;
  }
};
template <int OP> struct UnaryF {
  __device__ __forceinline__ float operator()(float x, float) const {
    switch (OP) {
      case UN_NEG: return -x;
      case UN_ABS: return fabsf(x);
      case UN_SQRT: return x < 0.0f ? 0.0f : sqrtf(x);
      case UN_LOG: return x <= 0.0f ? -INFINITY : logf(x);
      case UN_EXP: return expf(x);
      case UN_RELU: return x > 0.0f ? x : 0.0f;
      case UN_SIGMOID: return 1.0f / (1.0f + expf(-x));
      case UN_TANH: return tanhf(x);
      case UN_GELU: return gelu_exact_tanh(x);
      default: return x / (1.0f + expf(-x));
    }
  }
};
// (x, dy) -> dy * f'(x)
template <int OP> struct UnaryBwdF {
  __device__ __forceinline__ float operator()(float x, float dy) const {
    switch (OP) {
      case UN_RELU: return x > 0.0f ? dy : 0.0f;
      case UN_SIGMOID: { float s = 1.0f / (1.0f + expf(-x)); return dy * s * (1.0f - s); }
      case UN_TANH: { float t = tanhf(x); return dy * (1.0f - t * t); }
      case UN_GELU: return dy * dgelu_exact_tanh(x);
      default: { float s = 1.0f / (1.0f + expf(-x)); return dy * (s + x * s * (1.0f - s)); }
    }
  }
};

}  // namespace

cudaError_t binary_op(int op, int dtype, const void* a, const void* b, void* out, int64_t n,
                      cudaStream_t s) {
  LT_DISPATCH_DTYPE(dtype, T, switch (op) {
    case BIN_ADD: return launch_map<T>(a, b, out, n, BinF<BIN_ADD>(), s);
    case BIN_SUB: return launch_map<T>(a, b, out, n, BinF<BIN_SUB>(), s);
    case BIN_MUL: return launch_map<T>(a, b, out, n, BinF<BIN_MUL>(), s);
    case BIN_DIV: return launch_map<T>(a, b, out, n, BinF<BIN_DIV>(), s);
    default: return cudaErrorInvalidValue;
  })
  return cudaErrorInvalidValue;
}

cudaError_t scalar_op(int op, int dtype, const void* a, float sc, void* out, int64_t n,
                      cudaStream_t s) {
  LT_DISPATCH_DTYPE(dtype, T, switch (op) {
    case SC_ADD: return launch_map<T>(a, nullptr, out, n, ScalarF<SC_ADD>{sc}, s);
    case SC_MUL: return launch_map<T>(a, nullptr, out, n, ScalarF<SC_MUL>{sc}, s);
    case SC_DIV: return launch_map<T>(a, nullptr, out, n, ScalarF<SC_DIV>{sc}, s);
    case SC_POW: return launch_map<T>(a, nullptr, out, n, ScalarF<SC_POW>{sc}, s);
    case SC_GT: return launch_map<T>(a, nullptr, out, n, ScalarF<SC_GT>{sc}, s);
    default: return cudaErrorInvalidValue;
  })
  return cudaErrorInvalidValue;
}

cudaError_t unary_op(int op, int dtype, const void* a, void* out, int64_t n, cudaStream_t s) {
  LT_DISPATCH_DTYPE(dtype, T, switch (op) {
    case UN_NEG: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_NEG>(), s);
    case UN_ABS: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_ABS>(), s);
    case UN_SQRT: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_SQRT>(), s);
    case UN_LOG: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_LOG>(), s);
    case UN_EXP: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_EXP>(), s);
    case UN_RELU: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_RELU>(), s);
    case UN_SIGMOID: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_SIGMOID>(), s);
    case UN_TANH: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_TANH>(), s);
    case UN_GELU: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_GELU>(), s);
    case UN_SILU: return launch_map<T>(a, nullptr, out, n, UnaryF<UN_SILU>(), s);
    default: return cudaErrorInvalidValue;
  })
  return cudaErrorInvalidValue;
}

cudaError_t unary_backward(int op, int dtype, const void* x, const void* dy, void* dx, int64_t n,
                           cudaStream_t s) {
  LT_DISPATCH_DTYPE(dtype, T, switch (op) {
    case UN_RELU: return launch_map<T>(x, dy, dx, n, UnaryBwdF<UN_RELU>(), s);
    case UN_SIGMOID: return launch_map<T>(x, dy, dx, n, UnaryBwdF<UN_SIGMOID>(), s);
    case UN_TANH: return launch_map<T>(x, dy, dx, n, UnaryBwdF<UN_TANH>(), s);
    case UN_GELU: return launch_map<T>(x, dy, dx, n, UnaryBwdF<UN_GELU>(), s);
    case UN_SILU: return launch_map<T>(x, dy, dx, n, UnaryBwdF<UN_SILU>(), s);
    default: return cudaErrorInvalidValue;
  })
  return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------------ broadcast add
namespace {
template <typename T>
__global__ void __launch_bounds__(THREADS)
add_broadcast_kernel(const T* __restrict__ a, const T* __restrict__ bias, T* __restrict__ out,
                     int64_t rows, int64_t cols, int vec_ok) {
  constexpr int V = VecIO<T>::N;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec_ok) {
    const int64_t cv = cols / V, nvec = rows * cv;
    for (int64_t i = tid; i < nvec; i += nthreads) {
      const int64_t c = (i % cv) * V;
      float x[V], bb[V];
      VecIO<T>::load(a + i * V, x);
      VecIO<T>::load(bias + c, bb);
#pragma unroll
      for (int j = 0; j < V; ++j) x[j] += bb[j];
      VecIO<T>::store(out + i * V, x);
    }
  } else {
    const int64_t n = rows * cols;
    for (int64_t i = tid; i < n; i += nthreads)
      VecIO<T>::st(out + i, VecIO<T>::ld(a + i) + VecIO<T>::ld(bias + i % cols));
  }
}
}  // namespace

cudaError_t add_broadcast(int dtype, const void* a, const void* bias, void* out, int64_t rows,
                          int64_t cols, cudaStream_t s) {
  if (rows * cols <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    const int vec_ok = is_aligned16(a) && is_aligned16(bias) && is_aligned16(out) &&
                       cols % VecIO<T>::N == 0;
    const int grid = stream_grid(rows * cols / VecIO<T>::N + 1, THREADS);
    add_broadcast_kernel<T><<<grid, THREADS, 0, s>>>((const T*)a, (const T*)bias, (T*)out, rows,
                                                     cols, vec_ok);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

// out[r, c] = a[r, c] * scale[c] + shift[c]   (shift may be null)
namespace {
template <typename T>
__global__ void __launch_bounds__(THREADS)
affine_cols_kernel(const T* __restrict__ a, const T* __restrict__ scale,
                   const T* __restrict__ shift, T* __restrict__ out, int64_t rows, int64_t cols) {
  const int64_t n = rows * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c = i % cols;
    float v = VecIO<T>::ld(a + i) * VecIO<T>::ld(scale + c);
    if (shift) v += VecIO<T>::ld(shift + c);
    VecIO<T>::st(out + i, v);
  }
}
}  // namespace

cudaError_t affine_cols(int dtype, const void* a, const void* scale, const void* shift, void* out,
                        int64_t rows, int64_t cols, cudaStream_t s) {
  if (rows * cols <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    affine_cols_kernel<T><<<stream_grid(rows * cols, THREADS), THREADS, 0, s>>>(
        (const T*)a, (const T*)scale, (const T*)shift, (T*)out, rows, cols);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------------ column sum
// Stage 1: each block sums a 128-row slab for 32*V... columns into scratch[slab, col] (fp32).
// Stage 2: one thread per column adds the slabs in a fixed order => bitwise deterministic,
// unlike the reference's per-element atomicAdd (csrc/cuda/ops/arithmetic.cu:504-510).
namespace {
constexpr int CS_ROWS = 128;

template <typename T>
__global__ void __launch_bounds__(256)
colsum_stage1(const T* __restrict__ in, int64_t ld, int64_t rows, int64_t cols,
              float* __restrict__ scratch) {
  // block: 32 columns x 8 row-lanes
  __shared__ float sh[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int64_t col = blockIdx.x * 32 + cx;
  const int64_t r0 = (int64_t)blockIdx.y * CS_ROWS;
  float acc = 0.0f;
  if (col < cols) {
    const int64_t r1 = r0 + CS_ROWS < rows ? r0 + CS_ROWS : rows;
    for (int64_t r = r0 + ry; r < r1; r += 8) acc += VecIO<T>::ld(in + r * ld + col);
  }
  sh[ry][cx] = acc;
  __syncthreads();
  if (ry == 0 && col < cols) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sh[i][cx];
    scratch[(int64_t)blockIdx.y * cols + col] = t;
  }
}

template <typename TO>
__global__ void colsum_stage2(const float* __restrict__ scratch, int64_t slabs, int64_t cols,
                              TO* __restrict__ out, int accumulate) {
  const int64_t col = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (col >= cols) return;
  float t = 0.0f;
  for (int64_t sidx = 0; sidx < slabs; ++sidx) t += scratch[sidx * cols + col];
  if (accumulate) t += VecIO<TO>::ld(out + col);
  VecIO<TO>::st(out + col, t);
}

// Single-launch form for 16-byte-aligned inputs: block = (32 x V columns, slab of rows), eight
// warps stride over the slab with independent vector loads; the partial row of the slab goes to
// scratch and the LAST block of a column group (ticket) adds the slabs in index order, so the
// result does not depend on which block that is.  The ticket words live in this module and are
// left at zero; calls that can overlap on different streams must not share column groups.
constexpr int CS_MAX_GROUPS = 1024;
__device__ unsigned int g_colsum_tickets[CS_MAX_GROUPS];

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
colsum_fused(const T* __restrict__ in, int64_t ld, int64_t rows, int64_t cols,
             int64_t rows_per_slab, float* __restrict__ scratch, TO* __restrict__ out,
             int accumulate) {
  constexpr int V = VecIO<T>::N;
  __shared__ float sh[8][32 * V + 1];
  __shared__ int is_last;
  pdl_enter();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c0 = ((int64_t)blockIdx.x * 32 + lane) * V;
  const bool ok = c0 < cols;
  const int64_t r0 = blockIdx.y * rows_per_slab;
  const int64_t r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.0f;
  if (ok) {
    // eight rows requested at a time, added in row order
    for (int64_t rb = r0 + warp; rb < r1; rb += 8 * 8) {
      uint4 raw[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int64_t r = rb + 8 * k;
        if (r < r1) raw[k] = VecIO<T>::load_raw(in + r * ld + c0);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (rb + 8 * k < r1) {
          float v[V];
          VecIO<T>::unpack(raw[k], v);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += v[j];
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) sh[warp][lane * V + j] = acc[j];
  __syncthreads();
  const int64_t gcol0 = (int64_t)blockIdx.x * 32 * V;
  for (int c = threadIdx.x; c < 32 * V; c += 256) {
    if (gcol0 + c < cols) {
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += sh[w][c];
      scratch[(int64_t)blockIdx.y * cols + gcol0 + c] = t;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(&g_colsum_tickets[blockIdx.x], 1u);
    is_last = (t == gridDim.y - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int c = threadIdx.x; c < 32 * V; c += 256) {
    const int64_t col = gcol0 + c;
    if (col < cols) {
      float t = 0.0f;
      for (unsigned int s0 = 0; s0 < gridDim.y; s0 += 16) {   // 16 loads in flight, slab order kept
        float v[16];
#pragma unroll
        for (int k = 0; k < 16; ++k)
          v[k] = s0 + k < gridDim.y ? __ldcg(scratch + (int64_t)(s0 + k) * cols + col) : 0.0f;
#pragma unroll
        for (int k = 0; k < 16; ++k) t += v[k];
      }
      if (accumulate) t += VecIO<TO>::ld(out + col);
      VecIO<TO>::st(out + col, t);
    }
  }
  if (threadIdx.x == 0) g_colsum_tickets[blockIdx.x] = 0;
}
}  // namespace

int64_t column_sum_scratch_floats(int64_t rows, int64_t cols) {
  return ((rows + CS_ROWS - 1) / CS_ROWS) * cols;
}

cudaError_t column_sum(int dtype, const void* in, int64_t ld, void* out, int out_dtype,
                       int accumulate, int64_t rows, int64_t cols, float* scratch,
                       cudaStream_t s) {
  if (cols <= 0) return cudaSuccess;
  {
    const int v = dtype == DT_F32 ? 4 : 8;
    const int64_t groups = (cols + 32 * v - 1) / (32 * v);
    if (rows > 0 && cols % v == 0 && ld % v == 0 && is_aligned16(in) && groups <= CS_MAX_GROUPS) {
      // about four blocks per SM, and never more slabs than the scratch was sized for
      int64_t slabs = (4 * 148 + groups - 1) / groups;
      const int64_t max_slabs = (rows + CS_ROWS - 1) / CS_ROWS;
      if (slabs > max_slabs) slabs = max_slabs;
      if (slabs > 64) slabs = 64;   // the closing block adds the slabs one after another
      if (slabs < 1) slabs = 1;
      const int64_t rps = (rows + slabs - 1) / slabs;
      slabs = (rows + rps - 1) / rps;
      dim3 g((unsigned)groups, (unsigned)slabs);
      LT_DISPATCH_DTYPE(dtype, T, {
        LT_DISPATCH_DTYPE(out_dtype, TO, {
          launch_pdl(colsum_fused<T, TO>, g, dim3(256), 0, s, (const T*)in, ld, rows, cols, rps, scratch,
                     (TO*)out, accumulate);
          LT_COUNT_LAUNCH();
          return cudaGetLastError();
        })
      })
    }
  }
  const int64_t slabs = (rows + CS_ROWS - 1) / CS_ROWS;
  dim3 g1((unsigned)((cols + 31) / 32), (unsigned)(slabs > 0 ? slabs : 1));
  LT_DISPATCH_DTYPE(dtype, T, {
    colsum_stage1<T><<<g1, 256, 0, s>>>((const T*)in, ld, rows, cols, scratch);
    LT_COUNT_LAUNCH();
  })
  LT_DISPATCH_DTYPE(out_dtype, TO, {
    colsum_stage2<TO><<<(unsigned)((cols + 255) / 256), 256, 0, s>>>(scratch, slabs, cols,
                                                                      (TO*)out, accumulate);
    LT_COUNT_LAUNCH();
  })
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------ casts
namespace {
template <typename TI, typename TO>
__global__ void __launch_bounds__(THREADS)
cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, int64_t n, int vec_ok) {
  // process 8 elements per step so both 2-byte and 4-byte sides stay 16-byte aligned
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  int64_t done = 0;
  if (vec_ok) {
    const int64_t n8 = n / 8;
    for (int64_t i = tid; i < n8; i += nthreads) {
      float f[8];
      if constexpr (VecIO<TI>::N == 8) {
        VecIO<TI>::load(in + i * 8, f);
      } else {
        float t0[4], t1[4];
        VecIO<TI>::load(in + i * 8, t0);
        VecIO<TI>::load(in + i * 8 + 4, t1);
#pragma unroll
        for (int j = 0; j < 4; ++j) { f[j] = t0[j]; f[4 + j] = t1[j]; }
      }
      if constexpr (VecIO<TO>::N == 8) {
        VecIO<TO>::store(out + i * 8, f);
      } else {
        float t0[4], t1[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { t0[j] = f[j]; t1[j] = f[4 + j]; }
        VecIO<TO>::store(out + i * 8, t0);
        VecIO<TO>::store(out + i * 8 + 4, t1);
      }
    }
    done = n8 * 8;
  }
  for (int64_t i = done + tid; i < n; i += nthreads) VecIO<TO>::st(out + i, VecIO<TI>::ld(in + i));
}
}  // namespace

cudaError_t cast(int src_dtype, const void* src, int dst_dtype, void* dst, int64_t n,
                 cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int vec_ok = is_aligned16(src) && is_aligned16(dst);
  const int grid = stream_grid((n + 7) / 8, THREADS);
  LT_DISPATCH_DTYPE(src_dtype, TI, {
    LT_DISPATCH_DTYPE(dst_dtype, TO, {
      cast_kernel<TI, TO><<<grid, THREADS, 0, s>>>((const TI*)src, (TO*)dst, n, vec_ok);
      LT_COUNT_LAUNCH();
      return cudaGetLastError();
    })
  })
  return cudaErrorInvalidValue;
}

namespace {
__global__ void __launch_bounds__(THREADS)
split_bf16_kernel(const float* __restrict__ a, __nv_bfloat16* __restrict__ hi,
                  __nv_bfloat16* __restrict__ lo, int64_t n) {
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n; i += nthreads) {
    float x = a[i];
    __nv_bfloat16 h = __float2bfloat16(x);
    hi[i] = h;
    lo[i] = __float2bfloat16(x - __bfloat162float(h));
  }
}
}  // namespace

cudaError_t split_bf16(const float* a, void* hi, void* lo, int64_t n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  split_bf16_kernel<<<stream_grid(n, THREADS), THREADS, 0, s>>>(a, (__nv_bfloat16*)hi,
                                                               (__nv_bfloat16*)lo, n);
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------ transpose
namespace {
template <typename T>
__global__ void __launch_bounds__(256)
transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int64_t cols) {
  __shared__ T tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    int64_t r = r0 + ty + i, c = c0 + tx;
    if (r < rows && c < cols) tile[ty + i][tx] = in[r * cols + c];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    int64_t c = c0 + ty + i, r = r0 + tx;
    if (r < rows && c < cols) out[c * rows + r] = tile[tx][ty + i];
  }
}
}  // namespace

cudaError_t transpose2d(int dtype, const void* in, void* out, int64_t rows, int64_t cols,
                        cudaStream_t s) {
  if (rows * cols <= 0) return cudaSuccess;
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
  LT_DISPATCH_DTYPE(dtype, T, {
    transpose_kernel<T><<<grid, 256, 0, s>>>((const T*)in, (T*)out, rows, cols);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------------ RNG / dropout
namespace {
template <typename T>
__global__ void __launch_bounds__(THREADS)
fill_random_kernel(T* __restrict__ out, int64_t n, uint64_t seed, uint64_t offset, int normal) {
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int64_t groups = (n + 3) / 4;
  for (int64_t g = tid; g < groups; g += nthreads) {
    uint4 r = philox4(offset + (uint64_t)g, seed);
    float v[4];
    if (normal) {
      // Box-Muller on two pairs
      float u0 = u32_to_unit(r.x), u1 = u32_to_unit(r.y), u2 = u32_to_unit(r.z), u3 = u32_to_unit(r.w);
      float m0 = sqrtf(-2.0f * logf(u0)), m1 = sqrtf(-2.0f * logf(u2));
      float s0, c0, s1, c1;
      sincospif(2.0f * u1, &s0, &c0);
      sincospif(2.0f * u3, &s1, &c1);
      v[0] = m0 * c0; v[1] = m0 * s0; v[2] = m1 * c1; v[3] = m1 * s1;
    } else {
      v[0] = (r.x >> 8) * (1.0f / 16777216.0f); v[1] = (r.y >> 8) * (1.0f / 16777216.0f);
      v[2] = (r.z >> 8) * (1.0f / 16777216.0f); v[3] = (r.w >> 8) * (1.0f / 16777216.0f);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t i = g * 4 + j;
      if (i < n) VecIO<T>::st(out + i, v[j]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
dropout_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n, float p, float inv_keep,
               uint64_t seed, uint64_t offset, const uint64_t* __restrict__ dyn_offset) {
  if (dyn_offset) offset += *dyn_offset;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int64_t groups = (n + 3) / 4;
  for (int64_t g = tid; g < groups; g += nthreads) {
    uint4 r = philox4(offset + (uint64_t)g, seed);
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t i = g * 4 + j;
      if (i < n) {
        float u = (rr[j] >> 8) * (1.0f / 16777216.0f);
        VecIO<T>::st(out + i, u >= p ? VecIO<T>::ld(x + i) * inv_keep : 0.0f);
      }
    }
  }
}
}  // namespace

cudaError_t fill_random(int dtype, void* out, int64_t n, uint64_t seed, uint64_t offset,
                        int normal, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    fill_random_kernel<T><<<stream_grid((n + 3) / 4, THREADS), THREADS, 0, s>>>(
        (T*)out, n, seed, offset, normal);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

cudaError_t dropout(int dtype, const void* x, void* out, int64_t n, float p, uint64_t seed,
                    uint64_t offset, cudaStream_t s, const uint64_t* dyn_offset) {
  if (n <= 0) return cudaSuccess;
  const float inv_keep = p < 1.0f ? 1.0f / (1.0f - p) : 0.0f;
  LT_DISPATCH_DTYPE(dtype, T, {
    dropout_kernel<T><<<stream_grid((n + 3) / 4, THREADS), THREADS, 0, s>>>(
        (const T*)x, (T*)out, n, p, inv_keep, seed, offset, dyn_offset);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

}  // namespace lt
