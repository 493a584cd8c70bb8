// Row softmax, attention-score softmax (forward / backward, in place) and fused
// softmax-cross-entropy forward / backward.
//
// One CTA per row with an online (single read) max / sum-exp pass; cross entropy keeps the
// row log-sum-exp so backward needs one read of the logits and one write of the gradient.
// The reference computes cross entropy with ONE THREAD per row looping serially over the
// classes (csrc/cuda/ops/loss.cu:63-125) and its softmax reads each row three times
// (csrc/cuda/ops/activation.cu:65-112).
#include "ops.h"
#include "common.cuh"

namespace lt {
namespace {

constexpr int THREADS = 256;

struct MaxSum { float m, s; };
__device__ __forceinline__ MaxSum ms_combine(MaxSum a, MaxSum b) {
  float m = fmaxf(a.m, b.m);
  if (m == -INFINITY) return MaxSum{m, 0.0f};
  return MaxSum{m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}
__device__ __forceinline__ void ms_push(MaxSum& a, float x) {
  if (x > a.m) { a.s = a.s * __expf(a.m - x) + 1.0f; a.m = x; }
  else if (x != -INFINITY) a.s += __expf(x - a.m);
}
__device__ __forceinline__ MaxSum ms_block(MaxSum v, float* sh_m, float* sh_s) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum t{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = ms_combine(v, t);
  }
  __syncthreads();
  if (lane == 0) { sh_m[w] = v.m; sh_s[w] = v.s; }
  __syncthreads();
  MaxSum r = lane < nw ? MaxSum{sh_m[lane], sh_s[lane]} : MaxSum{-INFINITY, 0.0f};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum t{__shfl_xor_sync(0xffffffffu, r.m, o), __shfl_xor_sync(0xffffffffu, r.s, o)};
    r = ms_combine(r, t);
  }
  return r;
}

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// A row of `cols` elements starting at any element-aligned address splits into `head`
// leading elements (up to the first 16-byte boundary), `nvec` 16-byte vectors and a tail,
// so rows whose leading dimension is odd (a vocabulary of 50257 columns) still move as
// 16-byte accesses.
template <typename T>
struct RowSplit {
  int head, nvec;
  __device__ __forceinline__ RowSplit(const T* row, int64_t cols) {
    constexpr int V = VecIO<T>::N;
    const int mis = (int)((reinterpret_cast<uintptr_t>(row) & 15) / sizeof(T));
    int h = mis ? V - mis : 0;
    if (h > cols) h = (int)cols;
    head = h;
    nvec = (int)((cols - h) / V);
  }
  __device__ __forceinline__ int64_t tail_begin() const { return head + (int64_t)nvec * VecIO<T>::N; }
};

// Online max / sum-exp over one row: one read, in the exp2 domain (one FFMA and one MUFU per
// element); the running maximum moves only when a whole vector beats it.
template <typename T>
__device__ __forceinline__ MaxSum row_maxsum(const T* row, int64_t cols) {
  constexpr int V = VecIO<T>::N;
  const RowSplit<T> sp(row, cols);
  MaxSum acc{-INFINITY, 0.0f};
  if ((int)threadIdx.x < sp.head) ms_push(acc, VecIO<T>::ld(row + threadIdx.x));
  const T* vrow = row + sp.head;
  float c = acc.m == -INFINITY ? 0.0f : -acc.m * LOG2E;   // exponent offset of the running max
  float s0 = acc.s, s1 = 0.0f;
  for (int i = threadIdx.x; i < sp.nvec; i += blockDim.x) {
    float x[V];
    VecIO<T>::unpack(VecIO<T>::load_raw(vrow + (int64_t)i * V), x);
    float mx = x[0];
#pragma unroll
    for (int j = 1; j < V; ++j) mx = fmaxf(mx, x[j]);
    if (mx > acc.m) {
      const float f = ex2_fast(fmaf(acc.m == -INFINITY ? 0.0f : acc.m, LOG2E, -mx * LOG2E));
      s0 *= f; s1 *= f;
      acc.m = mx;
      c = -mx * LOG2E;
    }
#pragma unroll
    for (int j = 0; j < V; j += 2) {
      s0 += ex2_fast(fmaf(x[j], LOG2E, c));
      s1 += ex2_fast(fmaf(x[j + 1], LOG2E, c));
    }
  }
  acc.s = s0 + s1;
  for (int64_t i = sp.tail_begin() + threadIdx.x; i < cols; i += blockDim.x) ms_push(acc, VecIO<T>::ld(row + i));
  return acc;
}

// Second pass shared by the softmax / cross-entropy kernels: out[i] = exp(x[i] - l) * gs,
// minus gs at column `lab` (lab < 0: no label).  `in` and `out` may be the same row; they
// must share their misalignment within 16 bytes for the vector path.
template <typename T>
__device__ __forceinline__ void row_exp_scale(const T* in, T* out, int64_t cols, float l, float gs,
                                              int64_t lab) {
  constexpr int V = VecIO<T>::N;
  const float c = -l * LOG2E;
  const bool same_mis = ((reinterpret_cast<uintptr_t>(in) ^ reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const RowSplit<T> sp(in, same_mis ? cols : 0);
  int64_t first_tail = 0;
  if (same_mis) {
    if ((int)threadIdx.x < sp.head) {
      float pj = ex2_fast(fmaf(VecIO<T>::ld(in + threadIdx.x), LOG2E, c));
      if ((int64_t)threadIdx.x == lab) pj -= 1.0f;
      VecIO<T>::st(out + threadIdx.x, pj * gs);
    }
    const T* vin = in + sp.head;
    T* vout = out + sp.head;
    const int64_t vlab = lab - sp.head;
    const int lab_vec = vlab >= 0 ? (int)(vlab / V) : -1;
    // a positive scale folds into the exponent: exp2(x*log2e - l*log2e + log2(gs))
    const bool fold = gs > 0.0f;
    const float cf = fold ? c + __log2f(gs) : c;
    const float mul = fold ? 1.0f : gs;
    for (int i = threadIdx.x; i < sp.nvec; i += blockDim.x) {
      float x[V];
      VecIO<T>::unpack(VecIO<T>::load_raw(vin + (int64_t)i * V), x);
      if (fold) {
#pragma unroll
        for (int j = 0; j < V; ++j) x[j] = ex2_fast(fmaf(x[j], LOG2E, cf));
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) x[j] = ex2_fast(fmaf(x[j], LOG2E, cf)) * mul;
      }
      if (i == lab_vec) {
        const int jl = (int)(vlab - (int64_t)lab_vec * V);
#pragma unroll
        for (int j = 0; j < V; ++j) if (j == jl) x[j] -= gs;
      }
      VecIO<T>::store(vout + (int64_t)i * V, x);
    }
    first_tail = sp.tail_begin();
  }
  for (int64_t i = first_tail + threadIdx.x; i < cols; i += blockDim.x) {
    float pj = ex2_fast(fmaf(VecIO<T>::ld(in + i), LOG2E, c));
    if (i == lab) pj -= 1.0f;
    VecIO<T>::st(out + i, pj * gs);
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
softmax_rows_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t cols, int64_t ld) {
  __shared__ float sh_m[32], sh_s[32];
  const T* row = in + blockIdx.x * ld;
  T* orow = out + blockIdx.x * ld;
  MaxSum ms = ms_block(row_maxsum<T>(row, cols), sh_m, sh_s);
  row_exp_scale<T>(row, orow, cols, ms.m, 1.0f / ms.s, -1);
}

// Attention scores: in-place softmax over bf16 rows, columns beyond the diagonal masked
// when causal. One warp per row; a row of up to 2048 columns lives in registers.
__global__ void __launch_bounds__(256)
softmax_scores_kernel(__nv_bfloat16* __restrict__ sc, int64_t n_rows, int64_t rows_per_batch,
                      int64_t cols, int64_t ld, int causal) {
  const int lane = threadIdx.x & 31;
  const int64_t r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  __nv_bfloat16* row = sc + r * ld;
  const int64_t q = r % rows_per_batch;
  const int64_t valid = causal ? (q + 1 < cols ? q + 1 : cols) : cols;
  float m = -INFINITY;
  for (int64_t c = lane; c < valid; c += 32) m = fmaxf(m, __bfloat162float(row[c]));
  m = warp_max(m);
  float s = 0.0f;
  for (int64_t c = lane; c < valid; c += 32) s += __expf(__bfloat162float(row[c]) - m);
  s = warp_sum(s);
  const float inv = 1.0f / s;
  for (int64_t c = lane; c < cols; c += 32)
    row[c] = __float2bfloat16(c < valid ? __expf(__bfloat162float(row[c]) - m) * inv : 0.0f);
}

__global__ void __launch_bounds__(256)
softmax_scores_bwd_kernel(const __nv_bfloat16* __restrict__ p, __nv_bfloat16* __restrict__ dp,
                          int64_t n_rows, int64_t rows_per_batch, int64_t cols, int64_t ld,
                          float scale, int causal) {
  const int lane = threadIdx.x & 31;
  const int64_t r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const __nv_bfloat16* prow = p + r * ld;
  __nv_bfloat16* drow = dp + r * ld;
  const int64_t q = r % rows_per_batch;
  const int64_t valid = causal ? (q + 1 < cols ? q + 1 : cols) : cols;
  float dot = 0.0f;
  for (int64_t c = lane; c < valid; c += 32)
    dot += __bfloat162float(prow[c]) * __bfloat162float(drow[c]);
  dot = warp_sum(dot);
  for (int64_t c = lane; c < cols; c += 32) {
    float v = 0.0f;
    if (c < valid) v = __bfloat162float(prow[c]) * (__bfloat162float(drow[c]) - dot) * scale;
    drow[c] = __float2bfloat16(v);
  }
}

__device__ __forceinline__ int64_t read_label(const void* labels, int kind, int64_t r) {
  if (kind == 0) return ((const int64_t*)labels)[r];
  if (kind == 1) return ((const int*)labels)[r];
  return (int64_t)((const float*)labels)[r];
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
ce_forward_kernel(const T* __restrict__ logits, int64_t ld, const void* __restrict__ labels,
                  int label_kind, int64_t cols, float* __restrict__ lse,
                  float* __restrict__ row_loss, int* err_flag) {
  pdl_enter();
  __shared__ float sh_m[32], sh_s[32];
  const int64_t r = blockIdx.x;
  const T* row = logits + r * ld;
  MaxSum ms = ms_block(row_maxsum<T>(row, cols), sh_m, sh_s);
  if (threadIdx.x == 0) {
    const float l = ms.m + __logf(ms.s);
    lse[r] = l;
    const int64_t lab = read_label(labels, label_kind, r);
    if (lab < 0 || lab >= cols) {
      // status word, never a trap: [0] flag, [1] row, [2] offending label (first seen)
      if (err_flag && atomicOr(err_flag, 1) == 0) { err_flag[1] = (int)r; err_flag[2] = (int)lab; }
      row_loss[r] = 0.0f;
    } else {
      row_loss[r] = l - VecIO<T>::ld(row + lab);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
ce_backward_kernel(const T* logits, int64_t ld, const void* __restrict__ labels, int label_kind,
                   int64_t cols, const float* __restrict__ lse, float grad_scale,
                   const float* __restrict__ gs_dev, T* dlogits, int64_t ld_out) {
  pdl_enter();
  const int64_t r = blockIdx.x;
  const float gs = gs_dev ? grad_scale * gs_dev[0] : grad_scale;
  int64_t lab = read_label(labels, label_kind, r);
  if (lab >= cols) lab = -1;
  row_exp_scale<T>(logits + r * ld, dlogits + r * ld_out, cols, lse[r], gs, lab);
}

// Forward and backward in one pass over the logits (training with the gradient written in
// place): per row, max / sum (first read from DRAM), then loss, and the row is read again
// (from L2: 512-thread blocks keep the rows in flight under half of the L2 size) and overwritten
// with (softmax - onehot) * grad_scale.  Halves the DRAM traffic of separate forward + backward.
template <typename T>
__global__ void __launch_bounds__(512)
ce_fused_kernel(T* logits, int64_t ld, const void* __restrict__ labels, int label_kind,
                int64_t cols, float* __restrict__ lse, float* __restrict__ row_loss, int* err_flag,
                float grad_scale) {
  pdl_enter();
  __shared__ float sh_m[32], sh_s[32];
  const int64_t r = blockIdx.x;
  T* row = logits + r * ld;
  MaxSum ms = ms_block(row_maxsum<T>(row, cols), sh_m, sh_s);
  const float l = ms.m + __logf(ms.s);
  int64_t lab = read_label(labels, label_kind, r);
  const bool bad = lab < 0 || lab >= cols;
  if (threadIdx.x == 0) {
    lse[r] = l;
    if (bad) {
      if (err_flag && atomicOr(err_flag, 1) == 0) { err_flag[1] = (int)r; err_flag[2] = (int)lab; }
      row_loss[r] = 0.0f;
    } else {
      row_loss[r] = l - VecIO<T>::ld(row + lab);
    }
  }
  __syncthreads();   // the label's logit has been read before the row is overwritten
  row_exp_scale<T>(row, row, cols, l, grad_scale, bad ? -1 : lab);
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
pointwise_loss_bwd_kernel(const T* __restrict__ pred, const T* __restrict__ target, int64_t n,
                          float gscale, int mode, T* __restrict__ dpred) {
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n; i += nthreads) {
    float d = VecIO<T>::ld(pred + i) - VecIO<T>::ld(target + i);
    float g = mode == 0 ? 2.0f * d : (d > 0.0f ? 1.0f : (d < 0.0f ? -1.0f : 0.0f));
    VecIO<T>::st(dpred + i, g * gscale);
  }
}

}  // namespace

cudaError_t softmax_rows(int dtype, const void* in, void* out, int64_t rows, int64_t cols,
                         int64_t ld, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    softmax_rows_kernel<T><<<(unsigned)rows, THREADS, 0, s>>>((const T*)in, (T*)out, cols, ld);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

cudaError_t softmax_scores(void* sc, int64_t batch, int64_t rows, int64_t cols, int64_t ld,
                           int causal, cudaStream_t s) {
  const int64_t n_rows = batch * rows;
  if (n_rows <= 0) return cudaSuccess;
  softmax_scores_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, s>>>((__nv_bfloat16*)sc, n_rows,
                                                                     rows, cols, ld, causal);
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

cudaError_t softmax_scores_backward(const void* p, void* dp, int64_t n_rows, int64_t cols,
                                    int64_t ld, float scale, int causal, int64_t rows_per_batch,
                                    cudaStream_t s) {
  if (n_rows <= 0) return cudaSuccess;
  softmax_scores_bwd_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, s>>>(
      (const __nv_bfloat16*)p, (__nv_bfloat16*)dp, n_rows, rows_per_batch, cols, ld, scale, causal);
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

cudaError_t cross_entropy_forward(int dtype, const void* logits, int64_t ld, const void* labels,
                                  int label_kind, int64_t rows, int64_t cols, float* lse,
                                  float* row_loss, int* err_flag, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    launch_pdl(ce_forward_kernel<T>, dim3((unsigned)rows), dim3(THREADS), 0, s, (const T*)logits, ld,
               labels, label_kind, cols, lse, row_loss, err_flag);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

cudaError_t cross_entropy_fused(int dtype, void* logits, int64_t ld, const void* labels,
                                int label_kind, int64_t rows, int64_t cols, float* lse,
                                float* row_loss, int* err_flag, float grad_scale, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    launch_pdl(ce_fused_kernel<T>, dim3((unsigned)rows), dim3(512), 0, s, (T*)logits, ld, labels,
               label_kind, cols, lse, row_loss, err_flag, grad_scale);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

cudaError_t cross_entropy_backward(int dtype, const void* logits, int64_t ld, const void* labels,
                                   int label_kind, int64_t rows, int64_t cols, const float* lse,
                                   float grad_scale, const float* gs_dev, void* dlogits,
                                   int64_t ld_out, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    launch_pdl(ce_backward_kernel<T>, dim3((unsigned)rows), dim3(THREADS), 0, s, (const T*)logits, ld,
               labels, label_kind, cols, lse, grad_scale, gs_dev, (T*)dlogits, ld_out);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

cudaError_t pointwise_loss_backward(int mode, int dtype, const void* pred, const void* target,
                                    int64_t n, float grad_scale, void* dpred, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    pointwise_loss_bwd_kernel<T><<<stream_grid(n, THREADS), THREADS, 0, s>>>(
        (const T*)pred, (const T*)target, n, grad_scale / (float)n, mode, (T*)dpred);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

}  // namespace lt
