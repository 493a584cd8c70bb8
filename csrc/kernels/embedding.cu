// Embedding gather (+ fused positional add) and its deterministic scatter-add backward.
//
// The reference does both on the CPU with per-element Lua loops
// (lua/luatorch/nn/embedding.lua:34-82, lua/luatorch/nn/positional.lua:109-145).
// Backward here is a counting sort of the token ids (histogram -> exclusive scan -> bucket
// fill -> in-bucket rank) followed by one warp per vocabulary row summing its tokens'
// gradient rows in ascending token order with fp32 accumulation: no floating-point atomics,
// bitwise reproducible, and every row of the gradient table is written exactly once (so the
// table needs no separate zero fill).
#include "ops.h"
#include "common.cuh"

namespace lt {
namespace {

__device__ __forceinline__ int64_t read_id(const void* ids, int kind, int64_t t) {
  if (kind == 0) return ((const int64_t*)ids)[t];
  if (kind == 1) return ((const int*)ids)[t];
  return (int64_t)((const float*)ids)[t];
}

template <typename T>
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const T* __restrict__ table, const void* __restrict__ ids, int id_kind,
                     const T* __restrict__ pos_table, int64_t seq_len, T* __restrict__ out,
                     int64_t n_tokens, int64_t dim, int64_t vocab, int* err_flag, int vec_ok) {
  constexpr int V = VecIO<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x * 8ll + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  int64_t id = read_id(ids, id_kind, t);
  if (id < 0 || id >= vocab) {
    if (lane == 0 && err_flag) atomicOr(err_flag, 1);
    id = 0;
  }
  const T* src = table + id * dim;
  const T* pe = pos_table ? pos_table + (t % seq_len) * dim : nullptr;
  T* dst = out + t * dim;
  if (vec_ok) {
    for (int64_t i = lane; i < dim / V; i += 32) {
      float a[V];
      VecIO<T>::load(src + i * V, a);
      if (pe) {
        float b[V];
        VecIO<T>::load(pe + i * V, b);
#pragma unroll
        for (int j = 0; j < V; ++j) a[j] += b[j];
      }
      VecIO<T>::store(dst + i * V, a);
    }
  } else {
    for (int64_t i = lane; i < dim; i += 32)
      VecIO<T>::st(dst + i, VecIO<T>::ld(src + i) + (pe ? VecIO<T>::ld(pe + i) : 0.0f));
  }
}

struct BwdWs {
  int* counts;    // [vocab]
  int* offsets;   // [vocab + 1]
  int* cursor;    // [vocab]
  int* pos;       // [n_tokens] bucketed, unordered inside a bucket
  int* pos_sorted;  // [n_tokens]
};

__global__ void hist_kernel(const void* __restrict__ ids, int id_kind, int64_t n, int64_t vocab,
                            int* counts) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= n) return;
  const int64_t id = read_id(ids, id_kind, t);
  if (id >= 0 && id < vocab) atomicAdd(&counts[id], 1);
}

// Single-CTA exclusive scan (1024 threads, contiguous chunk per thread).
__global__ void __launch_bounds__(1024)
scan_kernel(const int* __restrict__ counts, int64_t vocab, int* __restrict__ offsets,
            int* __restrict__ cursor) {
  __shared__ int sh[1024];
  const int64_t per = (vocab + 1023) / 1024;
  const int64_t b = threadIdx.x * per, e = b + per < vocab ? b + per : vocab;
  int local = 0;
  for (int64_t i = b; i < e; ++i) local += counts[i];
  sh[threadIdx.x] = local;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    int v = threadIdx.x >= o ? sh[threadIdx.x - o] : 0;
    __syncthreads();
    sh[threadIdx.x] += v;
    __syncthreads();
  }
  int run = sh[threadIdx.x] - local;  // exclusive prefix of this chunk
  for (int64_t i = b; i < e; ++i) {
    offsets[i] = run;
    cursor[i] = run;
    run += counts[i];
  }
  if (threadIdx.x == 1023) offsets[vocab] = sh[1023];
}

__global__ void fill_kernel(const void* __restrict__ ids, int id_kind, int64_t n, int64_t vocab,
                            int* cursor, int* __restrict__ pos) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= n) return;
  const int64_t id = read_id(ids, id_kind, t);
  if (id >= 0 && id < vocab) pos[atomicAdd(&cursor[id], 1)] = (int)t;
}

template <typename T, typename TG>
__global__ void __launch_bounds__(256)
embedding_bwd_sum_kernel(const T* __restrict__ dy, const int* __restrict__ offsets,
                         const int* __restrict__ pos, int* __restrict__ pos_sorted,
                         TG* __restrict__ dtable, int accumulate, int64_t dim, int64_t vocab) {
  const int lane = threadIdx.x & 31;
  const int64_t v = blockIdx.x * 8ll + (threadIdx.x >> 5);
  if (v >= vocab) return;
  const int b = offsets[v], e = offsets[v + 1], cnt = e - b;
  // rank every token of the bucket by position => ascending, reproducible order
  for (int i = lane; i < cnt; i += 32) {
    const int p = pos[b + i];
    int rank = 0;
    for (int j = 0; j < cnt; ++j) rank += pos[b + j] < p;
    pos_sorted[b + rank] = p;
  }
  __syncwarp();
  TG* drow = dtable + v * dim;
  for (int64_t c0 = lane; c0 < dim; c0 += 32) {
    float acc = 0.0f;
    for (int i = 0; i < cnt; ++i) acc += VecIO<T>::ld(dy + (int64_t)pos_sorted[b + i] * dim + c0);
    if (accumulate) acc += VecIO<TG>::ld(drow + c0);
    VecIO<TG>::st(drow + c0, acc);
  }
}

template <typename T, typename TG>
__global__ void __launch_bounds__(256)
positional_bwd_kernel(const T* __restrict__ dy, TG* __restrict__ dpos, int accumulate,
                      int64_t batch, int64_t seq_len, int64_t max_seq, int64_t dim) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= max_seq * dim) return;
  const int64_t p = i / dim, c = i % dim;
  float acc = 0.0f;
  if (p < seq_len)
    for (int64_t b = 0; b < batch; ++b) acc += VecIO<T>::ld(dy + (b * seq_len + p) * dim + c);
  if (accumulate) acc += VecIO<TG>::ld(dpos + i);
  VecIO<TG>::st(dpos + i, acc);
}

size_t align_up(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace

cudaError_t embedding_forward(int dtype, const void* table, const void* ids, int id_kind,
                              const void* pos_table, int64_t seq_len, void* out, int64_t n_tokens,
                              int64_t dim, int64_t vocab, int* err_flag, cudaStream_t s) {
  if (n_tokens <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    const int vec_ok = dim % VecIO<T>::N == 0 && is_aligned16(table) && is_aligned16(out) &&
                       (!pos_table || is_aligned16(pos_table));
    embedding_fwd_kernel<T><<<(unsigned)((n_tokens + 7) / 8), 256, 0, s>>>(
        (const T*)table, ids, id_kind, (const T*)pos_table, seq_len, (T*)out, n_tokens, dim, vocab,
        err_flag, vec_ok);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

size_t embedding_backward_workspace(int64_t n_tokens, int64_t vocab) {
  return align_up(vocab * 4) + align_up((vocab + 1) * 4) + align_up(vocab * 4) +
         2 * align_up(n_tokens * 4);
}

cudaError_t embedding_backward(int dtype, const void* dy, const void* ids, int id_kind,
                               void* dtable, int grad_dtype, int accumulate, int64_t n_tokens,
                               int64_t dim, int64_t vocab, void* workspace, cudaStream_t s) {
  if (vocab <= 0) return cudaSuccess;
  char* w = (char*)workspace;
  BwdWs ws;
  ws.counts = (int*)w; w += align_up(vocab * 4);
  ws.offsets = (int*)w; w += align_up((vocab + 1) * 4);
  ws.cursor = (int*)w; w += align_up(vocab * 4);
  ws.pos = (int*)w; w += align_up(n_tokens * 4);
  ws.pos_sorted = (int*)w;
  cudaError_t e = cudaMemsetAsync(ws.counts, 0, vocab * 4, s);
  if (e != cudaSuccess) return e;
  if (n_tokens > 0) {
    hist_kernel<<<(unsigned)((n_tokens + 255) / 256), 256, 0, s>>>(ids, id_kind, n_tokens, vocab,
                                                                   ws.counts);
    LT_COUNT_LAUNCH();
  }
  scan_kernel<<<1, 1024, 0, s>>>(ws.counts, vocab, ws.offsets, ws.cursor);
  LT_COUNT_LAUNCH();
  if (n_tokens > 0) {
    fill_kernel<<<(unsigned)((n_tokens + 255) / 256), 256, 0, s>>>(ids, id_kind, n_tokens, vocab,
                                                                   ws.cursor, ws.pos);
    LT_COUNT_LAUNCH();
  }
  LT_DISPATCH_DTYPE(dtype, T, {
    LT_DISPATCH_DTYPE(grad_dtype, TG, {
      embedding_bwd_sum_kernel<T, TG><<<(unsigned)((vocab + 7) / 8), 256, 0, s>>>(
          (const T*)dy, ws.offsets, ws.pos, ws.pos_sorted, (TG*)dtable, accumulate, dim, vocab);
      LT_COUNT_LAUNCH();
    })
  })
  return cudaGetLastError();
}

cudaError_t positional_backward(int dtype, const void* dy, void* dpos, int grad_dtype,
                                int accumulate, int64_t batch, int64_t seq_len, int64_t max_seq,
                                int64_t dim, cudaStream_t s) {
  if (max_seq * dim <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    LT_DISPATCH_DTYPE(grad_dtype, TG, {
      positional_bwd_kernel<T, TG><<<(unsigned)((max_seq * dim + 255) / 256), 256, 0, s>>>(
          (const T*)dy, (TG*)dpos, accumulate, batch, seq_len, max_seq, dim);
      LT_COUNT_LAUNCH();
    })
  })
  return cudaGetLastError();
}

}  // namespace lt
