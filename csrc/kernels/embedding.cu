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
    // status word, never a trap: [0] flag, [1] token position, [2] offending id (first seen)
    if (lane == 0 && err_flag && atomicOr(err_flag, 1) == 0) {
      err_flag[1] = (int)t;
      err_flag[2] = (int)id;
    }
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

// Exclusive scan of the bucket counts with independent CTAs: CTA k owns elements
// [1024 k, 1024 k + 1024); it first adds up everything before its tile (coalesced reads of at
// most 4 bytes x vocab from L2, all CTAs in parallel), then scans its own tile.  No CTA waits
// for another one, and the whole scan is one short launch instead of a serial single-CTA walk.
constexpr int SCAN_TILE = 1024;
__global__ void __launch_bounds__(SCAN_TILE)
scan_kernel(const int* __restrict__ counts, int64_t vocab, int* __restrict__ offsets,
            int* __restrict__ cursor) {
  __shared__ int sh_warp[32];
  __shared__ int sh_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t tile0 = (int64_t)blockIdx.x * SCAN_TILE;
  // ---- sum of all counts before this tile
  int before = 0;
  for (int64_t i = threadIdx.x; i < tile0; i += SCAN_TILE) before += counts[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
  if (lane == 0) sh_warp[warp] = before;
  __syncthreads();
  if (warp == 0) {
    int t = sh_warp[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) sh_base = t;
  }
  __syncthreads();
  const int base = sh_base;
  // ---- inclusive scan of the tile: warp shuffles, then the warp totals
  const int64_t idx = tile0 + threadIdx.x;
  const int mine = idx < vocab ? counts[idx] : 0;
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();                       // sh_warp is reused
  if (lane == 31) sh_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int t = sh_warp[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) t += u;
    }
    sh_warp[lane] = t;                   // inclusive totals of warps 0..lane
  }
  __syncthreads();
  const int excl = base + (warp > 0 ? sh_warp[warp - 1] : 0) + incl - mine;
  if (idx < vocab) {
    offsets[idx] = excl;
    cursor[idx] = excl;
  }
  if (idx == vocab - 1) offsets[vocab] = excl + mine;
}

__global__ void fill_kernel(const void* __restrict__ ids, int id_kind, int64_t n, int64_t vocab,
                            int* cursor, int* __restrict__ pos) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= n) return;
  const int64_t id = read_id(ids, id_kind, t);
  if (id >= 0 && id < vocab) pos[atomicAdd(&cursor[id], 1)] = (int)t;
}

template <typename TG, int V>
__device__ __forceinline__ void store_grad_vec(TG* p, const float (&f)[V]) {
  if constexpr (sizeof(TG) == 4) {
#pragma unroll
    for (int q = 0; q < V / 4; ++q)
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + 4 * q) =
          make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
  } else if constexpr (V == 8) {
    VecIO<TG>::store(p, f);      // one 16-byte store
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) VecIO<TG>::st(p + j, f[j]);
  }
}
template <typename TG, int V>
__device__ __forceinline__ void load_grad_vec(const TG* p, float (&f)[V]) {
  if constexpr (sizeof(TG) == 4) {
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + 4 * q);
      f[4 * q] = t.x; f[4 * q + 1] = t.y; f[4 * q + 2] = t.z; f[4 * q + 3] = t.w;
    }
  } else if constexpr (V == 8) {
    VecIO<TG>::load(p, f);
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) f[j] = VecIO<TG>::ld(p + j);
  }
}

// One warp per vocabulary row.  `vec`: dim is a multiple of the 16-byte vector of T and every
// base pointer is 16-byte aligned, so rows are read and written as 16-byte vectors (the
// table gradient is mostly rows of zeros: writing them at full width is what this kernel's
// time consists of).
template <typename T, typename TG>
__global__ void __launch_bounds__(256)
embedding_bwd_sum_kernel(const T* __restrict__ dy, const int* __restrict__ offsets,
                         const int* __restrict__ pos, int* __restrict__ pos_sorted,
                         TG* __restrict__ dtable, int accumulate, int64_t dim, int64_t vocab,
                         int vec) {
  constexpr int V = VecIO<T>::N;
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
  if (vec) {
    for (int64_t c0 = (int64_t)lane * V; c0 < dim; c0 += 32 * V) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.0f;
      for (int i = 0; i < cnt; ++i) {
        float t[V];
        VecIO<T>::load(dy + (int64_t)pos_sorted[b + i] * dim + c0, t);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += t[j];
      }
      if (accumulate) {
        float old[V];
        load_grad_vec<TG, V>(drow + c0, old);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += old[j];
      }
      store_grad_vec<TG, V>(drow + c0, acc);
    }
    return;
  }
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
  scan_kernel<<<(unsigned)((vocab + SCAN_TILE - 1) / SCAN_TILE), SCAN_TILE, 0, s>>>(
      ws.counts, vocab, ws.offsets, ws.cursor);
  LT_COUNT_LAUNCH();
  if (n_tokens > 0) {
    fill_kernel<<<(unsigned)((n_tokens + 255) / 256), 256, 0, s>>>(ids, id_kind, n_tokens, vocab,
                                                                   ws.cursor, ws.pos);
    LT_COUNT_LAUNCH();
  }
  LT_DISPATCH_DTYPE(dtype, T, {
    LT_DISPATCH_DTYPE(grad_dtype, TG, {
      const int vec = dim % VecIO<T>::N == 0 && is_aligned16(dy) && is_aligned16(dtable) &&
                      (dim * sizeof(TG)) % 16 == 0;
      embedding_bwd_sum_kernel<T, TG><<<(unsigned)((vocab + 7) / 8), 256, 0, s>>>(
          (const T*)dy, ws.offsets, ws.pos, ws.pos_sorted, (TG*)dtable, accumulate, dim, vocab, vec);
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
