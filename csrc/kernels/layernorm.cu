// LayerNorm forward / backward and GELU+bias forward / backward.
//
// Forward: one warp per row, the row is read ONCE into registers (16-byte vectors), mean
// and variance are reduced with warp shuffles, mean / rstd are saved for backward.  The
// reference kernel reads each row three times from global memory and has no backward at
// all (csrc/cuda/ops/fused.cu:63-127); its Lua LayerNorm backward walks elements on the
// CPU (lua/luatorch/nn/layernorm.lua:76-126).
// Backward: persistent warps walk rows (x and dy of a row stay in registers between the two
// passes, the next row's loads are issued before the current row's arithmetic), write dx
// (optionally adding an incoming residual gradient) and accumulate their dgamma / dbeta terms
// in registers; a CTA adds its warps in a fixed tree through shared memory and writes one
// partial row to scratch; a second, small kernel adds the CTA partials in a fixed order
// (many columns in parallel; doing this inside the first kernel left one CTA walking all
// partials while every other SM idled).  Every sum has a fixed order, so the result does not
// depend on timing.  (Rows that the vector path cannot address fall back to separate dx /
// partial kernels.)
#include "ops.h"
#include "common.cuh"

namespace lt {
namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int BWD_MAX_BLOCKS = 296;  // two CTAs per SM on a 148-SM part

template <typename TP> __device__ __forceinline__ float ldp(const TP* p, int64_t i) {
  return VecIO<TP>::ld(p + i);
}

// V consecutive parameters starting at element i (i a multiple of V, base 16-byte aligned)
template <typename TP, int V>
__device__ __forceinline__ void load_params(const TP* __restrict__ p, int64_t i, float (&f)[V]) {
  if constexpr (sizeof(TP) == 4) {
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      const float4 t = *reinterpret_cast<const float4*>(p + i + 4 * q);
      f[4 * q] = t.x; f[4 * q + 1] = t.y; f[4 * q + 2] = t.z; f[4 * q + 3] = t.w;
    }
  } else if constexpr (V == 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(p + i);
    VecIO<TP>::unpack(u, f);
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) f[j] = VecIO<TP>::ld(p + i + j);
  }
}

// ----------------------------------------------------------------------------- forward
// NV = 16-byte vectors per lane (row length <= 32 * NV * V elements).
template <typename T, typename TP, int NV>
__global__ void __launch_bounds__(THREADS)
ln_fwd_kernel(const T* __restrict__ x, const TP* __restrict__ gamma, const TP* __restrict__ beta,
              float eps, T* __restrict__ y, float* __restrict__ mean_out,
              float* __restrict__ rstd_out, int64_t rows, int64_t cols, int vec_params) {
  pdl_enter();
  constexpr int V = VecIO<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t nvec = cols / V;
  const T* xr = x + row * cols;
  float v[NV][V];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int64_t vi = lane + 32 * i;
    if (vi < nvec) {
      VecIO<T>::load(xr + vi * V, v[i]);
#pragma unroll
      for (int j = 0; j < V; ++j) sum += v[i][j];
    }
  }
  const float mean = warp_sum(sum) / (float)cols;
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < nvec) {
#pragma unroll
      for (int j = 0; j < V; ++j) { float d = v[i][j] - mean; sq += d * d; }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / (float)cols + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  T* yr = y + row * cols;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int64_t vi = lane + 32 * i;
    if (vi < nvec) {
      float o[V], ga[V], be[V];
      if (vec_params) {
        load_params<TP, V>(gamma, vi * V, ga);
        load_params<TP, V>(beta, vi * V, be);
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) { ga[j] = ldp(gamma, vi * V + j); be[j] = ldp(beta, vi * V + j); }
      }
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = (v[i][j] - mean) * rstd * ga[j] + be[j];
      VecIO<T>::store(yr + vi * V, o);
    }
  }
}

// Any row length / alignment: one CTA per row, scalar accesses.
template <typename T, typename TP>
__global__ void __launch_bounds__(THREADS)
ln_fwd_generic(const T* __restrict__ x, const TP* __restrict__ gamma, const TP* __restrict__ beta,
               float eps, T* __restrict__ y, float* __restrict__ mean_out,
               float* __restrict__ rstd_out, int64_t cols) {
  __shared__ float sh[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * cols;
  float s = 0.0f;
  for (int64_t c = threadIdx.x; c < cols; c += THREADS) s += VecIO<T>::ld(xr + c);
  const float mean = block_sum(s, sh) / (float)cols;
  float q = 0.0f;
  for (int64_t c = threadIdx.x; c < cols; c += THREADS) {
    float d = VecIO<T>::ld(xr + c) - mean;
    q += d * d;
  }
  const float rstd = rsqrtf(block_sum(q, sh) / (float)cols + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  for (int64_t c = threadIdx.x; c < cols; c += THREADS)
    VecIO<T>::st(y + row * cols + c,
                 (VecIO<T>::ld(xr + c) - mean) * rstd * ldp(gamma, c) + ldp(beta, c));
}

// ----------------------------------------------------------------------------- backward
// dx: one warp per row, the row's x and dy stay in registers between the two passes; no
// per-column state, so many warps are resident and enough loads are in flight to fill HBM.
template <typename T, typename TP, int NV>
__global__ void __launch_bounds__(THREADS)
ln_dx_kernel(const T* __restrict__ x, const T* __restrict__ dy, const TP* __restrict__ gamma,
             const float* __restrict__ mean, const float* __restrict__ rstd,
             const T* __restrict__ dx_add, T* __restrict__ dx, int64_t rows, int64_t cols) {
  pdl_enter();
  constexpr int V = VecIO<T>::N;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t nvec = cols / V;
  for (int64_t row = blockIdx.x * (int64_t)WARPS + warp; row < rows;
       row += (int64_t)gridDim.x * WARPS) {
    const T* xr = x + row * cols;
    const T* dyr = dy + row * cols;
    // x and dy stay in registers as loaded (16 bytes per vector) between the two passes
    uint4 xraw[NV], graw[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (vi < nvec) {
        xraw[i] = VecIO<T>::load_raw(xr + vi * V);
        graw[i] = VecIO<T>::load_raw(dyr + vi * V);
      }
    }
    const float mu = mean[row], rs = rstd[row];
    float c1 = 0.0f, c2 = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (vi < nvec) {
        float xv[V], g[V];
        VecIO<T>::unpack(xraw[i], xv);
        VecIO<T>::unpack(graw[i], g);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float gg = g[j] * ldp(gamma, vi * V + j);   // dy * gamma
          c1 += gg;
          c2 += gg * ((xv[j] - mu) * rs);
        }
      }
    }
    c1 = warp_sum(c1) / (float)cols;
    c2 = warp_sum(c2) / (float)cols;
    T* dxr = dx + row * cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (vi < nvec) {
        // the residual-stream gradient is fetched here, not with x and dy: keeping it in
        // registers across the reductions would cost a third row of registers per lane
        float o[V], xv[V], g[V];
        if (dx_add) VecIO<T>::load(dx_add + row * cols + vi * V, o);
        VecIO<T>::unpack(xraw[i], xv);
        VecIO<T>::unpack(graw[i], g);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float r = rs * (g[j] * ldp(gamma, vi * V + j) - c1 - (xv[j] - mu) * rs * c2);
          o[j] = dx_add ? o[j] + r : r;
        }
        VecIO<T>::store(dxr + vi * V, o);
      }
    }
  }
}

// dgamma / dbeta partial sums: block (column group of 32 x V columns, slab of rows); the
// eight warps stride over the slab's rows with independent loads (x and dy were just read by
// the dx kernel, so they mostly come from L2) and are folded in warp order, so the result
// does not depend on timing.  scratch[slab][0:cols] = sum dy * x_hat, [cols:2 cols] = sum dy.
template <typename T>
__global__ void __launch_bounds__(THREADS)
ln_stats_kernel(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ mean,
                const float* __restrict__ rstd, float* __restrict__ scratch, int64_t rows,
                int64_t cols, int64_t rows_per_slab) {
  pdl_enter();
  constexpr int V = VecIO<T>::N;
  __shared__ float sh[WARPS][2][32 * V + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t vi = blockIdx.x * 32 + lane;
  const bool ok = vi < cols / V;
  const int64_t r0 = blockIdx.y * rows_per_slab;
  const int64_t r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
  float dg[V], db[V];
#pragma unroll
  for (int j = 0; j < V; ++j) { dg[j] = 0.0f; db[j] = 0.0f; }
  if (ok) {
#pragma unroll 4
    for (int64_t row = r0 + warp; row < r1; row += WARPS) {
      float xv[V], dv[V];
      VecIO<T>::load(x + row * cols + vi * V, xv);
      VecIO<T>::load(dy + row * cols + vi * V, dv);
      const float mu = mean[row], rs = rstd[row];
#pragma unroll
      for (int j = 0; j < V; ++j) {
        dg[j] += dv[j] * ((xv[j] - mu) * rs);
        db[j] += dv[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) {
    sh[warp][0][lane * V + j] = dg[j];
    sh[warp][1][lane * V + j] = db[j];
  }
  __syncthreads();
  float* out = scratch + (int64_t)blockIdx.y * 2 * cols;
  for (int c = threadIdx.x; c < 2 * 32 * V; c += THREADS) {
    const int which = c / (32 * V), cc = c - which * 32 * V;
    const int64_t col = blockIdx.x * 32 * V + cc;
    if (col < cols) {
      float acc = 0.0f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) acc += sh[w][which][cc];
      out[which * cols + col] = acc;
    }
  }
}

constexpr int FB_WARPS = 4;                 // 128 threads, three CTAs per SM: up to 168 registers a thread
constexpr int FB_THREADS = FB_WARPS * 32;
constexpr int FB_MAX_BLOCKS = 3 * 148;

// Persistent warps: a warp walks rows blockIdx.x * 4 + warp, + gridDim.x * 4, ... and loads the
// NEXT row's x and dy before it works on the current one, so HBM reads, arithmetic and the dx
// stores of neighbouring rows overlap.  The dgamma / dbeta terms accumulate in registers over
// all of a warp's rows; at the end the CTA's four warps are added in a fixed binary tree
// through shared memory (1->0 and 3->2, then 2->0) and warp 0 writes the CTA's partial row to
// scratch.
// FULL: the row is exactly NV x 32 vectors long (cols == NV * 32 * V), so no lane ever falls
// off its end and the bounds tests disappear (768 columns of bf16: NV = 3).
template <typename T, typename TP, int NV, bool DXS, bool FULL>
__global__ void __launch_bounds__(FB_THREADS, (DXS && NV >= 3) ? 2 : 3)
ln_bwd_fused_kernel(const T* __restrict__ x, const T* __restrict__ dy, const TP* __restrict__ gamma,
                    const float* __restrict__ mean, const float* __restrict__ rstd,
                    const T* __restrict__ dx_add, T* __restrict__ dx, int64_t rows, int64_t cols,
                    float* __restrict__ scratch) {
  pdl_enter();
  constexpr int V = VecIO<T>::N;
  __shared__ float sh_fold[(FB_WARPS / 2) * (DXS ? 3 : 2) * 32 * VecIO<T>::N];   // [WARPS / 2][sets][32 lanes x V]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t nvec = cols / V;
  const int64_t stride = (int64_t)gridDim.x * FB_WARPS;
  // DXS: also the column sums of dx itself (the bias gradient of the linear layer whose output
  // this LayerNorm normalised), a third set of partial sums
  constexpr int NS = DXS ? 3 : 2;
  float dg[NV][V], db[NV][V], dxs[DXS ? NV : 1][V];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < V; ++j) {
      dg[i][j] = 0.0f; db[i][j] = 0.0f;
      if (DXS) dxs[i][j] = 0.0f;
    }

  int64_t row = blockIdx.x * (int64_t)FB_WARPS + warp;
  uint4 xraw[NV], graw[NV];
  float mu = 0.0f, rs = 0.0f;
  if (row < rows) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (FULL || vi < nvec) {
        xraw[i] = VecIO<T>::load_raw(x + row * cols + vi * V);
        graw[i] = VecIO<T>::load_raw(dy + row * cols + vi * V);
      }
    }
    mu = mean[row];
    rs = rstd[row];
  }
  while (row < rows) {
    // ---- the next row's loads go out before this row's arithmetic
    const int64_t nrow = row + stride;
    uint4 nx[NV], ng[NV];
    float nmu = 0.0f, nrs = 0.0f;
    if (nrow < rows) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int64_t vi = lane + 32 * i;
        if (FULL || vi < nvec) {
          nx[i] = VecIO<T>::load_raw(x + nrow * cols + vi * V);
          ng[i] = VecIO<T>::load_raw(dy + nrow * cols + vi * V);
        }
      }
      nmu = mean[nrow];
      nrs = rstd[nrow];
    }
    // this row's residual-stream gradient: requested now, consumed after the two reductions
    uint4 araw[NV];
    if (dx_add) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int64_t vi = lane + 32 * i;
        if (FULL || vi < nvec) araw[i] = VecIO<T>::load_raw(dx_add + row * cols + vi * V);
      }
    }
    float c1 = 0.0f, c2 = 0.0f;
    const float shift = -mu * rs;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (FULL || vi < nvec) {
        float xv[V], g[V], ga[V];
        VecIO<T>::unpack(xraw[i], xv);
        VecIO<T>::unpack(graw[i], g);
        load_params<TP, V>(gamma, vi * V, ga);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = fmaf(xv[j], rs, shift);
          const float gg = g[j] * ga[j];
          c1 += gg;
          c2 = fmaf(gg, xh, c2);
          dg[i][j] = fmaf(g[j], xh, dg[i][j]);
          db[i][j] += g[j];
        }
      }
    }
    c1 = warp_sum(c1) / (float)cols;
    c2 = warp_sum(c2) / (float)cols;
    T* dxr = dx + row * cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (FULL || vi < nvec) {
        float o[V], xv[V], g[V], ga[V];
        if (dx_add) VecIO<T>::unpack(araw[i], o);
        VecIO<T>::unpack(xraw[i], xv);
        VecIO<T>::unpack(graw[i], g);
        load_params<TP, V>(gamma, vi * V, ga);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = fmaf(xv[j], rs, shift);
          const float r = rs * (fmaf(g[j], ga[j], -c1) - xh * c2);
          o[j] = dx_add ? o[j] + r : r;
          if (DXS) dxs[i][j] += o[j];
        }
        VecIO<T>::store(dxr + vi * V, o);
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) { xraw[i] = nx[i]; graw[i] = ng[i]; }
    mu = nmu;
    rs = nrs;
    row = nrow;
  }

  // ---- fixed binary tree over the CTA's warps, one 16-byte vector slice at a time
  const int64_t rowlen = NS * cols;
  float* mine = scratch + (int64_t)blockIdx.x * rowlen;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int64_t vi = lane + 32 * i;
    const bool has = FULL || vi < nvec;
#pragma unroll
    for (int step = 1; step < FB_WARPS; step <<= 1) {
      float* slot = sh_fold + (warp / (2 * step)) * (NS * 32 * V);
      if ((warp & (2 * step - 1)) == step) {          // sender at this level
#pragma unroll
        for (int j = 0; j < V; ++j) {
          slot[j * 32 + lane] = dg[i][j];             // lanes hit consecutive words
          slot[32 * V + j * 32 + lane] = db[i][j];
          if (DXS) slot[2 * 32 * V + j * 32 + lane] = dxs[i][j];
        }
      }
      __syncthreads();
      if ((warp & (2 * step - 1)) == 0) {             // receiver
#pragma unroll
        for (int j = 0; j < V; ++j) {
          dg[i][j] += slot[j * 32 + lane];
          db[i][j] += slot[32 * V + j * 32 + lane];
          if (DXS) dxs[i][j] += slot[2 * 32 * V + j * 32 + lane];
        }
      }
      __syncthreads();
    }
    if (warp == 0 && has) {
      float4* pg = reinterpret_cast<float4*>(mine + vi * V);
      float4* pb = reinterpret_cast<float4*>(mine + cols + vi * V);
#pragma unroll
      for (int q = 0; q < V / 4; ++q) {
        pg[q] = make_float4(dg[i][4 * q], dg[i][4 * q + 1], dg[i][4 * q + 2], dg[i][4 * q + 3]);
        pb[q] = make_float4(db[i][4 * q], db[i][4 * q + 1], db[i][4 * q + 2], db[i][4 * q + 3]);
      }
      if (DXS) {
        float4* ps = reinterpret_cast<float4*>(mine + 2 * cols + vi * V);
#pragma unroll
        for (int q = 0; q < V / 4; ++q)
          ps[q] = make_float4(dxs[i][4 * q], dxs[i][4 * q + 1], dxs[i][4 * q + 2], dxs[i][4 * q + 3]);
      }
    }
  }
}

template <typename T, typename TP>
__global__ void __launch_bounds__(THREADS)
ln_bwd_generic(const T* __restrict__ x, const T* __restrict__ dy, const TP* __restrict__ gamma,
               const float* __restrict__ mean, const float* __restrict__ rstd,
               const T* __restrict__ dx_add, T* __restrict__ dx, int64_t cols) {
  __shared__ float sh[32];
  const int64_t row = blockIdx.x;
  const float mu = mean[row], rs = rstd[row];
  float c1 = 0.0f, c2 = 0.0f;
  for (int64_t c = threadIdx.x; c < cols; c += THREADS) {
    const float xh = (VecIO<T>::ld(x + row * cols + c) - mu) * rs;
    const float g = VecIO<T>::ld(dy + row * cols + c) * ldp(gamma, c);
    c1 += g; c2 += g * xh;
  }
  c1 = block_sum(c1, sh) / (float)cols;
  c2 = block_sum(c2, sh) / (float)cols;
  for (int64_t c = threadIdx.x; c < cols; c += THREADS) {
    const float xh = (VecIO<T>::ld(x + row * cols + c) - mu) * rs;
    const float g = VecIO<T>::ld(dy + row * cols + c) * ldp(gamma, c);
    float r = rs * (g - c1 - xh * c2);
    if (dx_add) r += VecIO<T>::ld(dx_add + row * cols + c);
    VecIO<T>::st(dx + row * cols + c, r);
  }
}

// dgamma / dbeta partials for the generic path: slab sums over 128 rows, thread per column.
template <typename T>
__global__ void __launch_bounds__(256)
ln_param_partials_generic(const T* __restrict__ x, const T* __restrict__ dy,
                          const float* __restrict__ mean, const float* __restrict__ rstd,
                          float* __restrict__ scratch, int64_t rows, int64_t cols,
                          int64_t rows_per_slab) {
  const int64_t c = blockIdx.x * 256ll + threadIdx.x;
  if (c >= cols) return;
  const int64_t r0 = blockIdx.y * rows_per_slab;
  const int64_t r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
  float g = 0.0f, b = 0.0f;
  for (int64_t r = r0; r < r1; ++r) {
    const float d = VecIO<T>::ld(dy + r * cols + c);
    g += d * (VecIO<T>::ld(x + r * cols + c) - mean[r]) * rstd[r];
    b += d;
  }
  scratch[(int64_t)blockIdx.y * 2 * cols + c] = g;
  scratch[(int64_t)blockIdx.y * 2 * cols + cols + c] = b;
}

// 32 columns x 32 partial-lanes per block: lane py adds partials py, py + 32, ... (independent
// loads, 128 bytes per warp and row), then the 32 lanes are folded in a fixed order.
template <typename TG>
__global__ void __launch_bounds__(1024)
ln_param_reduce(const float* __restrict__ scratch, int nparts, int64_t cols, int nsets,
                TG* __restrict__ dgamma, TG* __restrict__ dbeta, int accumulate,
                TG* __restrict__ dxsum, int dxsum_accumulate) {
  pdl_enter();
  __shared__ float sh[32][33];
  const int cx = threadIdx.x & 31, py = threadIdx.x >> 5;
  const int64_t c = blockIdx.x * 32ll + cx;
  const int64_t rowlen = (int64_t)nsets * cols;
  float t = 0.0f;
  if (c < rowlen) {
    // all of a lane's loads are requested before the first add (fixed order kept)
    for (int p0 = py; p0 < nparts; p0 += 32 * 16) {
      float v[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const int p = p0 + 32 * k;
        v[k] = p < nparts ? __ldcg(scratch + (int64_t)p * rowlen + c) : 0.0f;
      }
#pragma unroll
      for (int k = 0; k < 16; ++k) t += v[k];
    }
  }
  sh[py][cx] = t;
  __syncthreads();
  if (py == 0 && c < rowlen) {
    float r = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) r += sh[i][cx];
    TG* dst;
    int acc;
    if (c < cols) { dst = dgamma + c; acc = accumulate; }
    else if (c < 2 * cols) { dst = dbeta + (c - cols); acc = accumulate; }
    else { dst = dxsum + (c - 2 * cols); acc = dxsum_accumulate; }
    if (acc) r += VecIO<TG>::ld(dst);
    VecIO<TG>::st(dst, r);
  }
}

int bwd_blocks(int64_t rows) {
  int64_t need = (rows + WARPS - 1) / WARPS;
  return (int)(need < BWD_MAX_BLOCKS ? (need < 1 ? 1 : need) : BWD_MAX_BLOCKS);
}

template <typename T, typename TP>
cudaError_t ln_fwd_dispatch(const void* x, const void* gamma, const void* beta, float eps, void* y,
                            float* mean, float* rstd, int64_t rows, int64_t cols,
                            cudaStream_t s) {
  constexpr int V = VecIO<T>::N;
  const bool fast = cols % V == 0 && cols <= 32 * 8 * V && is_aligned16(x) && is_aligned16(y);
  const unsigned grid = (unsigned)((rows + WARPS - 1) / WARPS);
#define LT_LN_FWD(NVV)                                                                       \
  launch_pdl(ln_fwd_kernel<T, TP, NVV>, dim3(grid), dim3(THREADS), 0, s, (const T*)x,          \
             (const TP*)gamma, (const TP*)beta, eps, (T*)y, mean, rstd, rows, cols, vec_params)
  const int vec_params = is_aligned16(gamma) && is_aligned16(beta) ? 1 : 0;
  if (fast) {
    const int64_t per_lane = (cols / V + 31) / 32;
    if (per_lane <= 1) LT_LN_FWD(1);
    else if (per_lane <= 2) LT_LN_FWD(2);
    else if (per_lane <= 3) LT_LN_FWD(3);
    else if (per_lane <= 4) LT_LN_FWD(4);
    else LT_LN_FWD(8);
  } else {
    ln_fwd_generic<T, TP><<<(unsigned)rows, THREADS, 0, s>>>(
        (const T*)x, (const TP*)gamma, (const TP*)beta, eps, (T*)y, mean, rstd, cols);
  }
#undef LT_LN_FWD
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

template <typename T, typename TP>
cudaError_t ln_bwd_dispatch(const void* x, const void* dy, const void* gamma, const float* mean,
                            const float* rstd, const void* dx_add, void* dx, float* scratch,
                            int64_t rows, int64_t cols, int* nparts, bool want_dxsum,
                            bool* dxsum_done, cudaStream_t s) {
  constexpr int V = VecIO<T>::N;
  const bool fast = cols % V == 0 && cols <= 32 * 8 * V && is_aligned16(x) && is_aligned16(dy) &&
                    is_aligned16(dx) && (!dx_add || is_aligned16(dx_add));
  *dxsum_done = false;
  if (fast && cols <= 32 * 4 * V && is_aligned16(gamma)) {
    // one kernel: dx, dgamma and dbeta (rows up to 4 vectors per lane keep their parameter
    // sums in registers)
    const int64_t want = (rows + FB_WARPS - 1) / FB_WARPS;
    const unsigned grid = (unsigned)(want < FB_MAX_BLOCKS ? want : FB_MAX_BLOCKS);
    const size_t smem = 0;
#define LT_LN_FUSED(NVV, DXSV)                                                                \
  do {                                                                                           \
    if (full_ok && cols == (int64_t)(NVV) * 32 * V)                                                \
      launch_pdl(ln_bwd_fused_kernel<T, TP, NVV, DXSV, true>, dim3(grid), dim3(FB_THREADS), smem, s, \
                 (const T*)x, (const T*)dy, (const TP*)gamma, mean, rstd, (const T*)dx_add,       \
                 (T*)dx, rows, cols, scratch);                                                    \
    else                                                                                         \
      launch_pdl(ln_bwd_fused_kernel<T, TP, NVV, DXSV, false>, dim3(grid), dim3(FB_THREADS), smem, s, \
                 (const T*)x, (const T*)dy, (const TP*)gamma, mean, rstd, (const T*)dx_add,       \
                 (T*)dx, rows, cols, scratch);                                                    \
  } while (0)
    const int64_t per_lane = (cols / V + 31) / 32;
    static const bool full_ok = [] { const char* e = getenv("LT_LN_FULL"); return !(e && e[0] == '0'); }();
    const bool dxs = want_dxsum && per_lane <= 3;   // a third register set fits up to 3 vectors a lane
    if (dxs) {
      if (per_lane <= 1) LT_LN_FUSED(1, true);
      else if (per_lane <= 2) LT_LN_FUSED(2, true);
      else LT_LN_FUSED(3, true);
      *dxsum_done = true;
    } else {
      if (per_lane <= 1) LT_LN_FUSED(1, false);
      else if (per_lane <= 2) LT_LN_FUSED(2, false);
      else if (per_lane <= 3) LT_LN_FUSED(3, false);
      else LT_LN_FUSED(4, false);
    }
#undef LT_LN_FUSED
    LT_COUNT_LAUNCH();
    *nparts = (int)grid;     // one partial row per CTA; ln_param_reduce adds them in CTA order
    return cudaGetLastError();
  }
  if (fast) {
    const unsigned grid = (unsigned)((rows + WARPS - 1) / WARPS);
#define LT_LN_BWD(NVV)                                                                       \
  launch_pdl(ln_dx_kernel<T, TP, NVV>, dim3(grid), dim3(THREADS), 0, s, (const T*)x,           \
             (const T*)dy, (const TP*)gamma, mean, rstd, (const T*)dx_add, (T*)dx, rows, cols)
    const int64_t per_lane = (cols / V + 31) / 32;
    if (per_lane <= 1) LT_LN_BWD(1);
    else if (per_lane <= 2) LT_LN_BWD(2);
    else if (per_lane <= 3) LT_LN_BWD(3);
    else if (per_lane <= 4) LT_LN_BWD(4);
    else LT_LN_BWD(8);
#undef LT_LN_BWD
    LT_COUNT_LAUNCH();
    const int colgroups = (int)((cols / V + 31) / 32);
    int slabs = 4 * 148 / colgroups;
    if (slabs > BWD_MAX_BLOCKS) slabs = BWD_MAX_BLOCKS;
    if (slabs > 96) slabs = 96;   // the parameter reduction walks the slabs one after another
    if (slabs > bwd_blocks(rows)) slabs = bwd_blocks(rows);
    if (slabs < 1) slabs = 1;
    const int64_t rps = (rows + slabs - 1) / slabs;
    slabs = (int)((rows + rps - 1) / rps);
    *nparts = slabs;
    launch_pdl(ln_stats_kernel<T>, dim3((unsigned)colgroups, (unsigned)slabs), dim3(THREADS), 0, s,
               (const T*)x, (const T*)dy, mean, rstd, scratch, rows, cols, rps);
    LT_COUNT_LAUNCH();
  } else {
    ln_bwd_generic<T, TP><<<(unsigned)rows, THREADS, 0, s>>>(
        (const T*)x, (const T*)dy, (const TP*)gamma, mean, rstd, (const T*)dx_add, (T*)dx, cols);
    LT_COUNT_LAUNCH();
    const int slabs = bwd_blocks(rows);
    const int64_t rps = (rows + slabs - 1) / slabs;
    *nparts = slabs;
    dim3 g((unsigned)((cols + 255) / 256), (unsigned)slabs);
    ln_param_partials_generic<T><<<g, 256, 0, s>>>((const T*)x, (const T*)dy, mean, rstd, scratch,
                                                   rows, cols, rps);
    LT_COUNT_LAUNCH();
  }
  return cudaGetLastError();
}

// ----------------------------------------------------------------------------- gelu + bias
template <typename T, typename TP, bool BWD>
__global__ void __launch_bounds__(256)
gelu_bias_kernel(const T* __restrict__ x, const TP* __restrict__ bias, const T* __restrict__ dy,
                 T* __restrict__ out, int64_t rows, int64_t cols, int vec_ok) {
  constexpr int V = VecIO<T>::N;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec_ok) {
    const int64_t cv = cols / V, nvec = rows * cv;
    for (int64_t i = tid; i < nvec; i += nthreads) {
      const int64_t c = (i % cv) * V;
      float xv[V], dv[V];
      VecIO<T>::load(x + i * V, xv);
      if (BWD) VecIO<T>::load(dy + i * V, dv);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float z = xv[j] + (bias ? ldp(bias, c + j) : 0.0f);
        xv[j] = BWD ? dv[j] * dgelu_exact_tanh(z) : gelu_exact_tanh(z);
      }
      VecIO<T>::store(out + i * V, xv);
    }
  } else {
    const int64_t n = rows * cols;
    for (int64_t i = tid; i < n; i += nthreads) {
      const float z = VecIO<T>::ld(x + i) + (bias ? ldp(bias, i % cols) : 0.0f);
      VecIO<T>::st(out + i, BWD ? VecIO<T>::ld(dy + i) * dgelu_exact_tanh(z) : gelu_exact_tanh(z));
    }
  }
}

template <typename T, typename TP, bool BWD>
cudaError_t gelu_bias_launch(const void* x, const void* bias, const void* dy, void* out,
                             int64_t rows, int64_t cols, cudaStream_t s) {
  if (rows * cols <= 0) return cudaSuccess;
  const int vec_ok = cols % VecIO<T>::N == 0 && is_aligned16(x) && is_aligned16(out) &&
                     (!BWD || is_aligned16(dy));
  gelu_bias_kernel<T, TP, BWD><<<stream_grid(rows * cols / VecIO<T>::N + 1, 256), 256, 0, s>>>(
      (const T*)x, (const TP*)bias, (const T*)dy, (T*)out, rows, cols, vec_ok);
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

}  // namespace

cudaError_t layernorm_forward(int dtype, const void* x, const void* gamma, const void* beta,
                              int param_dtype, float eps, void* y, float* mean, float* rstd,
                              int64_t rows, int64_t cols, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    LT_DISPATCH_DTYPE(param_dtype, TP, {
      return ln_fwd_dispatch<T, TP>(x, gamma, beta, eps, y, mean, rstd, rows, cols, s);
    })
  })
  return cudaErrorInvalidValue;
}

int64_t layernorm_backward_scratch_floats(int64_t rows, int64_t cols) {
  (void)rows;
  return (int64_t)FB_MAX_BLOCKS * 3 * cols;   // one partial row (dgamma, dbeta, dx sums) per CTA
}

cudaError_t layernorm_backward(int dtype, const void* x, const void* dy, const void* gamma,
                               int param_dtype, const float* mean, const float* rstd,
                               const void* dx_add, void* dx, void* dgamma, void* dbeta,
                               int grad_dtype, int accumulate, float* scratch, int64_t rows,
                               int64_t cols, cudaStream_t s, void* dxsum, int dxsum_accumulate,
                               int* dxsum_done, int scratch_is_private) {
  if (dxsum_done) *dxsum_done = 0;
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  int nparts = 0;
  bool dxs_done = false;
  cudaError_t e = cudaErrorInvalidValue;
  if (grad_dtype != DT_F32 && grad_dtype != DT_BF16 && grad_dtype != DT_F16) return e;
  const bool want_dxsum = dxsum != nullptr && dgamma != nullptr && dbeta != nullptr;
  LT_DISPATCH_DTYPE(dtype, T, {
    LT_DISPATCH_DTYPE(param_dtype, TP, {
      e = ln_bwd_dispatch<T, TP>(x, dy, gamma, mean, rstd, dx_add, dx, scratch, rows, cols,
                                 &nparts, want_dxsum, &dxs_done, s);
    })
  })
  if (e != cudaSuccess) return e;
  if (dgamma && dbeta) {
    const int nsets = dxs_done ? 3 : 2;
    LT_DISPATCH_DTYPE(grad_dtype, TG, {
      launch_pdl(ln_param_reduce<TG>, dim3((unsigned)((nsets * cols + 31) / 32)), dim3(1024), 0, s,
                 scratch, nparts, cols, nsets, (TG*)dgamma, (TG*)dbeta, accumulate, (TG*)dxsum,
                 dxsum_accumulate);
      LT_COUNT_LAUNCH();
    })
    // dx is final before this reduction starts and nothing downstream reads what it writes:
    // the kernel launched next may run beside it (see mark_side_kernel in common.cuh)
    if (scratch_is_private) mark_side_kernel();
    if (dxsum_done) *dxsum_done = dxs_done ? 1 : 0;
  }
  return cudaGetLastError();
}

cudaError_t gelu_bias_forward(int dtype, const void* x, const void* bias, int bias_dtype,
                              void* out, int64_t rows, int64_t cols, cudaStream_t s) {
  LT_DISPATCH_DTYPE(dtype, T, {
    LT_DISPATCH_DTYPE(bias_dtype, TP, {
      return gelu_bias_launch<T, TP, false>(x, bias, nullptr, out, rows, cols, s);
    })
  })
  return cudaErrorInvalidValue;
}

cudaError_t gelu_bias_backward(int dtype, const void* x, const void* bias, int bias_dtype,
                               const void* dy, void* dx, int64_t rows, int64_t cols,
                               cudaStream_t s) {
  LT_DISPATCH_DTYPE(dtype, T, {
    LT_DISPATCH_DTYPE(bias_dtype, TP, {
      return gelu_bias_launch<T, TP, true>(x, bias, dy, dx, rows, cols, s);
    })
  })
  return cudaErrorInvalidValue;
}

}  // namespace lt
