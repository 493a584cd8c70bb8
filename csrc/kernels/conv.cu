// Convolution lowering on the GPU: im2col (patch matrix for the tensor-core GEMM), col2im
// (its adjoint, giving the gradient w.r.t. the convolution input that the reference never
// computes, lua/luatorch/nn/conv2d.lua:52-95) and the NHWC-flat <-> NCHW-flat re-layout
// needed to chain convolutions whose input is NCHW-flat and whose output is
// [batch*out_h*out_w, out_c].  The reference has only a CPU im2col (csrc/ops/conv2d.c:11-49).
#include "ops.h"
#include "common.cuh"

namespace lt {
namespace {

// cols[(b*oh*ow + oy*ow + ox), (c*k*k + ky*k + kx)] = in[b, c, oy*stride+ky-pad, ox*stride+kx-pad]
template <typename T>
__global__ void __launch_bounds__(256)
im2col_kernel(const T* __restrict__ in, T* __restrict__ cols, int batch, int C, int H, int W,
              int k, int stride, int pad, int oh, int ow, int64_t ld) {
  const int64_t patch = (int64_t)C * k * k;
  const int64_t total = (int64_t)batch * oh * ow * patch;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t col = i % patch, row = i / patch;
    const int kx = col % k, ky = (col / k) % k, c = col / (k * k);
    const int ox = row % ow, oy = (row / ow) % oh;
    const int64_t b = row / ((int64_t)ow * oh);
    const int iy = oy * stride + ky - pad, ix = ox * stride + kx - pad;
    T v = T(0.0f);
    if (iy >= 0 && iy < H && ix >= 0 && ix < W) v = in[((b * C + c) * H + iy) * W + ix];
    cols[row * ld + col] = v;
  }
}

// Same mapping, one 16-byte store per thread: a thread owns VecIO<T>::N consecutive columns
// of one cols row and walks (c, ky, kx) incrementally, so the index arithmetic is 32-bit and
// paid once per vector.  Needs ld % N == 0 and a 16-byte aligned cols; columns in
// [patch, ld) are written as zero.
template <typename T>
__global__ void __launch_bounds__(256)
im2col_vec_kernel(const T* __restrict__ in, T* __restrict__ cols, int batch, int C, int H, int W,
                  int k, int stride, int pad, int oh, int ow, int ld, int patch) {
  constexpr int V = VecIO<T>::N;
  const int vpr = ld / V;
  const int64_t total = (int64_t)batch * oh * ow * vpr;
  const int kk = k * k;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / vpr);
    const int col0 = (int)(i - (int64_t)row * vpr) * V;
    const int ox = row % ow, t = row / ow;
    const int oy = t % oh, b = t / oh;
    int c = col0 / kk, r = col0 - c * kk;
    int ky = r / k, kx = r - ky * k;
    const int iy0 = oy * stride - pad, ix0 = ox * stride - pad;
    const T* img = in + (int64_t)b * C * H * W;
    alignas(16) T v[V];
#pragma unroll
    for (int e = 0; e < V; ++e) {
      T x = T(0.0f);
      if (col0 + e < patch) {
        const int iy = iy0 + ky, ix = ix0 + kx;
        if (iy >= 0 && iy < H && ix >= 0 && ix < W) x = img[((int64_t)c * H + iy) * W + ix];
      }
      v[e] = x;
      if (++kx == k) { kx = 0; if (++ky == k) { ky = 0; ++c; } }
    }
    *reinterpret_cast<uint4*>(cols + (int64_t)row * ld + col0) = *reinterpret_cast<const uint4*>(v);
  }
}

// din[b, c, iy, ix] = sum over (ky, kx, oy, ox) hitting (iy, ix) of cols[row, col] (gather form:
// one thread per input element, no atomics, deterministic).
template <typename T>
__global__ void __launch_bounds__(256)
col2im_kernel(const T* __restrict__ cols, T* __restrict__ din, int batch, int C, int H, int W,
              int k, int stride, int pad, int oh, int ow, int64_t ld) {
  const int64_t total = (int64_t)batch * C * H * W;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int ix = i % W, iy = (i / W) % H, c = (i / ((int64_t)W * H)) % C;
    const int64_t b = i / ((int64_t)W * H * C);
    float acc = 0.0f;
    for (int ky = 0; ky < k; ++ky) {
      const int ty = iy + pad - ky;
      if (ty < 0 || ty % stride) continue;
      const int oy = ty / stride;
      if (oy >= oh) continue;
      for (int kx = 0; kx < k; ++kx) {
        const int tx = ix + pad - kx;
        if (tx < 0 || tx % stride) continue;
        const int ox = tx / stride;
        if (ox >= ow) continue;
        const int64_t row = (b * oh + oy) * ow + ox;
        const int64_t col = ((int64_t)c * k + ky) * k + kx;
        acc += VecIO<T>::ld(cols + row * ld + col);
      }
    }
    VecIO<T>::st(din + i, acc);
  }
}

// The same gather with the cols rows staged in shared memory: one block per (image, input
// row).  Only the <= k output rows oy that touch input row iy contribute; their ow * ld
// elements are contiguous in cols and come in with 16-byte loads, then every (c, ix) of the
// input row sums its <= k*k taps from shared memory (row stride padded by two elements so that
// neighbouring ox fall into different banks) and the stores run along ix.
// STRIDE_ / K_ > 0 fix the stride and the kernel size at compile time (the tap tests are
// divisions by the stride: shifts when it is a constant); 0 takes the run-time values.
template <typename T, int STRIDE_, int K_>
__global__ void __launch_bounds__(256)
col2im_rows_kernel(const T* __restrict__ cols, T* __restrict__ din, int C, int H, int W, int k_rt,
                   int stride_rt, int pad, int oh, int ow, int ld) {
  const int k = K_ > 0 ? K_ : k_rt;
  const int stride = STRIDE_ > 0 ? STRIDE_ : stride_rt;
  extern __shared__ __align__(16) unsigned char c2i_smem[];
  T* sm = reinterpret_cast<T*>(c2i_smem);
  constexpr int V = VecIO<T>::N;
  const int lds = ld + 2;
  const int iy = blockIdx.x % H, b = blockIdx.x / H;
  // slot ky holds output row oy = (iy + pad - ky) / stride when that is a valid row
  const int vpr = ld / V;
#pragma unroll
  for (int ky = 0; ky < k; ++ky) {
    const int ty = iy + pad - ky;
    if (ty < 0 || ty % stride || ty / stride >= oh) continue;
    const T* src = cols + ((int64_t)(b * oh + ty / stride) * ow) * ld;
    T* dst = sm + (int64_t)ky * ow * lds;
    for (int i = threadIdx.x; i < ow * vpr; i += blockDim.x) {
      const int ox = i / vpr, j = i - ox * vpr;
      const uint4 u = *reinterpret_cast<const uint4*>(src + (int64_t)ox * ld + j * V);
      uint32_t* d = reinterpret_cast<uint32_t*>(dst + ox * lds + j * V);   // 4-byte aligned
      d[0] = u.x; d[1] = u.y; d[2] = u.z; d[3] = u.w;
    }
  }
  __syncthreads();
  const int kk = k * k;
  for (int idx = threadIdx.x; idx < C * W; idx += blockDim.x) {
    const int c = idx / W, ix = idx - c * W;
    float acc = 0.0f;
#pragma unroll
    for (int ky = 0; ky < k; ++ky) {
      const int ty = iy + pad - ky;
      if (ty < 0 || ty % stride || ty / stride >= oh) continue;
      const T* rowp = sm + ky * ow * lds + c * kk + ky * k;
#pragma unroll
      for (int kx = 0; kx < k; ++kx) {
        const int tx = ix + pad - kx;
        if (tx < 0 || tx % stride) continue;
        const int ox = tx / stride;
        if (ox >= ow) continue;
        acc += VecIO<T>::ld(rowp + ox * lds + kx);
      }
    }
    VecIO<T>::st(din + (((int64_t)b * C + c) * H + iy) * W + ix, acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
relayout_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t batch, int64_t C,
                int64_t hw, int to_nchw) {
  // tiled transpose of the [hw, C] (NHWC) <-> [C, hw] (NCHW) plane of each image
  __shared__ T tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t b = blockIdx.z;
  const int64_t rows = to_nchw ? hw : C, cols_ = to_nchw ? C : hw;
  const T* src = in + b * C * hw;
  T* dst = out + b * C * hw;
  const int64_t c0 = blockIdx.x * 32ll, r0 = blockIdx.y * 32ll;
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    int64_t r = r0 + ty + i, c = c0 + tx;
    if (r < rows && c < cols_) tile[ty + i][tx] = src[r * cols_ + c];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    int64_t c = c0 + ty + i, r = r0 + tx;
    if (r < rows && c < cols_) dst[c * rows + r] = tile[tx][ty + i];
  }
}

}  // namespace

cudaError_t im2col(int dtype, const void* in, void* cols, int batch, int C, int H, int W, int k,
                   int stride, int pad, int64_t ld_cols, cudaStream_t s) {
  const int oh = (H + 2 * pad - k) / stride + 1, ow = (W + 2 * pad - k) / stride + 1;
  const int64_t total = (int64_t)batch * oh * ow * C * k * k;
  if (total <= 0) return cudaSuccess;
  const int64_t patch = (int64_t)C * k * k;
  LT_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = VecIO<T>::N;
    if (ld_cols % V == 0 && is_aligned16(cols) && (int64_t)batch * oh * ow < (1ll << 31) &&
        ld_cols < (1ll << 30)) {
      const int64_t vecs = (int64_t)batch * oh * ow * (ld_cols / V);
      im2col_vec_kernel<T><<<stream_grid(vecs, 256), 256, 0, s>>>(
          (const T*)in, (T*)cols, batch, C, H, W, k, stride, pad, oh, ow, (int)ld_cols, (int)patch);
    } else {
      im2col_kernel<T><<<stream_grid(total, 256), 256, 0, s>>>((const T*)in, (T*)cols, batch, C, H,
                                                              W, k, stride, pad, oh, ow, ld_cols);
    }
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

cudaError_t col2im(int dtype, const void* cols, void* din, int batch, int C, int H, int W, int k,
                   int stride, int pad, int64_t ld_cols, cudaStream_t s) {
  const int oh = (H + 2 * pad - k) / stride + 1, ow = (W + 2 * pad - k) / stride + 1;
  const int64_t total = (int64_t)batch * C * H * W;
  if (total <= 0) return cudaSuccess;
  LT_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = VecIO<T>::N;
    const size_t smem = (size_t)k * ow * (ld_cols + 2) * sizeof(T);
    // the staged form needs 16-byte rows and 4-byte aligned padded rows (ld even), and room
    if (ld_cols % V == 0 && is_aligned16(cols) && smem <= 160 * 1024 &&
        (int64_t)batch * H < (1ll << 31) && ld_cols < (1ll << 24)) {
      auto launch = [&](auto kern) -> cudaError_t {
        if (smem > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               160 * 1024);
          if (e != cudaSuccess) return e;
        }
        kern<<<(unsigned)(batch * H), 256, smem, s>>>((const T*)cols, (T*)din, C, H, W, k, stride,
                                                      pad, oh, ow, (int)ld_cols);
        return cudaSuccess;
      };
      cudaError_t le;
      if (k == 3 && stride == 1) le = launch(col2im_rows_kernel<T, 1, 3>);
      else if (k == 3 && stride == 2) le = launch(col2im_rows_kernel<T, 2, 3>);
      else le = launch(col2im_rows_kernel<T, 0, 0>);
      if (le != cudaSuccess) return le;
    } else {
      col2im_kernel<T><<<stream_grid(total, 256), 256, 0, s>>>((const T*)cols, (T*)din, batch, C, H,
                                                              W, k, stride, pad, oh, ow, ld_cols);
    }
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

cudaError_t nhwc_to_nchw(int dtype, const void* in, void* out, int batch, int C, int hw,
                         int to_nchw, cudaStream_t s) {
  if ((int64_t)batch * C * hw <= 0) return cudaSuccess;
  const int64_t rows = to_nchw ? hw : C, cols_ = to_nchw ? C : hw;
  dim3 grid((unsigned)((cols_ + 31) / 32), (unsigned)((rows + 31) / 32), (unsigned)batch);
  LT_DISPATCH_DTYPE(dtype, T, {
    relayout_kernel<T><<<grid, 256, 0, s>>>((const T*)in, (T*)out, batch, C, hw, to_nchw);
    LT_COUNT_LAUNCH();
    return cudaGetLastError();
  })
  return cudaErrorInvalidValue;
}

}  // namespace lt
