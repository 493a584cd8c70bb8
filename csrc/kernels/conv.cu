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
  LT_DISPATCH_DTYPE(dtype, T, {
    im2col_kernel<T><<<stream_grid(total, 256), 256, 0, s>>>((const T*)in, (T*)cols, batch, C, H,
                                                            W, k, stride, pad, oh, ow, ld_cols);
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
    col2im_kernel<T><<<stream_grid(total, 256), 256, 0, s>>>((const T*)cols, (T*)din, batch, C, H,
                                                            W, k, stride, pad, oh, ow, ld_cols);
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
