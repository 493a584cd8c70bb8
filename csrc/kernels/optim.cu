// Optimizer steps over flat parameter arenas: ONE launch updates every parameter of the
// model (fp32 master weights, fp32 moments, bf16 or fp32 gradient, optional bf16 shadow copy
// that the forward kernels read).  Per-tensor weight decay comes from a small segment table.
//
// The reference launches its Adam kernel once per parameter tensor
// (csrc/cuda/ops/fused.cu:132-174, lua/luatorch/optim/adam.lua:44-86) and has no fused SGD
// (lua/luatorch/optim/sgd.lua:33-56).  Update rule kept identical: decoupled decay
// p *= 1 - lr*wd first, then p -= lr * (m/bc1) / (sqrt(v/bc2) + eps).
#include "ops.h"
#include "common.cuh"

namespace lt {
namespace {

constexpr int THREADS = 256;

template <typename TG> __device__ __forceinline__ void load_grad4(const TG* g, float (&f)[4]);
template <> __device__ __forceinline__ void load_grad4<float>(const float* g, float (&f)[4]) {
  float4 v = *reinterpret_cast<const float4*>(g);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load_grad4<__nv_bfloat16>(const __nv_bfloat16* g,
                                                                      float (&f)[4]) {
  uint2 u = *reinterpret_cast<const uint2*>(g);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void store_shadow4(__nv_bfloat16* p, const float (&f)[4]) {
  uint2 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
  h[0] = __floats2bfloat162_rn(f[0], f[1]);
  h[1] = __floats2bfloat162_rn(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = u;
}

__device__ __forceinline__ int find_segment(const int64_t* seg_end, int nseg, int64_t i) {
  int lo = 0, hi = nseg - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (i < seg_end[mid]) hi = mid; else lo = mid + 1;
  }
  return lo;
}

__device__ __forceinline__ void apply_dyn(AdamArgs& a) {
  if (a.dyn) {
    a.lr = a.dyn[0];
    a.bc1 = a.dyn[1];
    a.bc2 = a.dyn[2];
  }
}

__device__ __forceinline__ void adam_update(float& p, float g, float& m, float& v, float wd,
                                            const AdamArgs& a) {
  p *= 1.0f - a.lr * wd;
  m = a.beta1 * m + (1.0f - a.beta1) * g;
  v = a.beta2 * v + (1.0f - a.beta2) * g * g;
  const float mh = m / a.bc1, vh = v / a.bc2;
  p -= a.lr * mh / (sqrtf(vh) + a.eps);
}

// n must be a multiple of 4 and segment boundaries multiples of 4 for the vector path;
// the launcher falls back to the scalar kernel otherwise.
template <typename TG>
__global__ void __launch_bounds__(THREADS)
adamw_vec_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ shadow,
                 const TG* __restrict__ grad, float* __restrict__ m, float* __restrict__ v,
                 int64_t n4, const int64_t* __restrict__ seg_end, const float* __restrict__ seg_wd,
                 int nseg, AdamArgs a) {
  pdl_enter();
  if (a.skip_flag && *a.skip_flag) return;
  apply_dyn(a);
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n4; i += nthreads) {
    const int64_t e = i * 4;
    const float wd = nseg > 0 ? seg_wd[find_segment(seg_end, nseg, e)] : 0.0f;
    float g[4];
    load_grad4<TG>(grad + e, g);
    float4 p4 = *reinterpret_cast<float4*>(master + e);
    float4 m4 = *reinterpret_cast<float4*>(m + e);
    float4 v4 = *reinterpret_cast<float4*>(v + e);
    float p[4] = {p4.x, p4.y, p4.z, p4.w};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) adam_update(p[j], g[j] * a.grad_scale, mm[j], vv[j], wd, a);
    *reinterpret_cast<float4*>(master + e) = make_float4(p[0], p[1], p[2], p[3]);
    *reinterpret_cast<float4*>(m + e) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(v + e) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (shadow) store_shadow4(shadow + e, p);
  }
}

template <typename TG>
__global__ void __launch_bounds__(THREADS)
adamw_scalar_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ shadow,
                    const TG* __restrict__ grad, float* __restrict__ m, float* __restrict__ v,
                    int64_t n, const int64_t* __restrict__ seg_end,
                    const float* __restrict__ seg_wd, int nseg, AdamArgs a) {
  if (a.skip_flag && *a.skip_flag) return;
  apply_dyn(a);
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n; i += nthreads) {
    const float wd = nseg > 0 ? seg_wd[find_segment(seg_end, nseg, i)] : 0.0f;
    float p = master[i], mm = m[i], vv = v[i];
    adam_update(p, VecIO<TG>::ld(grad + i) * a.grad_scale, mm, vv, wd, a);
    master[i] = p; m[i] = mm; v[i] = vv;
    if (shadow) shadow[i] = __float2bfloat16(p);
  }
}

template <typename TG>
__global__ void __launch_bounds__(THREADS)
sgd_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ shadow,
           const TG* __restrict__ grad, float* __restrict__ vel, int64_t n, float lr, float mu,
           int nesterov, float gscale, const float* __restrict__ dyn_lr) {
  if (dyn_lr) lr = *dyn_lr;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n; i += nthreads) {
    const float g = VecIO<TG>::ld(grad + i) * gscale;
    float p = master[i];
    if (vel) {
      const float vn = mu * vel[i] + g;
      vel[i] = vn;
      p -= lr * (nesterov ? mu * vn + g : vn);
    } else {
      p -= lr * g;
    }
    master[i] = p;
    if (shadow) shadow[i] = __float2bfloat16(p);
  }
}

__global__ void set_step_scalars_kernel(float* dyn, float lr, float bc1, float bc2,
                                        uint64_t* dyn_offset, uint64_t offset) {
  if (threadIdx.x != 0) return;
  if (dyn) {
    dyn[0] = lr;
    dyn[1] = bc1;
    dyn[2] = bc2;
  }
  if (dyn_offset) *dyn_offset = offset;
}

}  // namespace

cudaError_t set_step_scalars(float* dyn, float lr, float bc1, float bc2, uint64_t* dyn_offset,
                             uint64_t offset, cudaStream_t s) {
  set_step_scalars_kernel<<<1, 32, 0, s>>>(dyn, lr, bc1, bc2, dyn_offset, offset);
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

cudaError_t adamw_flat(float* master, void* shadow, const void* grad, int grad_dtype, float* m,
                       float* v, int64_t n, const int64_t* seg_end, const float* seg_wd, int nseg,
                       AdamArgs args, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const bool vec = n % 4 == 0 && is_aligned16(master) && is_aligned16(m) && is_aligned16(v) &&
                   (reinterpret_cast<uintptr_t>(grad) % (grad_dtype == DT_F32 ? 16 : 8) == 0) &&
                   (!shadow || reinterpret_cast<uintptr_t>(shadow) % 8 == 0);
  if (grad_dtype != DT_F32 && grad_dtype != DT_BF16) return cudaErrorInvalidValue;
  if (vec) {
    const int grid = stream_grid(n / 4, THREADS);
    if (grad_dtype == DT_F32)
      launch_pdl(adamw_vec_kernel<float>, dim3(grid), dim3(THREADS), 0, s, master,
                 (__nv_bfloat16*)shadow, (const float*)grad, m, v, n / 4, seg_end, seg_wd, nseg, args);
    else
      launch_pdl(adamw_vec_kernel<__nv_bfloat16>, dim3(grid), dim3(THREADS), 0, s, master,
                 (__nv_bfloat16*)shadow, (const __nv_bfloat16*)grad, m, v, n / 4, seg_end, seg_wd,
                 nseg, args);
  } else {
    const int grid = stream_grid(n, THREADS);
    if (grad_dtype == DT_F32)
      adamw_scalar_kernel<float><<<grid, THREADS, 0, s>>>(master, (__nv_bfloat16*)shadow,
                                                          (const float*)grad, m, v, n, seg_end,
                                                          seg_wd, nseg, args);
    else
      adamw_scalar_kernel<__nv_bfloat16><<<grid, THREADS, 0, s>>>(
          master, (__nv_bfloat16*)shadow, (const __nv_bfloat16*)grad, m, v, n, seg_end, seg_wd,
          nseg, args);
  }
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

cudaError_t sgd_flat(float* master, void* shadow, const void* grad, int grad_dtype, float* vel,
                     int64_t n, float lr, float momentum, int nesterov, float grad_scale,
                     cudaStream_t s, const float* dyn_lr) {
  if (n <= 0) return cudaSuccess;
  const int grid = stream_grid(n, THREADS);
  if (grad_dtype == DT_F32)
    sgd_kernel<float><<<grid, THREADS, 0, s>>>(master, (__nv_bfloat16*)shadow, (const float*)grad,
                                               vel, n, lr, momentum, nesterov, grad_scale,
                                               dyn_lr);
  else if (grad_dtype == DT_BF16)
    sgd_kernel<__nv_bfloat16><<<grid, THREADS, 0, s>>>(master, (__nv_bfloat16*)shadow,
                                                       (const __nv_bfloat16*)grad, vel, n, lr,
                                                       momentum, nesterov, grad_scale, dyn_lr);
  else
    return cudaErrorInvalidValue;
  LT_COUNT_LAUNCH();
  return cudaGetLastError();
}

}  // namespace lt
