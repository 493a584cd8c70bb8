// GPU half of the C ABI: device runtime (transfers, allocation) and every tensor_*_cuda op,
// implemented on the sm_100a kernels of csrc/kernels (counterpart of the reference's
// csrc/cuda/tensor.cu and csrc/cuda/ops/*.cu).
//
// Differences from the reference that matter:
//   * matmul / bmm run on the tensor cores: each fp32 operand is split into bf16 hi + lo
//     parts and a_hi*b_hi + a_hi*b_lo + a_lo*b_hi is evaluated as ONE tcgen05 GEMM over a 3x
//     longer K (fp32 accumulation), which keeps fp32-level accuracy without cuBLAS SGEMM;
//   * reductions and losses are single launches whose only host interaction is the final
//     4-byte read the ABI's `float` return type demands (the reference does a cudaMalloc +
//     copy + host loop + cudaFree per call);
//   * async transfers stage through pinned memory on a dedicated stream and really overlap;
//   * flash attention covers head_dim 64 and 128 (other sizes use tensor-core GEMMs + the
//     fused score softmax), where the reference kernel cannot launch at 128.
#include "luatorch_abi.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <vector>

#include "../kernels/attention.h"
#include "../kernels/gemm.h"
#include "../kernels/ops.h"

extern "C" Tensor* lt_tensor_new_meta(const int64_t* shape, int ndim, int dtype);
extern "C" void pool_free_async(void* ptr, void* stream);

namespace {

constexpr cudaStream_t kStream = 0;   // ABI ops run in order on the default stream

Tensor* fail(const char* what, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess) fprintf(stderr, "luatorch cuda error in %s: %s\n", what, cudaGetErrorString(e));
  else fprintf(stderr, "luatorch error: %s\n", what);
  return nullptr;
}
bool dev(Tensor* t) { return t && t->cuda_data; }

Tensor* gpu_tensor(const int64_t* shape, int ndim, int dtype = DTYPE_FLOAT32) {
  Tensor* t = lt_tensor_new_meta(shape, ndim, dtype);
  if (!t) return nullptr;
  const size_t bytes = (size_t)(t->numel > 0 ? t->numel : 1) * sizeof(float);
  t->cuda_data = (float*)pool_alloc(bytes);
  if (!t->cuda_data) { tensor_free(t); return nullptr; }
  t->device = DEVICE_CUDA;
  return t;
}
Tensor* gpu_like(Tensor* a) { return gpu_tensor(a->shape, a->ndim, a->dtype); }

struct Scratch {   // device scratch that lives as long as the library
  void* reduce = nullptr;
  float* result = nullptr;
  int* flag = nullptr;
};
Scratch& scratch() {
  static Scratch s[64];
  int d = 0;
  cudaGetDevice(&d);
  Scratch& x = s[d & 63];
  if (!x.reduce) {
    x.reduce = pool_alloc(lt::reduce_scratch_bytes());
    cudaMemsetAsync(x.reduce, 0, lt::reduce_scratch_bytes(), kStream);
    x.result = (float*)pool_alloc(512);
    x.flag = (int*)pool_alloc(512);
  }
  return x;
}
float read_result() {
  float v = 0.0f;
  cudaMemcpyAsync(&v, scratch().result, sizeof(float), cudaMemcpyDeviceToHost, kStream);
  cudaStreamSynchronize(kStream);
  return v;
}

cudaStream_t g_xfer = nullptr;
std::mutex g_xfer_mu;
std::vector<void*> g_pinned_pending;
cudaStream_t xfer_stream() {
  std::lock_guard<std::mutex> lock(g_xfer_mu);
  if (!g_xfer) cudaStreamCreateWithFlags(&g_xfer, cudaStreamNonBlocking);
  return g_xfer;
}

template <typename F> Tensor* unary_like(Tensor* a, const char* name, F launch) {
  if (!dev(a)) return fail("null or non-cuda tensor");
  Tensor* o = gpu_like(a);
  if (!o) return nullptr;
  cudaError_t e = launch(o);
  if (e != cudaSuccess) { tensor_free(o); return fail(name, e); }
  return o;
}
Tensor* binary(int op, Tensor* a, Tensor* b, const char* name) {
  if (!dev(a) || !dev(b)) return fail("null or non-cuda tensor");
  if (a->numel != b->numel) {
    fprintf(stderr, "luatorch error: %s size mismatch (%lld vs %lld)\n", name, (long long)a->numel, (long long)b->numel);
    return nullptr;
  }
  return unary_like(a, name, [&](Tensor* o) {
    return lt::binary_op(op, lt::DT_F32, a->cuda_data, b->cuda_data, o->cuda_data, a->numel, kStream);
  });
}
Tensor* scalar(int op, Tensor* a, float s, const char* name) {
  return unary_like(a, name, [&](Tensor* o) {
    return lt::scalar_op(op, lt::DT_F32, a->cuda_data, s, o->cuda_data, a->numel, kStream);
  });
}
Tensor* unary(int op, Tensor* a, const char* name) {
  return unary_like(a, name, [&](Tensor* o) {
    return lt::unary_op(op, lt::DT_F32, a->cuda_data, o->cuda_data, a->numel, kStream);
  });
}
float reduce(int op, Tensor* a, float scale) {
  if (!dev(a) || a->numel <= 0) return 0.0f;
  Scratch& s = scratch();
  if (lt::reduce_all(op, lt::DT_F32, a->cuda_data, a->numel, scale, s.result, s.reduce, kStream) != cudaSuccess)
    return 0.0f;
  return read_result();
}

// ---- fp32-accurate GEMM on bf16 tensor cores: [hi | hi | lo] x [hi ; lo ; hi] ------------
__global__ void split_a_kernel(const float* __restrict__ a, __nv_bfloat16* __restrict__ out,
                               long long rows, long long K, long long ld) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= rows * K) return;
  const long long r = i / K, k = i % K;
  const float x = a[i];
  const __nv_bfloat16 hi = __float2bfloat16(x);
  const __nv_bfloat16 lo = __float2bfloat16(x - __bfloat162float(hi));
  __nv_bfloat16* row = out + r * ld;
  row[k] = hi; row[K + k] = hi; row[2 * K + k] = lo;
}
__global__ void split_b_kernel(const float* __restrict__ b, __nv_bfloat16* __restrict__ out,
                               long long K, long long N, long long ld) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= K * N) return;
  const long long k = i / N, n = i % N;
  const float x = b[i];
  const __nv_bfloat16 hi = __float2bfloat16(x);
  const __nv_bfloat16 lo = __float2bfloat16(x - __bfloat162float(hi));
  out[k * ld + n] = hi; out[(K + k) * ld + n] = lo; out[(2 * K + k) * ld + n] = hi;
}
long long pad8(long long v) { return (v + 7) / 8 * 8; }

cudaError_t gemm_fp32(const float* A, const float* B, float* C, long long batch, long long M,
                      long long K, long long N) {
  const long long lda = pad8(3 * K), ldb = pad8(N);
  __nv_bfloat16* a3 = (__nv_bfloat16*)pool_alloc((size_t)(batch * M * lda) * 2);
  __nv_bfloat16* b3 = (__nv_bfloat16*)pool_alloc((size_t)(batch * 3 * K * ldb) * 2);
  if (!a3 || !b3) return cudaErrorMemoryAllocation;
  if (lda != 3 * K) cudaMemsetAsync(a3, 0, (size_t)(batch * M * lda) * 2, kStream);
  if (ldb != N) cudaMemsetAsync(b3, 0, (size_t)(batch * 3 * K * ldb) * 2, kStream);
  for (long long i = 0; i < batch; ++i) {
    split_a_kernel<<<(unsigned)((M * K + 255) / 256), 256, 0, kStream>>>(A + i * M * K, a3 + i * M * lda, M, K, lda);
    split_b_kernel<<<(unsigned)((K * N + 255) / 256), 256, 0, kStream>>>(B + i * K * N, b3 + i * 3 * K * ldb, K, N, ldb);
  }
  lt::GemmArgs g;
  g.M = (int)M; g.N = (int)N; g.K = (int)(3 * K);
  g.A = a3; g.B = b3; g.C = C;
  g.lda = lda; g.ldb = ldb; g.ldc = N;
  g.a_mn_major = 0; g.b_mn_major = 1;
  g.batch_inner = (int)batch; g.batch_outer = 1;
  g.a_stride_inner = M * lda; g.b_stride_inner = 3 * K * ldb; g.c_stride_inner = M * N;
  g.c_fp32 = 1;
  cudaError_t e = lt::gemm_bf16(g, kStream);
  pool_free_async(a3, kStream);
  pool_free_async(b3, kStream);
  return e;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ device runtime
Tensor* tensor_to_cuda(Tensor* t) {
  if (!t) return nullptr;
  if (t->cuda_data) return t;
  const size_t bytes = (size_t)(t->numel > 0 ? t->numel : 1) * sizeof(float);
  float* d = (float*)pool_alloc(bytes);
  if (!d) return nullptr;
  cudaError_t e = cudaMemcpy(d, t->data, (size_t)t->numel * sizeof(float), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) { pool_free(d); return fail("tensor_to_cuda", e); }
  free(t->data);
  t->data = nullptr;
  t->cuda_data = d;
  t->device = DEVICE_CUDA;
  return t;
}

Tensor* tensor_to_cpu(Tensor* t) {
  if (!t) return nullptr;
  if (!t->cuda_data) return t;
  float* h = (float*)malloc((size_t)(t->numel > 0 ? t->numel : 1) * sizeof(float));
  if (!h) return fail("out of host memory");
  cudaError_t e = cudaMemcpy(h, t->cuda_data, (size_t)t->numel * sizeof(float), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { free(h); return fail("tensor_to_cpu", e); }
  pool_free(t->cuda_data);
  t->cuda_data = nullptr;
  t->data = h;
  t->device = DEVICE_CPU;
  return t;
}

// Async upload: the host buffer is copied into pinned staging memory, the copy runs on the
// transfer stream and the default stream waits on its event, so later ops are ordered after
// the copy without a host synchronise.
Tensor* tensor_to_cuda_async(Tensor* t) {
  if (!t) return nullptr;
  if (t->cuda_data) return t;
  const size_t bytes = (size_t)(t->numel > 0 ? t->numel : 1) * sizeof(float);
  float* d = (float*)pool_alloc(bytes);
  void* pinned = nullptr;
  if (!d || cudaMallocHost(&pinned, bytes) != cudaSuccess) {
    if (d) pool_free(d);
    return tensor_to_cuda(t);            // no pinned memory available: synchronous path
  }
  memcpy(pinned, t->data, (size_t)t->numel * sizeof(float));
  cudaStream_t xs = xfer_stream();
  cudaMemcpyAsync(d, pinned, (size_t)t->numel * sizeof(float), cudaMemcpyHostToDevice, xs);
  cudaEvent_t ev;
  cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  cudaEventRecord(ev, xs);
  cudaStreamWaitEvent(kStream, ev, 0);
  cudaEventDestroy(ev);
  { std::lock_guard<std::mutex> lock(g_xfer_mu); g_pinned_pending.push_back(pinned); }
  free(t->data);
  t->data = nullptr;
  t->cuda_data = d;
  t->device = DEVICE_CUDA;
  return t;
}

// Async download into pinned memory; tensor_sync() must be called before the data is read.
Tensor* tensor_to_cpu_async(Tensor* t) {
  if (!t) return nullptr;
  if (!t->cuda_data) return t;
  const size_t bytes = (size_t)(t->numel > 0 ? t->numel : 1) * sizeof(float);
  float* h = (float*)malloc(bytes);
  if (!h) return fail("out of host memory");
  cudaHostRegister(h, bytes, cudaHostRegisterDefault);
  cudaStream_t xs = xfer_stream();
  cudaEvent_t ev;
  cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  cudaEventRecord(ev, kStream);
  cudaStreamWaitEvent(xs, ev, 0);        // the copy starts after the producing kernels
  cudaEventDestroy(ev);
  cudaMemcpyAsync(h, t->cuda_data, (size_t)t->numel * sizeof(float), cudaMemcpyDeviceToHost, xs);
  pool_free_async(t->cuda_data, xs);
  { std::lock_guard<std::mutex> lock(g_xfer_mu); g_pinned_pending.push_back((void*)((uintptr_t)h | 1)); }
  t->cuda_data = nullptr;
  t->data = h;
  t->device = DEVICE_CPU;
  return t;
}

void tensor_sync(void) {
  if (g_xfer) cudaStreamSynchronize(g_xfer);
  std::lock_guard<std::mutex> lock(g_xfer_mu);
  for (void* p : g_pinned_pending) {
    if ((uintptr_t)p & 1) cudaHostUnregister((void*)((uintptr_t)p & ~(uintptr_t)1));   // registered user buffer
    else cudaFreeHost(p);
  }
  g_pinned_pending.clear();
}

Tensor* tensor_new_cuda(int64_t* shape, int ndim, int dtype) {
  Tensor* t = gpu_tensor(shape, ndim, dtype);
  if (!t) return nullptr;
  cudaMemsetAsync(t->cuda_data, 0, (size_t)(t->numel > 0 ? t->numel : 1) * sizeof(float), kStream);
  return t;
}

void tensor_cuda_free(Tensor* t) {
  if (t && t->cuda_data) {
    pool_free(t->cuda_data);
    t->cuda_data = nullptr;
  }
}

// ------------------------------------------------------------------ elementwise family
Tensor* tensor_add_cuda(Tensor* a, Tensor* b) { return binary(lt::BIN_ADD, a, b, "add"); }
Tensor* tensor_sub_cuda(Tensor* a, Tensor* b) { return binary(lt::BIN_SUB, a, b, "sub"); }
Tensor* tensor_mul_cuda(Tensor* a, Tensor* b) { return binary(lt::BIN_MUL, a, b, "mul"); }
Tensor* tensor_div_cuda(Tensor* a, Tensor* b) { return binary(lt::BIN_DIV, a, b, "div"); }
Tensor* tensor_add_scalar_cuda(Tensor* a, float s) { return scalar(lt::SC_ADD, a, s, "add_scalar"); }
Tensor* tensor_mul_scalar_cuda(Tensor* a, float s) { return scalar(lt::SC_MUL, a, s, "mul_scalar"); }
Tensor* tensor_div_scalar_cuda(Tensor* a, float s) {
  if (s == 0.0f) { fprintf(stderr, "luatorch error: division by zero scalar\n"); return scalar(lt::SC_MUL, a, 0.0f, "div_scalar"); }
  return scalar(lt::SC_DIV, a, s, "div_scalar");
}
Tensor* tensor_pow_scalar_cuda(Tensor* a, float e) { return scalar(lt::SC_POW, a, e, "pow_scalar"); }
Tensor* tensor_gt_scalar_cuda(Tensor* a, float s) { return scalar(lt::SC_GT, a, s, "gt_scalar"); }
Tensor* tensor_neg_cuda(Tensor* a) { return unary(lt::UN_NEG, a, "neg"); }
Tensor* tensor_abs_cuda(Tensor* a) { return unary(lt::UN_ABS, a, "abs"); }
Tensor* tensor_sqrt_cuda(Tensor* a) { return unary(lt::UN_SQRT, a, "sqrt"); }
Tensor* tensor_log_cuda(Tensor* a) { return unary(lt::UN_LOG, a, "log"); }
Tensor* tensor_exp_cuda(Tensor* a) { return unary(lt::UN_EXP, a, "exp"); }
Tensor* tensor_relu_cuda(Tensor* a) { return unary(lt::UN_RELU, a, "relu"); }
Tensor* tensor_sigmoid_cuda(Tensor* a) { return unary(lt::UN_SIGMOID, a, "sigmoid"); }
Tensor* tensor_tanh_cuda(Tensor* a) { return unary(lt::UN_TANH, a, "tanh"); }
Tensor* tensor_gelu_cuda(Tensor* a) { return unary(lt::UN_GELU, a, "gelu"); }
Tensor* tensor_silu_cuda(Tensor* a) { return unary(lt::UN_SILU, a, "silu"); }

float tensor_sum_cuda(Tensor* a) { return reduce(lt::RED_SUM, a, 1.0f); }
float tensor_mean_cuda(Tensor* a) { return dev(a) && a->numel ? reduce(lt::RED_SUM, a, 1.0f / (float)a->numel) : 0.0f; }
float tensor_max_cuda(Tensor* a) { return reduce(lt::RED_MAX, a, 1.0f); }
float tensor_min_cuda(Tensor* a) { return reduce(lt::RED_MIN, a, 1.0f); }

void tensor_add_cuda_(Tensor* a, Tensor* b) {
  if (!dev(a) || !dev(b) || a->numel != b->numel) { fail("add_ size mismatch"); return; }
  lt::binary_op(lt::BIN_ADD, lt::DT_F32, a->cuda_data, b->cuda_data, a->cuda_data, a->numel, kStream);
}
void tensor_sub_cuda_(Tensor* a, Tensor* b) {
  if (!dev(a) || !dev(b) || a->numel != b->numel) { fail("sub_ size mismatch"); return; }
  lt::binary_op(lt::BIN_SUB, lt::DT_F32, a->cuda_data, b->cuda_data, a->cuda_data, a->numel, kStream);
}
void tensor_mul_scalar_cuda_(Tensor* a, float s) {
  if (dev(a)) lt::scalar_op(lt::SC_MUL, lt::DT_F32, a->cuda_data, s, a->cuda_data, a->numel, kStream);
}
void tensor_add_scalar_cuda_(Tensor* a, float s) {
  if (dev(a)) lt::scalar_op(lt::SC_ADD, lt::DT_F32, a->cuda_data, s, a->cuda_data, a->numel, kStream);
}

Tensor* tensor_add_broadcast_cuda(Tensor* a, Tensor* b) {
  if (!dev(a) || !dev(b)) return fail("null or non-cuda tensor");
  if (a->ndim != 2 || b->numel != a->shape[1]) return fail("add_broadcast expects [rows, cols] + [cols]");
  return unary_like(a, "add_broadcast", [&](Tensor* o) {
    return lt::add_broadcast(lt::DT_F32, a->cuda_data, b->cuda_data, o->cuda_data, a->shape[0], a->shape[1], kStream);
  });
}
Tensor* tensor_add_broadcast_backward_cuda(Tensor* g) {
  if (!dev(g) || g->ndim != 2) return fail("add_broadcast_backward expects a 2-d cuda tensor");
  int64_t cols = g->shape[1];
  Tensor* o = gpu_tensor(&cols, 1, g->dtype);
  if (!o) return nullptr;
  const size_t sb = (size_t)lt::column_sum_scratch_floats(g->shape[0], cols) * sizeof(float);
  float* sc = (float*)pool_alloc(sb);
  cudaError_t e = lt::column_sum(lt::DT_F32, g->cuda_data, cols, o->cuda_data, lt::DT_F32, 0, g->shape[0], cols, sc, kStream);
  pool_free_async(sc, kStream);
  if (e != cudaSuccess) { tensor_free(o); return fail("add_broadcast_backward", e); }
  return o;
}

// ------------------------------------------------------------------ matmul family
Tensor* tensor_matmul_cuda(Tensor* a, Tensor* b) {
  if (!dev(a) || !dev(b)) return fail("null or non-cuda tensor");
  if (a->ndim != 2 || b->ndim != 2) return fail("matmul requires 2-d tensors");
  if (a->shape[1] != b->shape[0]) {
    fprintf(stderr, "luatorch error: matmul shape mismatch [%lld,%lld] x [%lld,%lld]\n", (long long)a->shape[0],
            (long long)a->shape[1], (long long)b->shape[0], (long long)b->shape[1]);
    return nullptr;
  }
  int64_t shp[2] = {a->shape[0], b->shape[1]};
  Tensor* o = gpu_tensor(shp, 2, a->dtype);
  if (!o) return nullptr;
  cudaError_t e = gemm_fp32(a->cuda_data, b->cuda_data, o->cuda_data, 1, shp[0], a->shape[1], shp[1]);
  if (e != cudaSuccess) { tensor_free(o); return fail("matmul", e); }
  return o;
}
// Kept for ABI parity with the reference's debug kernel; same tensor-core path.
Tensor* tensor_matmul_cuda_naive(Tensor* a, Tensor* b) { return tensor_matmul_cuda(a, b); }

Tensor* tensor_bmm_cuda(Tensor* a, Tensor* b) {
  if (!dev(a) || !dev(b)) return fail("null or non-cuda tensor");
  if (a->ndim != 3 || b->ndim != 3 || a->shape[0] != b->shape[0] || a->shape[2] != b->shape[1])
    return fail("bmm shape mismatch");
  int64_t shp[3] = {a->shape[0], a->shape[1], b->shape[2]};
  Tensor* o = gpu_tensor(shp, 3, a->dtype);
  if (!o) return nullptr;
  cudaError_t e = gemm_fp32(a->cuda_data, b->cuda_data, o->cuda_data, shp[0], shp[1], a->shape[2], shp[2]);
  if (e != cudaSuccess) { tensor_free(o); return fail("bmm", e); }
  return o;
}

Tensor* tensor_transpose_cuda(Tensor* a) {
  if (!dev(a) || a->ndim != 2) return fail("transpose requires a 2-d cuda tensor");
  int64_t shp[2] = {a->shape[1], a->shape[0]};
  Tensor* o = gpu_tensor(shp, 2, a->dtype);
  if (!o) return nullptr;
  cudaError_t e = lt::transpose2d(lt::DT_F32, a->cuda_data, o->cuda_data, a->shape[0], a->shape[1], kStream);
  if (e != cudaSuccess) { tensor_free(o); return fail("transpose", e); }
  return o;
}

float tensor_dot_cuda(Tensor* a, Tensor* b) {
  if (!dev(a) || !dev(b) || a->numel != b->numel) { fail("dot size mismatch"); return 0.0f; }
  Scratch& s = scratch();
  if (lt::dot_all(lt::DT_F32, a->cuda_data, b->cuda_data, a->numel, s.result, s.reduce, kStream) != cudaSuccess) return 0.0f;
  return read_result();
}

// ------------------------------------------------------------------ softmax and losses
Tensor* tensor_softmax_cuda(Tensor* a) {
  if (!dev(a)) return fail("null or non-cuda tensor");
  const int64_t cols = a->ndim >= 2 ? a->shape[a->ndim - 1] : a->numel;
  const int64_t rows = cols ? a->numel / cols : 0;
  return unary_like(a, "softmax", [&](Tensor* o) {
    return lt::softmax_rows(lt::DT_F32, a->cuda_data, o->cuda_data, rows, cols, cols, kStream);
  });
}

static Tensor* pointwise_loss(int mode, Tensor* p, Tensor* t, const char* name) {
  if (!dev(p) || !dev(t) || p->numel != t->numel) return fail(name);
  int64_t one = 1;
  Tensor* o = gpu_tensor(&one, 1, p->dtype);
  if (!o) return nullptr;
  cudaError_t e = lt::pointwise_loss(mode, lt::DT_F32, p->cuda_data, t->cuda_data, p->numel, o->cuda_data,
                                     scratch().reduce, kStream);
  if (e != cudaSuccess) { tensor_free(o); return fail(name, e); }
  return o;
}
static Tensor* pointwise_loss_bwd(int mode, Tensor* p, Tensor* t, const char* name) {
  if (!dev(p) || !dev(t) || p->numel != t->numel) return fail(name);
  return unary_like(p, name, [&](Tensor* o) {
    return lt::pointwise_loss_backward(mode, lt::DT_F32, p->cuda_data, t->cuda_data, p->numel, 1.0f, o->cuda_data, kStream);
  });
}
Tensor* tensor_mse_loss_cuda(Tensor* p, Tensor* t) { return pointwise_loss(0, p, t, "mse_loss size mismatch"); }
Tensor* tensor_mae_loss_cuda(Tensor* p, Tensor* t) { return pointwise_loss(1, p, t, "mae_loss size mismatch"); }
Tensor* tensor_mse_loss_backward_cuda(Tensor* p, Tensor* t) { return pointwise_loss_bwd(0, p, t, "mse_loss_backward size mismatch"); }
Tensor* tensor_mae_loss_backward_cuda(Tensor* p, Tensor* t) { return pointwise_loss_bwd(1, p, t, "mae_loss_backward size mismatch"); }

// Per-row losses (lse - logit[label]); rows with an out-of-range label give 0 and set a flag.
static cudaError_t ce_rows(Tensor* p, Tensor* t, float* lse, float* row_loss, int* flag) {
  return lt::cross_entropy_forward(lt::DT_F32, p->cuda_data, p->shape[1], t->cuda_data, 2, p->shape[0], p->shape[1],
                                   lse, row_loss, flag, kStream);
}

Tensor* tensor_cross_entropy_loss_cuda(Tensor* p, Tensor* t) {
  if (!dev(p) || !dev(t) || p->ndim != 2 || t->numel != p->shape[0])
    return fail("cross_entropy_loss expects logits [batch, classes] and labels [batch]");
  const int64_t rows = p->shape[0];
  float* buf = (float*)pool_alloc((size_t)rows * 2 * sizeof(float));
  Scratch& s = scratch();
  cudaMemsetAsync(s.flag, 0, sizeof(int), kStream);
  int64_t one = 1;
  Tensor* o = gpu_tensor(&one, 1, p->dtype);
  cudaError_t e = ce_rows(p, t, buf, buf + rows, s.flag);
  if (e == cudaSuccess)
    e = lt::reduce_all(lt::RED_SUM, lt::DT_F32, buf + rows, rows, 1.0f / (float)rows, o->cuda_data, s.reduce, kStream);
  pool_free_async(buf, kStream);
  if (e != cudaSuccess) { tensor_free(o); return fail("cross_entropy_loss", e); }
  return o;
}

Tensor* tensor_cross_entropy_loss_backward_cuda(Tensor* p, Tensor* t) {
  if (!dev(p) || !dev(t) || p->ndim != 2 || t->numel != p->shape[0])
    return fail("cross_entropy_loss_backward shape mismatch");
  const int64_t rows = p->shape[0], cols = p->shape[1];
  float* buf = (float*)pool_alloc((size_t)rows * 2 * sizeof(float));
  Tensor* o = gpu_like(p);
  cudaError_t e = ce_rows(p, t, buf, buf + rows, nullptr);
  if (e == cudaSuccess)
    e = lt::cross_entropy_backward(lt::DT_F32, p->cuda_data, cols, t->cuda_data, 2, rows, cols, buf, 1.0f / (float)rows,
                                   nullptr, o->cuda_data, cols, kStream);
  pool_free_async(buf, kStream);
  if (e != cudaSuccess) { tensor_free(o); return fail("cross_entropy_loss_backward", e); }
  return o;
}

// Per-sample losses [batch] (exported by the reference library, absent from its Lua cdef).
Tensor* tensor_fused_cross_entropy_cuda(Tensor* p, Tensor* t) {
  if (!dev(p) || !dev(t) || p->ndim != 2 || t->numel != p->shape[0]) return fail("fused_cross_entropy shape mismatch");
  int64_t rows = p->shape[0];
  Tensor* o = gpu_tensor(&rows, 1, p->dtype);
  float* lse = (float*)pool_alloc((size_t)rows * sizeof(float));
  cudaError_t e = ce_rows(p, t, lse, o->cuda_data, nullptr);
  pool_free_async(lse, kStream);
  if (e != cudaSuccess) { tensor_free(o); return fail("fused_cross_entropy", e); }
  return o;
}

// ------------------------------------------------------------------ fused ops
Tensor* tensor_fused_gelu_bias_cuda(Tensor* x, Tensor* bias) {
  if (!dev(x) || !dev(bias) || bias->numel == 0 || x->numel % bias->numel) return fail("fused_gelu_bias shape mismatch");
  return unary_like(x, "fused_gelu_bias", [&](Tensor* o) {
    return lt::gelu_bias_forward(lt::DT_F32, x->cuda_data, bias->cuda_data, lt::DT_F32, o->cuda_data,
                                 x->numel / bias->numel, bias->numel, kStream);
  });
}

Tensor* tensor_fused_layernorm_cuda(Tensor* x, Tensor* gamma, Tensor* beta, float eps) {
  if (!dev(x) || !dev(gamma) || !dev(beta) || gamma->numel == 0 || gamma->numel != beta->numel ||
      x->numel % gamma->numel)
    return fail("fused_layernorm shape mismatch");
  return unary_like(x, "fused_layernorm", [&](Tensor* o) {
    return lt::layernorm_forward(lt::DT_F32, x->cuda_data, gamma->cuda_data, beta->cuda_data, lt::DT_F32, eps,
                                 o->cuda_data, nullptr, nullptr, x->numel / gamma->numel, gamma->numel, kStream);
  });
}

void tensor_fused_adam_cuda(Tensor* p, Tensor* g, Tensor* m, Tensor* v, float lr, float beta1, float beta2,
                            float eps, float bc1, float bc2, float weight_decay) {
  if (!dev(p) || !dev(g) || !dev(m) || !dev(v) || p->numel != g->numel || p->numel != m->numel || p->numel != v->numel) {
    fail("fused_adam shape mismatch");
    return;
  }
  // one weight-decay segment covering the tensor: the table lives in a tiny device buffer
  struct Seg { int64_t end; float wd; };
  char* tab = (char*)pool_alloc(512);
  const int64_t end = p->numel;
  cudaMemcpyAsync(tab, &end, sizeof(end), cudaMemcpyHostToDevice, kStream);
  cudaMemcpyAsync(tab + 256, &weight_decay, sizeof(float), cudaMemcpyHostToDevice, kStream);
  lt::AdamArgs a{lr, beta1, beta2, eps, bc1, bc2, 1.0f, nullptr};
  cudaError_t e = lt::adamw_flat(p->cuda_data, nullptr, g->cuda_data, lt::DT_F32, m->cuda_data, v->cuda_data, p->numel,
                                 (const int64_t*)tab, (const float*)(tab + 256), 1, a, kStream);
  pool_free_async(tab, kStream);
  if (e != cudaSuccess) fail("fused_adam", e);
}

// ------------------------------------------------------------------ attention
__global__ void f32_to_bf16_kernel(const float* in, __nv_bfloat16* out, long long n) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(in[i]);
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* in, float* out, long long n) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < n) out[i] = __bfloat162float(in[i]);
}

Tensor* tensor_flash_attention_cuda(Tensor* Q, Tensor* K, Tensor* V, int batch_heads, int seq_len, int head_dim,
                                    int causal) {
  if (!dev(Q) || !dev(K) || !dev(V)) return fail("null or non-cuda tensor");
  const long long n = (long long)batch_heads * seq_len * head_dim;
  if (Q->numel != n || K->numel != n || V->numel != n) return fail("flash_attention shape mismatch");
  Tensor* out = gpu_like(Q);
  if (!out) return nullptr;
  __nv_bfloat16* buf = (__nv_bfloat16*)pool_alloc((size_t)n * 2 * 4);
  __nv_bfloat16 *q = buf, *k = buf + n, *v = buf + 2 * n, *o = buf + 3 * n;
  const unsigned grid = (unsigned)((n + 255) / 256);
  f32_to_bf16_kernel<<<grid, 256, 0, kStream>>>(Q->cuda_data, q, n);
  f32_to_bf16_kernel<<<grid, 256, 0, kStream>>>(K->cuda_data, k, n);
  f32_to_bf16_kernel<<<grid, 256, 0, kStream>>>(V->cuda_data, v, n);
  const float scale = 1.0f / sqrtf((float)head_dim);
  cudaError_t e;
  const long long S = seq_len, D = head_dim;
  if ((head_dim == 64 || head_dim == 128)) {
    lt::AttnArgs a;
    a.B = batch_heads; a.H = 1; a.S = seq_len; a.D = head_dim;
    a.q = q; a.k = k; a.v = v; a.o = o; a.lse = nullptr;
    a.q_sb = a.k_sb = a.v_sb = a.o_sb = S * D;
    a.q_ss = a.k_ss = a.v_ss = a.o_ss = D;
    a.q_sh = a.k_sh = a.v_sh = a.o_sh = D;
    a.causal = causal; a.scale = scale;
    e = lt::flash_attention_forward(a, kStream);
  } else {
    // scores = scale * Q K^T, softmax (causal), O = P V: batched tensor-core GEMMs
    __nv_bfloat16* sc = (__nv_bfloat16*)pool_alloc((size_t)batch_heads * S * S * 2);
    lt::GemmArgs g;
    g.M = (int)S; g.N = (int)S; g.K = (int)D; g.A = q; g.B = k; g.C = sc;
    g.lda = D; g.ldb = D; g.ldc = S; g.a_mn_major = 0; g.b_mn_major = 0;
    g.batch_inner = batch_heads; g.a_stride_inner = S * D; g.b_stride_inner = S * D; g.c_stride_inner = S * S;
    g.alpha = scale;
    e = lt::gemm_bf16(g, kStream);
    if (e == cudaSuccess) e = lt::softmax_scores(sc, batch_heads, S, S, S, causal, kStream);
    lt::GemmArgs h;
    h.M = (int)S; h.N = (int)D; h.K = (int)S; h.A = sc; h.B = v; h.C = o;
    h.lda = S; h.ldb = D; h.ldc = D; h.a_mn_major = 0; h.b_mn_major = 1;
    h.batch_inner = batch_heads; h.a_stride_inner = S * S; h.b_stride_inner = S * D; h.c_stride_inner = S * D;
    if (e == cudaSuccess) e = lt::gemm_bf16(h, kStream);
    pool_free_async(sc, kStream);
  }
  bf16_to_f32_kernel<<<grid, 256, 0, kStream>>>(o, out->cuda_data, n);
  pool_free_async(buf, kStream);
  if (e != cudaSuccess) { tensor_free(out); return fail("flash attention", e); }
  return out;
}

// ------------------------------------------------------------------ casts / AMP helpers
void* tensor_cast_f32_to_f16_cuda(Tensor* t) {
  if (!dev(t)) return nullptr;
  void* out = pool_alloc((size_t)t->numel * 2);
  if (out) lt::cast(lt::DT_F32, t->cuda_data, lt::DT_F16, out, t->numel, kStream);
  return out;
}
void tensor_cast_f16_to_f32_cuda(void* src, Tensor* dst) {
  if (src && dev(dst)) lt::cast(lt::DT_F16, src, lt::DT_F32, dst->cuda_data, dst->numel, kStream);
}
int tensor_has_inf_nan_cuda(Tensor* t) {
  if (!dev(t)) return 0;
  Scratch& s = scratch();
  cudaMemsetAsync(s.flag, 0, sizeof(int), kStream);
  lt::check_finite_scale(lt::DT_F32, t->cuda_data, t->numel, 1.0f, 0, s.flag, kStream);
  int v = 0;
  cudaMemcpyAsync(&v, s.flag, sizeof(int), cudaMemcpyDeviceToHost, kStream);
  cudaStreamSynchronize(kStream);
  return v != 0;
}
void tensor_scale_cuda(Tensor* t, float scale) {
  if (dev(t)) lt::scalar_op(lt::SC_MUL, lt::DT_F32, t->cuda_data, scale, t->cuda_data, t->numel, kStream);
}

}  // extern "C"
