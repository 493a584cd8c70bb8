// Host (fp32) implementations of the op set: elementwise / scalar / unary, reductions,
// in-place forms, bias broadcast, matmul / bmm / transpose / dot, activations, softmax,
// losses and im2col (counterparts of the reference's csrc/ops/*.c).  They are the oracle for
// the GPU kernels and what a front end gets for CPU tensors.  Error convention as in the
// reference: print `luatorch error: ...` to stderr and return NULL / 0 instead of aborting.
// The matmul is cache-blocked with an i-k-j inner order (the reference uses the naive
// i-j-k triple loop, csrc/ops/matmul.c:46-57).
#include "luatorch_abi.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace {

Tensor* err(const char* msg) {
  fprintf(stderr, "luatorch error: %s\n", msg);
  return nullptr;
}
Tensor* like(Tensor* a) { return tensor_new(a->shape, a->ndim, a->dtype, DEVICE_CPU); }
bool host(Tensor* t) { return t && t->data; }

template <typename F> Tensor* map2(Tensor* a, Tensor* b, const char* name, F f) {
  if (!host(a) || !host(b)) return err("null or non-cpu tensor");
  if (a->numel != b->numel) {
    fprintf(stderr, "luatorch error: %s size mismatch (%lld vs %lld)\n", name, (long long)a->numel,
            (long long)b->numel);
    return nullptr;
  }
  Tensor* o = like(a);
  if (!o) return nullptr;
  for (int64_t i = 0; i < a->numel; ++i) o->data[i] = f(a->data[i], b->data[i]);
  return o;
}
template <typename F> Tensor* map1(Tensor* a, F f) {
  if (!host(a)) return err("null or non-cpu tensor");
  Tensor* o = like(a);
  if (!o) return nullptr;
  for (int64_t i = 0; i < a->numel; ++i) o->data[i] = f(a->data[i]);
  return o;
}
Tensor* scalar1() {
  int64_t s = 1;
  return tensor_new(&s, 1, DTYPE_FLOAT32, DEVICE_CPU);
}
float gelu(float x) { return 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x))); }

void matmul_block(const float* A, const float* B, float* C, int64_t M, int64_t K, int64_t N) {
  memset(C, 0, sizeof(float) * (size_t)(M * N));
  const int64_t BK = 64, BI = 32;
  for (int64_t i0 = 0; i0 < M; i0 += BI)
    for (int64_t k0 = 0; k0 < K; k0 += BK)
      for (int64_t i = i0; i < (i0 + BI < M ? i0 + BI : M); ++i)
        for (int64_t k = k0; k < (k0 + BK < K ? k0 + BK : K); ++k) {
          const float a = A[i * K + k];
          const float* b = B + k * N;
          float* c = C + i * N;
          for (int64_t j = 0; j < N; ++j) c[j] += a * b[j];
        }
}

}  // namespace

extern "C" {

Tensor* tensor_add(Tensor* a, Tensor* b) { return map2(a, b, "add", [](float x, float y) { return x + y; }); }
Tensor* tensor_sub(Tensor* a, Tensor* b) { return map2(a, b, "sub", [](float x, float y) { return x - y; }); }
Tensor* tensor_mul(Tensor* a, Tensor* b) { return map2(a, b, "mul", [](float x, float y) { return x * y; }); }
Tensor* tensor_div(Tensor* a, Tensor* b) {
  bool warned = false;
  return map2(a, b, "div", [&](float x, float y) {
    if (y == 0.0f) {
      if (!warned) { fprintf(stderr, "luatorch error: division by zero, result set to 0\n"); warned = true; }
      return 0.0f;
    }
    return x / y;
  });
}
Tensor* tensor_add_scalar(Tensor* a, float s) { return map1(a, [=](float x) { return x + s; }); }
Tensor* tensor_mul_scalar(Tensor* a, float s) { return map1(a, [=](float x) { return x * s; }); }
Tensor* tensor_div_scalar(Tensor* a, float s) {
  if (s == 0.0f) { fprintf(stderr, "luatorch error: division by zero scalar\n"); return map1(a, [](float) { return 0.0f; }); }
  return map1(a, [=](float x) { return x / s; });
}
Tensor* tensor_pow_scalar(Tensor* a, float e) { return map1(a, [=](float x) { return powf(x, e); }); }
Tensor* tensor_neg(Tensor* a) { return map1(a, [](float x) { return -x; }); }
Tensor* tensor_abs(Tensor* a) { return map1(a, [](float x) { return fabsf(x); }); }
Tensor* tensor_sqrt(Tensor* a) { return map1(a, [](float x) { return x < 0.0f ? 0.0f : sqrtf(x); }); }
Tensor* tensor_log(Tensor* a) { return map1(a, [](float x) { return x <= 0.0f ? -INFINITY : logf(x); }); }
Tensor* tensor_exp(Tensor* a) { return map1(a, [](float x) { return expf(x); }); }

float tensor_sum(Tensor* a) {
  if (!host(a)) return 0.0f;
  double s = 0.0;
  for (int64_t i = 0; i < a->numel; ++i) s += a->data[i];
  return (float)s;
}
float tensor_mean(Tensor* a) { return host(a) && a->numel ? tensor_sum(a) / (float)a->numel : 0.0f; }
float tensor_max(Tensor* a) {
  if (!host(a) || !a->numel) return 0.0f;
  float m = a->data[0];
  for (int64_t i = 1; i < a->numel; ++i) m = a->data[i] > m ? a->data[i] : m;
  return m;
}
float tensor_min(Tensor* a) {
  if (!host(a) || !a->numel) return 0.0f;
  float m = a->data[0];
  for (int64_t i = 1; i < a->numel; ++i) m = a->data[i] < m ? a->data[i] : m;
  return m;
}

void tensor_add_(Tensor* a, Tensor* b) {
  if (!host(a) || !host(b) || a->numel != b->numel) { err("add_ size mismatch"); return; }
  for (int64_t i = 0; i < a->numel; ++i) a->data[i] += b->data[i];
}
void tensor_sub_(Tensor* a, Tensor* b) {
  if (!host(a) || !host(b) || a->numel != b->numel) { err("sub_ size mismatch"); return; }
  for (int64_t i = 0; i < a->numel; ++i) a->data[i] -= b->data[i];
}
void tensor_mul_scalar_(Tensor* a, float s) { if (host(a)) for (int64_t i = 0; i < a->numel; ++i) a->data[i] *= s; }
void tensor_add_scalar_(Tensor* a, float s) { if (host(a)) for (int64_t i = 0; i < a->numel; ++i) a->data[i] += s; }

Tensor* tensor_add_broadcast(Tensor* a, Tensor* b) {
  if (!host(a) || !host(b)) return err("null or non-cpu tensor");
  if (a->ndim != 2 || b->numel != a->shape[1]) return err("add_broadcast expects [rows, cols] + [cols]");
  Tensor* o = like(a);
  const int64_t R = a->shape[0], Cn = a->shape[1];
  for (int64_t r = 0; r < R; ++r)
    for (int64_t c = 0; c < Cn; ++c) o->data[r * Cn + c] = a->data[r * Cn + c] + b->data[c];
  return o;
}
Tensor* tensor_add_broadcast_backward(Tensor* g) {
  if (!host(g) || g->ndim != 2) return err("add_broadcast_backward expects a 2-d tensor");
  int64_t Cn = g->shape[1];
  Tensor* o = tensor_new(&Cn, 1, g->dtype, DEVICE_CPU);
  for (int64_t r = 0; r < g->shape[0]; ++r)
    for (int64_t c = 0; c < Cn; ++c) o->data[c] += g->data[r * Cn + c];
  return o;
}

Tensor* tensor_matmul(Tensor* a, Tensor* b) {
  if (!host(a) || !host(b)) return err("null or non-cpu tensor");
  if (a->ndim != 2 || b->ndim != 2) return err("matmul requires 2-d tensors");
  if (a->shape[1] != b->shape[0]) {
    fprintf(stderr, "luatorch error: matmul shape mismatch [%lld,%lld] x [%lld,%lld]\n",
            (long long)a->shape[0], (long long)a->shape[1], (long long)b->shape[0], (long long)b->shape[1]);
    return nullptr;
  }
  int64_t shp[2] = {a->shape[0], b->shape[1]};
  Tensor* o = tensor_new(shp, 2, a->dtype, DEVICE_CPU);
  matmul_block(a->data, b->data, o->data, shp[0], a->shape[1], shp[1]);
  return o;
}
Tensor* tensor_bmm(Tensor* a, Tensor* b) {
  if (!host(a) || !host(b)) return err("null or non-cpu tensor");
  if (a->ndim != 3 || b->ndim != 3 || a->shape[0] != b->shape[0] || a->shape[2] != b->shape[1])
    return err("bmm shape mismatch");
  int64_t shp[3] = {a->shape[0], a->shape[1], b->shape[2]};
  Tensor* o = tensor_new(shp, 3, a->dtype, DEVICE_CPU);
  const int64_t M = shp[1], K = a->shape[2], N = shp[2];
  for (int64_t i = 0; i < shp[0]; ++i)
    matmul_block(a->data + i * M * K, b->data + i * K * N, o->data + i * M * N, M, K, N);
  return o;
}
Tensor* tensor_transpose(Tensor* a) {
  if (!host(a) || a->ndim != 2) return err("transpose requires a 2-d tensor");
  int64_t shp[2] = {a->shape[1], a->shape[0]};
  Tensor* o = tensor_new(shp, 2, a->dtype, DEVICE_CPU);
  for (int64_t r = 0; r < a->shape[0]; ++r)
    for (int64_t c = 0; c < a->shape[1]; ++c) o->data[c * a->shape[0] + r] = a->data[r * a->shape[1] + c];
  return o;
}
float tensor_dot(Tensor* a, Tensor* b) {
  if (!host(a) || !host(b) || a->numel != b->numel) { err("dot size mismatch"); return 0.0f; }
  double s = 0.0;
  for (int64_t i = 0; i < a->numel; ++i) s += (double)a->data[i] * b->data[i];
  return (float)s;
}

Tensor* tensor_relu(Tensor* a) { return map1(a, [](float x) { return x > 0.0f ? x : 0.0f; }); }
Tensor* tensor_sigmoid(Tensor* a) { return map1(a, [](float x) { return 1.0f / (1.0f + expf(-x)); }); }
Tensor* tensor_tanh(Tensor* a) { return map1(a, [](float x) { return tanhf(x); }); }
Tensor* tensor_gelu(Tensor* a) { return map1(a, [](float x) { return gelu(x); }); }
Tensor* tensor_silu(Tensor* a) { return map1(a, [](float x) { return x / (1.0f + expf(-x)); }); }
Tensor* tensor_gt_scalar(Tensor* a, float s) { return map1(a, [=](float x) { return x > s ? 1.0f : 0.0f; }); }

Tensor* tensor_softmax(Tensor* a) {
  if (!host(a)) return err("null or non-cpu tensor");
  Tensor* o = like(a);
  const int64_t cols = a->ndim >= 2 ? a->shape[a->ndim - 1] : a->numel;
  const int64_t rows = cols ? a->numel / cols : 0;
  for (int64_t r = 0; r < rows; ++r) {
    const float* x = a->data + r * cols;
    float* y = o->data + r * cols;
    float m = x[0];
    for (int64_t c = 1; c < cols; ++c) m = x[c] > m ? x[c] : m;
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) { y[c] = expf(x[c] - m); s += y[c]; }
    for (int64_t c = 0; c < cols; ++c) y[c] = (float)(y[c] / s);
  }
  return o;
}

Tensor* tensor_mse_loss(Tensor* p, Tensor* t) {
  if (!host(p) || !host(t) || p->numel != t->numel) return err("mse_loss size mismatch");
  Tensor* o = scalar1();
  double s = 0.0;
  for (int64_t i = 0; i < p->numel; ++i) { const double d = p->data[i] - t->data[i]; s += d * d; }
  o->data[0] = (float)(s / (double)p->numel);
  return o;
}
Tensor* tensor_mse_loss_backward(Tensor* p, Tensor* t) {
  if (!host(p) || !host(t) || p->numel != t->numel) return err("mse_loss_backward size mismatch");
  Tensor* o = like(p);
  for (int64_t i = 0; i < p->numel; ++i) o->data[i] = 2.0f * (p->data[i] - t->data[i]) / (float)p->numel;
  return o;
}
Tensor* tensor_mae_loss(Tensor* p, Tensor* t) {
  if (!host(p) || !host(t) || p->numel != t->numel) return err("mae_loss size mismatch");
  Tensor* o = scalar1();
  double s = 0.0;
  for (int64_t i = 0; i < p->numel; ++i) s += fabs((double)p->data[i] - t->data[i]);
  o->data[0] = (float)(s / (double)p->numel);
  return o;
}
Tensor* tensor_mae_loss_backward(Tensor* p, Tensor* t) {
  if (!host(p) || !host(t) || p->numel != t->numel) return err("mae_loss_backward size mismatch");
  Tensor* o = like(p);
  for (int64_t i = 0; i < p->numel; ++i) {
    const float d = p->data[i] - t->data[i];
    o->data[i] = (d > 0.0f ? 1.0f : (d < 0.0f ? -1.0f : 0.0f)) / (float)p->numel;
  }
  return o;
}
Tensor* tensor_cross_entropy_loss(Tensor* p, Tensor* t) {
  if (!host(p) || !host(t) || p->ndim != 2 || t->numel != p->shape[0])
    return err("cross_entropy_loss expects logits [batch, classes] and labels [batch]");
  const int64_t Bn = p->shape[0], Cn = p->shape[1];
  double total = 0.0;
  for (int64_t b = 0; b < Bn; ++b) {
    const int64_t lab = (int64_t)t->data[b];
    if (lab < 0 || lab >= Cn) {
      fprintf(stderr, "luatorch error: label %lld out of range [0, %lld)\n", (long long)lab, (long long)Cn);
      return nullptr;
    }
    const float* x = p->data + b * Cn;
    float m = x[0];
    for (int64_t c = 1; c < Cn; ++c) m = x[c] > m ? x[c] : m;
    double s = 0.0;
    for (int64_t c = 0; c < Cn; ++c) s += exp((double)x[c] - m);
    total += log(s) + m - x[lab];
  }
  Tensor* o = scalar1();
  o->data[0] = (float)(total / (double)Bn);
  return o;
}
Tensor* tensor_cross_entropy_loss_backward(Tensor* p, Tensor* t) {
  if (!host(p) || !host(t) || p->ndim != 2 || t->numel != p->shape[0])
    return err("cross_entropy_loss_backward shape mismatch");
  const int64_t Bn = p->shape[0], Cn = p->shape[1];
  Tensor* o = like(p);
  for (int64_t b = 0; b < Bn; ++b) {
    const float* x = p->data + b * Cn;
    float* g = o->data + b * Cn;
    float m = x[0];
    for (int64_t c = 1; c < Cn; ++c) m = x[c] > m ? x[c] : m;
    double s = 0.0;
    for (int64_t c = 0; c < Cn; ++c) s += exp((double)x[c] - m);
    const int64_t lab = (int64_t)t->data[b];
    for (int64_t c = 0; c < Cn; ++c)
      g[c] = (float)((exp((double)x[c] - m) / s - (c == lab ? 1.0 : 0.0)) / (double)Bn);
  }
  return o;
}

Tensor* tensor_im2col(Tensor* in, int batch, int C, int H, int W, int k, int stride, int pad) {
  if (!host(in)) return err("null or non-cpu tensor");
  if ((int64_t)batch * C * H * W != in->numel) return err("im2col input size mismatch");
  const int oh = (H + 2 * pad - k) / stride + 1, ow = (W + 2 * pad - k) / stride + 1;
  int64_t shp[2] = {(int64_t)batch * oh * ow, (int64_t)C * k * k};
  Tensor* o = tensor_new(shp, 2, in->dtype, DEVICE_CPU);
  for (int b = 0; b < batch; ++b)
    for (int oy = 0; oy < oh; ++oy)
      for (int ox = 0; ox < ow; ++ox) {
        float* row = o->data + (((int64_t)b * oh + oy) * ow + ox) * shp[1];
        for (int c = 0; c < C; ++c)
          for (int ky = 0; ky < k; ++ky)
            for (int kx = 0; kx < k; ++kx) {
              const int iy = oy * stride + ky - pad, ix = ox * stride + kx - pad;
              row[(c * k + ky) * k + kx] =
                  (iy >= 0 && iy < H && ix >= 0 && ix < W) ? in->data[(((int64_t)b * C + c) * H + iy) * W + ix] : 0.0f;
            }
      }
  return o;
}

}  // extern "C"
