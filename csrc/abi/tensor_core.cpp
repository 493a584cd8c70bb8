// Tensor struct runtime on the host: allocation, reference counting, fills, RNG, element
// access, views (counterpart of the reference's csrc/tensor.c).
//
// Deliberate differences: views hold a reference on their source and the storage is released
// when the LAST owner goes away (in the reference freeing a view frees the shared storage,
// csrc/tensor.c:108-128 with :260-294); the RNG is a seedable xoshiro generator instead of
// rand() seeded from time().
#include "luatorch_abi.h"

#include <math.h>
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

extern "C" void tensor_cuda_free(Tensor* t);

namespace {

size_t dtype_size(int dtype) {
  switch (dtype) {
    case DTYPE_FLOAT64: case DTYPE_INT64: return 8;
    case DTYPE_FLOAT16: return 2;
    default: return 4;
  }
}

int64_t calc_numel(const int64_t* shape, int ndim) {
  int64_t n = 1;
  for (int i = 0; i < ndim; ++i) n *= shape[i];
  return n;
}

void calc_strides(const int64_t* shape, int64_t* strides, int ndim) {
  int64_t s = 1;
  for (int i = ndim - 1; i >= 0; --i) { strides[i] = s; s *= shape[i]; }
}

std::mutex g_rng_mu;
uint64_t g_rng[4] = {0x9E3779B97F4A7C15ull, 0xBF58476D1CE4E5B9ull, 0x94D049BB133111EBull, 0x2545F4914F6CDD1Dull};

uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
uint64_t next_u64() {
  uint64_t* s = g_rng;
  const uint64_t r = rotl(s[1] * 5, 7) * 9, t = s[1] << 17;
  s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]; s[2] ^= t; s[3] = rotl(s[3], 45);
  return r;
}
double next_unit() { return (double)(next_u64() >> 11) * (1.0 / 9007199254740992.0); }

}  // namespace

// Every tensor is allocated as a block {Tensor, magic, source}: for a view, `magic` holds
// kViewMagic and `source` the tensor whose storage it shares; is_view() compares the word.
namespace {
constexpr uint64_t kViewMagic = 0x4c54564945570001ull;
struct ViewBlock { Tensor t; uint64_t magic; Tensor* source; };
bool is_view(Tensor* t) { return reinterpret_cast<ViewBlock*>(t)->magic == kViewMagic; }
struct OwnBlock { Tensor t; uint64_t magic; Tensor* source; };
}  // namespace

extern "C" {

void luatorch_manual_seed(uint64_t seed) {
  std::lock_guard<std::mutex> lock(g_rng_mu);
  uint64_t z = seed + 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < 4; ++i) {
    z += 0x9E3779B97F4A7C15ull;
    uint64_t x = z;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    g_rng[i] = x ^ (x >> 31);
  }
}

// Shape-only tensor (no storage): used for results that live on the GPU.
Tensor* lt_tensor_new_meta(const int64_t* shape, int ndim, int dtype) {
  if (ndim < 0 || (ndim > 0 && !shape)) return nullptr;
  OwnBlock* blk = (OwnBlock*)calloc(1, sizeof(OwnBlock));
  if (!blk) return nullptr;
  Tensor* t = &blk->t;
  t->ndim = ndim;
  t->shape = (int64_t*)malloc(sizeof(int64_t) * (ndim > 0 ? ndim : 1));
  t->strides = (int64_t*)malloc(sizeof(int64_t) * (ndim > 0 ? ndim : 1));
  memcpy(t->shape, shape, sizeof(int64_t) * ndim);
  calc_strides(shape, t->strides, ndim);
  t->numel = calc_numel(shape, ndim);
  t->dtype = dtype;
  t->device = DEVICE_CPU;
  t->ref_count = 1;
  return t;
}

Tensor* tensor_new(int64_t* shape, int ndim, int dtype, int device) {
  Tensor* t = lt_tensor_new_meta(shape, ndim, dtype);
  if (!t) return nullptr;
  OwnBlock* blk = reinterpret_cast<OwnBlock*>(t);
  const size_t bytes = (size_t)(t->numel > 0 ? t->numel : 1) * dtype_size(dtype);
  t->data = (float*)calloc(1, bytes < 4 ? 4 : bytes);
  if (!t->data) {
    fprintf(stderr, "luatorch error: out of memory allocating %zu bytes\n", bytes);
    free(t->shape); free(t->strides); free(blk);
    return nullptr;
  }
  (void)device;   // tensors are born on the host; tensor_to_cuda moves them (as in the reference)
  return t;
}

void tensor_free(Tensor* t) {
  if (!t) return;
  if (--t->ref_count > 0) return;
  if (t->grad) { tensor_free((Tensor*)t->grad); t->grad = nullptr; }
  if (is_view(t)) {
    Tensor* src = reinterpret_cast<ViewBlock*>(t)->source;
    free(t->shape); free(t->strides);
    free(t);
    tensor_free(src);          // drops the reference the view held; storage dies with the last owner
    return;
  }
  if (t->cuda_data) tensor_cuda_free(t);
  free(t->data); free(t->strides); free(t->shape);
  free(t);
}

void tensor_fill(Tensor* t, float v) {
  if (!t || !t->data) return;
  for (int64_t i = 0; i < t->numel; ++i) t->data[i] = v;
}
void tensor_zeros(Tensor* t) { tensor_fill(t, 0.0f); }
void tensor_ones(Tensor* t) { tensor_fill(t, 1.0f); }

void tensor_rand(Tensor* t) {
  if (!t || !t->data) return;
  std::lock_guard<std::mutex> lock(g_rng_mu);
  for (int64_t i = 0; i < t->numel; ++i) t->data[i] = (float)next_unit();
}

void tensor_randn(Tensor* t) {
  if (!t || !t->data) return;
  std::lock_guard<std::mutex> lock(g_rng_mu);
  for (int64_t i = 0; i < t->numel; i += 2) {       // Box-Muller in pairs
    double u1 = next_unit(), u2 = next_unit();
    if (u1 < 1e-300) u1 = 1e-300;
    const double m = sqrt(-2.0 * log(u1));
    t->data[i] = (float)(m * cos(6.283185307179586 * u2));
    if (i + 1 < t->numel) t->data[i + 1] = (float)(m * sin(6.283185307179586 * u2));
  }
}

void tensor_print(Tensor* t) {
  if (!t) { printf("Tensor(NULL)\n"); return; }
  printf("Tensor(shape=[");
  for (int i = 0; i < t->ndim; ++i) printf(i ? ", %lld" : "%lld", (long long)t->shape[i]);
  printf("], device=%s", t->device == DEVICE_CUDA ? "cuda" : "cpu");
  if (t->data) {
    printf(", data=[");
    const int64_t n = t->numel < 20 ? t->numel : 20;
    for (int64_t i = 0; i < n; ++i) printf(i ? ", %.4f" : "%.4f", t->data[i]);
    if (t->numel > 20) printf(", ...");
    printf("]");
  }
  printf(")\n");
}

Tensor* tensor_copy(Tensor* t) {
  if (!t) return nullptr;
  Tensor* c = tensor_new(t->shape, t->ndim, t->dtype, DEVICE_CPU);
  if (!c) return nullptr;
  if (t->data) memcpy(c->data, t->data, (size_t)t->numel * sizeof(float));
  c->requires_grad = t->requires_grad;
  return c;
}

void tensor_copy_data(Tensor* dst, Tensor* src) {
  if (!dst || !src || !dst->data || !src->data) return;
  if (dst->numel != src->numel) {
    fprintf(stderr, "luatorch error: copy_data size mismatch (%lld vs %lld)\n",
            (long long)dst->numel, (long long)src->numel);
    return;
  }
  memcpy(dst->data, src->data, (size_t)src->numel * sizeof(float));
}

float tensor_get(Tensor* t, int64_t idx) {
  if (!t) return 0.0f;
  if (!t->data) { fprintf(stderr, "luatorch error: tensor_get on a gpu tensor, call cpu() first\n"); return 0.0f; }
  if (idx < 0 || idx >= t->numel) {
    fprintf(stderr, "luatorch error: index %lld out of bounds for tensor with %lld elements\n",
            (long long)idx, (long long)t->numel);
    return 0.0f;
  }
  return t->data[idx];
}

void tensor_set(Tensor* t, int64_t idx, float v) {
  if (!t) return;
  if (!t->data) { fprintf(stderr, "luatorch error: tensor_set on a gpu tensor, call cpu() first\n"); return; }
  if (idx < 0 || idx >= t->numel) {
    fprintf(stderr, "luatorch error: index %lld out of bounds for tensor with %lld elements\n",
            (long long)idx, (long long)t->numel);
    return;
  }
  t->data[idx] = v;
}

Tensor* tensor_reshape(Tensor* src, int64_t* new_shape, int new_ndim) {
  if (!src) return nullptr;
  const int64_t n = calc_numel(new_shape, new_ndim);
  if (n != src->numel) {
    fprintf(stderr, "luatorch error: reshape size mismatch, %lld vs %lld\n", (long long)src->numel,
            (long long)n);
    return nullptr;
  }
  ViewBlock* blk = (ViewBlock*)calloc(1, sizeof(ViewBlock));
  if (!blk) return nullptr;
  blk->magic = kViewMagic;
  blk->source = src;
  Tensor* t = &blk->t;
  *t = *src;
  t->grad = nullptr;
  t->ref_count = 1;
  t->ndim = new_ndim;
  t->shape = (int64_t*)malloc(sizeof(int64_t) * (new_ndim > 0 ? new_ndim : 1));
  t->strides = (int64_t*)malloc(sizeof(int64_t) * (new_ndim > 0 ? new_ndim : 1));
  memcpy(t->shape, new_shape, sizeof(int64_t) * new_ndim);
  calc_strides(new_shape, t->strides, new_ndim);
  src->ref_count++;
  return t;
}

int64_t tensor_numel(Tensor* t) { return t ? t->numel : 0; }

}  // extern "C"
