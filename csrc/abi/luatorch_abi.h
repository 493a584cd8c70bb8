// C ABI of libluatorch.so: the exact struct layout and symbol list the reference's LuaJIT
// front end binds through FFI (lua/luatorch/tensor.lua:8-179, lua/luatorch/distributed/
// init.lua:16-22; struct in csrc/tensor.h:27-39), so that front end loads this library
// unchanged.  Data is fp32 through this interface (the reference treats every buffer as
// float* whatever the dtype field says, csrc/tensor.c:25-34).
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { DEVICE_CPU = 0, DEVICE_CUDA = 1 } Device;
typedef enum {
  DTYPE_FLOAT32 = 0, DTYPE_FLOAT64 = 1, DTYPE_INT32 = 2, DTYPE_INT64 = 3, DTYPE_FLOAT16 = 4
} DType;

typedef struct Tensor {
  float* data;        // host storage (NULL while the tensor lives on the GPU)
  float* cuda_data;   // device storage (NULL while on the host)
  int64_t* shape;
  int64_t* strides;
  int ndim;
  int64_t numel;
  int dtype;
  int device;
  int requires_grad;
  void* grad;
  int ref_count;
} Tensor;

// lifecycle / access
Tensor* tensor_new(int64_t* shape, int ndim, int dtype, int device);
void tensor_free(Tensor* t);
void tensor_fill(Tensor* t, float value);
void tensor_zeros(Tensor* t);
void tensor_ones(Tensor* t);
void tensor_rand(Tensor* t);
void tensor_randn(Tensor* t);
void tensor_print(Tensor* t);
Tensor* tensor_copy(Tensor* t);
void tensor_copy_data(Tensor* dst, Tensor* src);
float tensor_get(Tensor* t, int64_t idx);
void tensor_set(Tensor* t, int64_t idx, float value);
Tensor* tensor_reshape(Tensor* src, int64_t* new_shape, int new_ndim);
int64_t tensor_numel(Tensor* t);
void luatorch_manual_seed(uint64_t seed);   // extension: the reference seeds from time()

// device runtime
Tensor* tensor_to_cuda(Tensor* t);
Tensor* tensor_to_cpu(Tensor* t);
Tensor* tensor_to_cuda_async(Tensor* t);
Tensor* tensor_to_cpu_async(Tensor* t);
void tensor_sync(void);
Tensor* tensor_new_cuda(int64_t* shape, int ndim, int dtype);
void tensor_cuda_free(Tensor* t);

// memory pool
void pool_init(void);
void* pool_alloc(size_t bytes);
void pool_free(void* ptr);
void pool_clear(void);
size_t pool_allocated_bytes(void);
size_t pool_cached_bytes(void);
/* extensions: stream-ordered release, debug canaries (memory_pool.cpp) */
void pool_free_async(void* ptr, void* stream);
void pool_set_debug(int on);
int pool_check_canaries(void);
size_t pool_overruns_seen(void);
size_t cuda_memory_allocated(void);
size_t cuda_memory_cached(void);

// distributed
int luatorch_nccl_get_gpu_count(void);
int luatorch_nccl_init(int num_gpus);
int luatorch_nccl_allreduce(float** ptrs, int64_t count, int num_gpus);
int luatorch_nccl_broadcast(float** ptrs, int64_t count, int root, int num_gpus);
void luatorch_nccl_destroy(void);

#ifdef __cplusplus
}
static_assert(offsetof(Tensor, data) == 0 && offsetof(Tensor, cuda_data) == 8 &&
              offsetof(Tensor, shape) == 16 && offsetof(Tensor, strides) == 24 &&
              offsetof(Tensor, ndim) == 32 && offsetof(Tensor, numel) == 40 &&
              offsetof(Tensor, dtype) == 48 && offsetof(Tensor, device) == 52 &&
              offsetof(Tensor, requires_grad) == 56 && offsetof(Tensor, grad) == 64 &&
              offsetof(Tensor, ref_count) == 72 && sizeof(Tensor) == 80,
              "Tensor layout must match the reference ABI");
#endif
