// Shared device helpers: 16-byte vector access with fp32 math for fp32 / bf16 / fp16
// storage, warp and block reductions, launch sizing for a 148-SM part.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdlib.h>
#include <atomic>

namespace lt {

extern std::atomic<uint64_t> g_ops_launches;
#define LT_COUNT_LAUNCH() ::lt::g_ops_launches.fetch_add(1, std::memory_order_relaxed)

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with launch_pdl() may be scheduled while
// the kernel before it in the stream is still running, so its launch latency and prologue
// overlap that kernel's tail; pdl_wait() then blocks until the earlier kernel has completed
// and its writes are visible.  Rules: a kernel launched this way touches no global memory
// before pdl_wait(), and every kernel calls pdl_trigger() (allow the NEXT kernel to be
// scheduled) AFTER its own pdl_wait().  The dependent kernel is released once every CTA of
// this one has triggered, so whenever it runs, everything BEFORE this kernel is complete.
// A kernel that is independent of its immediate predecessor (a weight-gradient GEMM after the
// input-gradient GEMM of the same layer) can therefore skip the wait in its prologue, work in
// the predecessor's tail, and call pdl_wait() just before it exits, which keeps completion
// transitive for the kernel after it ("late wait").  LT_PDL=0 in the environment turns the
// launch attribute off (plain stream order); set_pdl_override() does it at run time.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
  pdl_wait();
  pdl_trigger();
}
// late == true: the caller is independent of the previous kernel; pair with pdl_leave(late)
__device__ __forceinline__ void pdl_enter(bool late) {
  if (!late) pdl_wait();
  pdl_trigger();
}
__device__ __forceinline__ void pdl_leave(bool late) {
  if (late) pdl_wait();
}

// -1: follow LT_PDL; 0 / 1: forced off / on at run time (set_pdl_override in ops.h)
extern int g_pdl_override;

inline bool pdl_enabled() {
  if (g_pdl_override >= 0) return g_pdl_override != 0;
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LT_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

// LT_LATE_WAIT=0 makes every kernel wait for its predecessor in its prologue (comparison runs)
inline bool late_wait_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LT_LATE_WAIT");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0 && pdl_enabled();
}

// Bookkeeping for late wait.  A late kernel triggers without having waited, so the kernel after
// it can start while the ones before it still run.  When a kernel K is about to be launched,
// the launches in front of it look like   ... N [S] C1 .. Cc   where N is a normal kernel (it
// waited, then triggered), S an optional side kernel (below) and C1..Cc the late kernels
// launched back to back just before now.  When K runs, everything before N is complete; N
// (or S, which waited for N) and C1..Cc may still be running.  K may therefore be late only
// if it is independent of C1..Cc and of N: its caller vouches for the `independent_of`
// launches in front of it, and that number must cover them.  late_wait_begin() decides, the
// caller launches (launch_pdl resets the chain) and calls late_wait_commit().
//
// Side kernels.  A kernel whose only outputs are parameter gradients (the LayerNorm parameter
// reduction) is a dead end of the stream's data flow until the optimizer runs: its launcher
// calls mark_side_kernel() right after it.  Every later kernel is independent of it by
// construction, so it does not count: in  N S C1 .. Cc  the kernel K needs to vouch for c
// launches only (S waited for N, so N is complete), and the first kernel behind S may be late
// without vouching for anything.  This relies on two facts: the late-wait kernels (GEMM,
// attention backward) never read a parameter gradient, and the side kernel's scratch is not
// memory that the stream's allocator could hand to the next kernel (the binding keeps it in a
// buffer of its own).
extern int g_late_chain;       // c: late kernels launched back to back just before now
extern int g_late_side;        // 1: that chain stands right behind a side kernel
extern unsigned long long g_pdl_seq, g_side_mark;
inline void mark_side_kernel() { g_side_mark = g_pdl_seq; }
struct LateWait { int on, chain, side; };
inline LateWait late_wait_begin(int independent_of) {
  LateWait l{0, g_late_chain, 0};
  l.side = l.chain == 0 ? (g_side_mark != 0 && g_side_mark == g_pdl_seq) : (g_late_side != 0);
  const int need = l.chain + (l.side ? 0 : 1);
  l.on = (late_wait_enabled() && independent_of >= need) ? 1 : 0;
  return l;
}
inline void late_wait_commit(const LateWait& l) {
  if (l.on) { g_late_chain = l.chain + 1; g_late_side = l.side; }
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  g_late_chain = 0;
  g_late_side = 0;
  ++g_pdl_seq;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T> struct VecIO;

template <> struct VecIO<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void load(const float* p, float (&f)[4]) {
    float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  // 16 bytes kept as loaded (registers: 4), converted to fp32 only where they are used
  __device__ static __forceinline__ uint4 load_raw(const float* p) { return *reinterpret_cast<const uint4*>(p); }
  __device__ static __forceinline__ void unpack(const uint4& u, float (&f)[4]) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y);
    f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
  __device__ static __forceinline__ void store(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
  __device__ static __forceinline__ float ld(const float* p) { return *p; }
  __device__ static __forceinline__ void st(float* p, float v) { *p = v; }
};

template <> struct VecIO<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    unpack(u, f);
  }
  __device__ static __forceinline__ uint4 load_raw(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
  __device__ static __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  __device__ static __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  __device__ static __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
};

template <> struct VecIO<__half> {
  static constexpr int N = 8;
  __device__ static __forceinline__ uint4 load_raw(const __half* p) { return *reinterpret_cast<const uint4*>(p); }
  __device__ static __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  __device__ static __forceinline__ void load(const __half* p, float (&f)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  __device__ static __forceinline__ void store(__half* p, const float (&f)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  __device__ static __forceinline__ float ld(const __half* p) { return __half2float(*p); }
  __device__ static __forceinline__ void st(__half* p, float v) { *p = __float2half(v); }
};

__host__ __device__ inline bool is_aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions for up to 1024 threads; `sh` needs 32 floats. Result in all threads.
__device__ __forceinline__ float block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : 0.0f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : -INFINITY;
  return warp_max(r);
}

inline int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}
// Grid for a grid-stride loop over `work_items` items with `threads` per block: enough
// blocks to fill every SM eight deep, never more than needed.
inline int stream_grid(int64_t work_items, int threads) {
  int64_t need = (work_items + threads - 1) / threads;
  int64_t cap = (int64_t)sm_count() * 8;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

#define LT_DISPATCH_DTYPE(dtype, T, ...)                                   \
  switch (dtype) {                                                         \
    case ::lt::DT_F32: { using T = float; __VA_ARGS__; break; }            \
    case ::lt::DT_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }   \
    case ::lt::DT_F16: { using T = __half; __VA_ARGS__; break; }           \
    default: return cudaErrorInvalidValue;                                 \
  }

__device__ __forceinline__ float gelu_exact_tanh(float x) {
  const float k0 = 0.7978845608f, k1 = 0.044715f;
  return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float dgelu_exact_tanh(float x) {
  const float k0 = 0.7978845608f, k1 = 0.044715f;
  float t = tanhf(k0 * (x + k1 * x * x * x));
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * k0 * (1.0f + 3.0f * k1 * x * x);
}

// Philox-4x32-10 counter RNG: 4 uniform 32-bit words per (counter, key).
__device__ __forceinline__ uint4 philox4(uint64_t counter, uint64_t key) {
  uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}
__device__ __forceinline__ float u32_to_unit(uint32_t x) {  // (0, 1]
  return ((x >> 8) + 1) * (1.0f / 16777216.0f);
}

}  // namespace lt
