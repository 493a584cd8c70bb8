// Peer-memory collectives fused with the optimizer step (interface in comm_kernels.h).
//
// Protocol of every kernel here:
//   start barrier : block 0 publishes `epoch` into slot [rank] of every peer's "start" pad;
//                   every block waits until its own pad shows `epoch` from all peers, i.e.
//                   every rank's stream has reached this collective and the buffers it
//                   exposes are final.
//   data phase    : 16-byte vector loads / stores on peer-mapped addresses, fp32 math.
//   done barrier  : the last block to finish (ticket counter) publishes `epoch` into the
//                   "done" pads, then waits for every peer's, so when the kernel retires no
//                   peer is still reading this rank's buffers or writing into them.
// All waits are bounded by a cycle budget; expiry is reported through `status`, never by a
// trap or an endless spin.
//
// Epochs: a caller may pass the collective's sequence number, or 0 to let the kernel number
// itself from a counter word in its own signal pad (the last block advances it), so that a
// captured CUDA graph can be replayed: no launch argument changes from step to step.
//
// NVLS: when the caller passes multicast addresses of the gradient and shadow arenas, the
// sharded kernel reads its slice with multimem.ld_reduce (the NVSwitch adds the ranks'
// values and returns one vector) and publishes the updated weights with multimem.st (one
// store, delivered to every rank), which halves the bytes each GPU moves over its links.
#include "comm_kernels.h"

#include <cuda_bf16.h>
#include <atomic>

namespace lt {

namespace {

std::atomic<uint64_t> g_comm_launches{0};

constexpr int THREADS = 512;
constexpr int DEFAULT_BLOCKS = 296;   // two CTAs per SM on a 148-SM part
constexpr int MAX_WORLD = 16;
constexpr int SLOT_START = 0;
constexpr int SLOT_DONE = 16;
constexpr int SLOT_TICKET = 32;
constexpr int SLOT_EPOCH = 33;        // local sequence counter for self-numbered collectives
constexpr long long DEFAULT_BUDGET = 6000000000ll;  // about three seconds of SM clocks

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_peer16(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Sum over all ranks of 8 bf16 values at a multicast address (fp32 accumulation in the switch).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
// One 16-byte store delivered to the same offset of every rank's buffer.
__device__ __forceinline__ void multimem_st16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ bool reached(uint32_t seen, uint32_t epoch) {
  return (int32_t)(seen - epoch) >= 0;
}

__device__ void report(int* status, int code, int rank, uint32_t epoch, int phase, int peer,
                       uint32_t seen) {
  if (!status) return;
  if (atomicCAS(&status[0], 0, code) == 0) {
    status[1] = rank; status[2] = (int)epoch; status[3] = phase; status[4] = peer;
    status[5] = (int)seen;
  }
}

// Waits until slot[base + peer] >= epoch for every peer; threads 0..world-1 each poll one.
// Returns false for the whole block on expiry.
__device__ bool wait_peers(const uint32_t* my_pad, int base, int world, int rank, uint32_t epoch,
                           int phase, long long budget, int* status, int* sh_fail) {
  if (threadIdx.x == 0) *sh_fail = 0;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const uint32_t* slot = my_pad + base + threadIdx.x;
    uint32_t seen = ld_acquire_sys(slot);
    if (!reached(seen, epoch)) {
      const long long t0 = clock64();
      unsigned spins = 0;
      while (true) {
        seen = ld_acquire_sys(slot);
        if (reached(seen, epoch)) break;
        if ((++spins & 0xff) == 0) {
          if (status && ((volatile int*)status)[0] != 0) { *sh_fail = 1; break; }
          if (clock64() - t0 > budget) {
            report(status, 1, rank, epoch, phase, (int)threadIdx.x, seen);
            *sh_fail = 1;
            break;
          }
        }
        __nanosleep(64);
      }
    }
  }
  __syncthreads();
  return *sh_fail == 0;
}

// Sequence number of this collective: the caller's, or (caller passed 0) one more than the
// counter word of this rank's own pad.  Every block reads the word before any block can
// advance it (the advance happens after the last block has taken its ticket).
__device__ __forceinline__ uint32_t resolve_epoch(const uint64_t* signal_ptrs, int rank,
                                                  uint32_t epoch_arg) {
  if (epoch_arg) return epoch_arg;
  const volatile uint32_t* my_pad = reinterpret_cast<const volatile uint32_t*>(signal_ptrs[rank]);
  return my_pad[SLOT_EPOCH] + 1u;
}

__device__ bool start_barrier(const uint64_t* signal_ptrs, int rank, int world, uint32_t epoch,
                              long long budget, int* status, int* sh_fail) {
  if (blockIdx.x == 0 && (int)threadIdx.x < world) {
    __threadfence_system();
    uint32_t* peer_pad = reinterpret_cast<uint32_t*>(signal_ptrs[threadIdx.x]);
    st_release_sys(peer_pad + SLOT_START + rank, epoch);
  }
  const uint32_t* my_pad = reinterpret_cast<const uint32_t*>(signal_ptrs[rank]);
  return wait_peers(my_pad, SLOT_START, world, rank, epoch, 1, budget, status, sh_fail);
}

// Called by every block after its data phase. Only the last block talks to the peers.
__device__ void done_barrier(const uint64_t* signal_ptrs, int rank, int world, uint32_t epoch,
                             long long budget, int* status, int* sh_fail,
                             bool self_numbered = false) {
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  uint32_t* my_pad = reinterpret_cast<uint32_t*>(signal_ptrs[rank]);
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(my_pad + SLOT_TICKET, 1u);
    is_last = (t == gridDim.x - 1);
    if (is_last) {
      my_pad[SLOT_TICKET] = 0;
      if (self_numbered) my_pad[SLOT_EPOCH] = epoch;
    }
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence_system();
  if ((int)threadIdx.x < world) {
    uint32_t* peer_pad = reinterpret_cast<uint32_t*>(signal_ptrs[threadIdx.x]);
    st_release_sys(peer_pad + SLOT_DONE + rank, epoch);
  }
  wait_peers(my_pad, SLOT_DONE, world, rank, epoch, 2, budget, status, sh_fail);
}

__device__ __forceinline__ void acc_bf16x8(const uint4& u, float (&acc)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    acc[2 * i] += t.x;
    acc[2 * i + 1] += t.y;
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

__device__ __forceinline__ int find_segment(const int64_t* seg_end, int nseg, int64_t i) {
  int lo = 0, hi = nseg - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (i < seg_end[mid]) hi = mid; else lo = mid + 1;
  }
  return lo;
}

// State of 8 consecutive parameters, loaded early so the HBM reads overlap the NVLink reads.
struct Adam8State { float4 p0, p1, m0, m1, v0, v1; };
__device__ __forceinline__ Adam8State adam8_load(const float* master, const float* m, const float* v,
                                                 long long e) {
  Adam8State s;
  s.p0 = *reinterpret_cast<const float4*>(master + e); s.p1 = *reinterpret_cast<const float4*>(master + e + 4);
  s.m0 = *reinterpret_cast<const float4*>(m + e); s.m1 = *reinterpret_cast<const float4*>(m + e + 4);
  s.v0 = *reinterpret_cast<const float4*>(v + e); s.v1 = *reinterpret_cast<const float4*>(v + e + 4);
  return s;
}
__device__ __forceinline__ void adam8(float* master, float* m, float* v, long long e, const Adam8State& s,
                                      const float (&g)[8], float wd, const AdamArgs& a,
                                      float (&p_out)[8]) {
  float p[8] = {s.p0.x, s.p0.y, s.p0.z, s.p0.w, s.p1.x, s.p1.y, s.p1.z, s.p1.w};
  float mm[8] = {s.m0.x, s.m0.y, s.m0.z, s.m0.w, s.m1.x, s.m1.y, s.m1.z, s.m1.w};
  float vv[8] = {s.v0.x, s.v0.y, s.v0.z, s.v0.w, s.v1.x, s.v1.y, s.v1.z, s.v1.w};
  const float decay = 1.0f - a.lr * wd;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float gj = g[j] * a.grad_scale;
    p[j] *= decay;
    mm[j] = a.beta1 * mm[j] + (1.0f - a.beta1) * gj;
    vv[j] = a.beta2 * vv[j] + (1.0f - a.beta2) * gj * gj;
    p[j] -= a.lr * (mm[j] / a.bc1) / (sqrtf(vv[j] / a.bc2) + a.eps);
    p_out[j] = p[j];
  }
  *reinterpret_cast<float4*>(master + e) = make_float4(p[0], p[1], p[2], p[3]);
  *reinterpret_cast<float4*>(master + e + 4) = make_float4(p[4], p[5], p[6], p[7]);
  *reinterpret_cast<float4*>(m + e) = make_float4(mm[0], mm[1], mm[2], mm[3]);
  *reinterpret_cast<float4*>(m + e + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
  *reinterpret_cast<float4*>(v + e) = make_float4(vv[0], vv[1], vv[2], vv[3]);
  *reinterpret_cast<float4*>(v + e + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
}

// SGD with momentum on 8 consecutive parameters (lua/luatorch/optim/sgd.lua:33-56 in the
// reference): v = mu v + g; p -= lr v, or with Nesterov p -= lr (mu v + g).
__device__ __forceinline__ void sgd8(float* master, float* vel, long long e, const float (&g)[8],
                                     float lr, float mu, int nesterov, float gscale,
                                     float (&p_out)[8]) {
  float4 p0 = *reinterpret_cast<const float4*>(master + e), p1 = *reinterpret_cast<const float4*>(master + e + 4);
  float p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
  if (vel) {
    float4 v0 = *reinterpret_cast<const float4*>(vel + e), v1 = *reinterpret_cast<const float4*>(vel + e + 4);
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gscale;
      vv[j] = mu * vv[j] + gj;
      p[j] -= lr * (nesterov ? mu * vv[j] + gj : vv[j]);
    }
    *reinterpret_cast<float4*>(vel + e) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(vel + e + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] -= lr * g[j] * gscale;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) p_out[j] = p[j];
  *reinterpret_cast<float4*>(master + e) = make_float4(p[0], p[1], p[2], p[3]);
  *reinterpret_cast<float4*>(master + e + 4) = make_float4(p[4], p[5], p[6], p[7]);
}

struct KArgs {
  const uint64_t* grad_ptrs;
  const uint64_t* signal_ptrs;
  const uint64_t* shadow_ptrs;
  const __nv_bfloat16* grad_mc;   // multicast address of the gradient arena, or null
  __nv_bfloat16* shadow_mc;       // multicast address of the shadow arena, or null
  int rank, world;
  long long elem_offset, n;
  long long state_base;           // index into master / m / v of this rank's first element
  float* master; float* m; float* v;
  const int64_t* seg_end; const float* seg_wd; int nseg;
  AdamArgs adam;
  int opt_kind; float momentum; int nesterov;
  uint32_t epoch;
  int mode;
  long long budget;
  int* status;
};

// WORLD: 0 = runtime world size.  OPT (optimizer body) and NVLS are compile-time so that each
// variant keeps only its own state in registers: two 512-thread CTAs per SM need <= 64.
template <int WORLD, int OPT, bool NVLS>
__global__ void __launch_bounds__(THREADS, 2)
allreduce_adamw_kernel(const KArgs k) {
  __shared__ int sh_fail;
  __shared__ uint64_t sh_grad[MAX_WORLD], sh_shadow[MAX_WORLD];
  const int world = WORLD ? WORLD : k.world;
  if ((int)threadIdx.x < world) {
    sh_grad[threadIdx.x] = k.grad_ptrs[threadIdx.x];
    sh_shadow[threadIdx.x] = k.shadow_ptrs ? k.shadow_ptrs[threadIdx.x] : 0;
  }
  const uint32_t epoch = resolve_epoch(k.signal_ptrs, k.rank, k.epoch);
  if (!start_barrier(k.signal_ptrs, k.rank, world, epoch, k.budget, k.status, &sh_fail)) return;

  AdamArgs adam = k.adam;
  if (adam.dyn) { adam.lr = adam.dyn[0]; adam.bc1 = adam.dyn[1]; adam.bc2 = adam.dyn[2]; }
  // an overflow flag must read the same on every rank (it is set from all-reduced data)
  const bool skip = adam.skip_flag && *adam.skip_flag;

  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const bool sharded = NVLS || k.mode == COMM_TWO_SHOT_SHARDED;
  constexpr bool nvls = NVLS;
  const long long span = sharded ? k.n / world : k.n;
  const long long base = k.elem_offset + (sharded ? (long long)k.rank * span : 0);
  for (long long i = skip ? span : tid; i < span / 8; i += nthreads) {
    const long long e = base + i * 8;          // arena coordinate (gradients, shadow, segments)
    const long long es = k.state_base + i * 8; // optimizer-state coordinate
    Adam8State st;
    if (OPT == COMM_OPT_ADAMW) st = adam8_load(k.master, k.m, k.v, es);  // HBM reads go out first
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if constexpr (nvls) {
      const uint4 r = multimem_ld_reduce_bf16x8(k.grad_mc + e);
      acc_bf16x8(r, g);
    } else {
      uint4 part[WORLD ? WORLD : MAX_WORLD];
#pragma unroll
      for (int q = 0; q < (WORLD ? WORLD : MAX_WORLD); ++q) {
        if (q < world) {
          const int src = (k.rank + q) % world;  // spread the first touch over the links
          part[q] = ld_peer16(reinterpret_cast<const __nv_bfloat16*>(sh_grad[src]) + e);
        }
      }
      // fixed summation order (rank 0 .. world-1) so every rank computes identical bits
#pragma unroll
      for (int r = 0; r < (WORLD ? WORLD : MAX_WORLD); ++r) {
        if (r < world) {
          const int q = (r - k.rank + world) % world;
          acc_bf16x8(part[q], g);
        }
      }
    }
    float p[8];
    if (OPT == COMM_OPT_ADAMW) {
      const float wd = k.nseg > 0 ? k.seg_wd[find_segment(k.seg_end, k.nseg, e)] : 0.0f;
      adam8(k.master, k.m, k.v, es, st, g, wd, adam, p);
    } else {
      sgd8(k.master, k.m, es, g, adam.lr, k.momentum, k.nesterov, adam.grad_scale, p);
    }
    const uint4 packed = pack_bf16x8(p);
    if (sharded) {
      if (nvls) {
        multimem_st16(k.shadow_mc + e, packed);
      } else {
#pragma unroll
        for (int q = 0; q < (WORLD ? WORLD : MAX_WORLD); ++q) {
          if (q < world) {
            const int dst = (k.rank + q) % world;
            if (sh_shadow[dst])
              st_peer16(reinterpret_cast<__nv_bfloat16*>(sh_shadow[dst]) + e, packed);
          }
        }
      }
    } else if (sh_shadow[k.rank]) {
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(sh_shadow[k.rank]) + e) = packed;
    }
  }
  done_barrier(k.signal_ptrs, k.rank, world, epoch, k.budget, k.status, &sh_fail, k.epoch == 0);
}

__global__ void __launch_bounds__(THREADS)
peer_broadcast_kernel(const uint64_t* buf_ptrs, const uint64_t* signal_ptrs, int rank, int world,
                      int root, long long byte_offset, long long nbytes, uint32_t epoch_arg,
                      long long budget, int* status) {
  __shared__ int sh_fail;
  const uint32_t epoch = resolve_epoch(signal_ptrs, rank, epoch_arg);
  if (!start_barrier(signal_ptrs, rank, world, epoch, budget, status, &sh_fail)) return;
  if (rank != root) {
    const char* src = reinterpret_cast<const char*>(buf_ptrs[root]) + byte_offset;
    char* dst = reinterpret_cast<char*>(buf_ptrs[rank]) + byte_offset;
    const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
    long long done = 0;
    if (vec) {
      for (long long i = tid; i < nbytes / 16; i += nthreads)
        *reinterpret_cast<uint4*>(dst + i * 16) = ld_peer16(src + i * 16);
      done = (nbytes / 16) * 16;
    }
    for (long long i = done + tid; i < nbytes; i += nthreads)
      dst[i] = *reinterpret_cast<const volatile char*>(src + i);
  }
  done_barrier(signal_ptrs, rank, world, epoch, budget, status, &sh_fail, epoch_arg == 0);
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
peer_allreduce_kernel(const uint64_t* buf_ptrs, const uint64_t* signal_ptrs, int rank, int world,
                      long long elem_offset, long long n, float scale, uint32_t epoch_arg,
                      long long budget, int* status) {
  __shared__ int sh_fail;
  __shared__ uint64_t sh_buf[MAX_WORLD];
  if ((int)threadIdx.x < world) sh_buf[threadIdx.x] = buf_ptrs[threadIdx.x];
  const uint32_t epoch = resolve_epoch(signal_ptrs, rank, epoch_arg);
  if (!start_barrier(signal_ptrs, rank, world, epoch, budget, status, &sh_fail)) return;
  constexpr int V = 16 / sizeof(T);  // elements per 16-byte vector
  const long long span = n / world;
  const long long base = elem_offset + (long long)rank * span;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < span / V; i += nthreads) {
    const long long e = base + i * V;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) {
      uint4 u = ld_peer16(reinterpret_cast<const T*>(sh_buf[r]) + e);
      if (sizeof(T) == 2) {
        acc_bf16x8(u, acc);
      } else {
        acc[0] += __uint_as_float(u.x); acc[1] += __uint_as_float(u.y);
        acc[2] += __uint_as_float(u.z); acc[3] += __uint_as_float(u.w);
      }
    }
    uint4 out;
    if (sizeof(T) == 2) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= scale;
      out = pack_bf16x8(acc);
    } else {
      out = make_uint4(__float_as_uint(acc[0] * scale), __float_as_uint(acc[1] * scale),
                       __float_as_uint(acc[2] * scale), __float_as_uint(acc[3] * scale));
    }
    for (int q = 0; q < world; ++q) {
      const int dst = (rank + q) % world;
      st_peer16(reinterpret_cast<T*>(sh_buf[dst]) + e, out);
    }
  }
  done_barrier(signal_ptrs, rank, world, epoch, budget, status, &sh_fail, epoch_arg == 0);
}

__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t expected, long long budget,
                                 int* status) {
  const long long t0 = clock64();
  while (true) {
    const uint32_t seen = ld_acquire_sys(flag);
    if (reached(seen, expected)) return;
    if (clock64() - t0 > budget) {
      report(status, 100, 0, expected, 0, 0, seen);
      return;
    }
    __nanosleep(128);
  }
}

int pick_blocks(long long vectors, int max_blocks) {
  int cap = max_blocks > 0 ? max_blocks : DEFAULT_BLOCKS;
  long long need = (vectors + THREADS - 1) / THREADS;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

}  // namespace

uint64_t comm_launch_count() { return g_comm_launches.load(); }

cudaError_t allreduce_adamw(const CommAdamArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  if (a.world < 1 || a.world > MAX_WORLD || a.n % (8 * a.world) != 0 || a.elem_offset % 8 != 0)
    return cudaErrorInvalidValue;
  KArgs k;
  k.grad_ptrs = a.grad_ptrs; k.signal_ptrs = a.signal_ptrs; k.shadow_ptrs = a.shadow_ptrs;
  k.grad_mc = a.mode == COMM_TWO_SHOT_SHARDED ? reinterpret_cast<const __nv_bfloat16*>(a.grad_mc) : nullptr;
  k.shadow_mc = reinterpret_cast<__nv_bfloat16*>(a.shadow_mc);
  k.rank = a.rank; k.world = a.world;
  k.elem_offset = a.elem_offset; k.n = a.n;
  k.master = a.master; k.m = a.m; k.v = a.v;
  k.opt_kind = a.opt_kind; k.momentum = a.momentum; k.nesterov = a.nesterov;
  if (a.opt_kind != COMM_OPT_ADAMW && a.opt_kind != COMM_OPT_SGD) return cudaErrorInvalidValue;
  if (a.opt_kind == COMM_OPT_ADAMW && (!a.m || !a.v)) return cudaErrorInvalidValue;
  {
    const long long own = a.mode == COMM_TWO_SHOT_SHARDED ? a.n / a.world : a.n;
    const long long first = a.elem_offset + (a.mode == COMM_TWO_SHOT_SHARDED ? (long long)a.rank * own : 0);
    k.state_base = a.state_base >= 0 ? a.state_base : first;
    if (k.state_base % 4 != 0) return cudaErrorInvalidValue;
  }
  k.seg_end = a.seg_end; k.seg_wd = a.seg_wd; k.nseg = a.nseg;
  k.adam = a.adam; k.epoch = a.epoch; k.mode = a.mode;
  k.budget = DEFAULT_BUDGET; k.status = a.status;
  const long long span = a.mode == COMM_TWO_SHOT_SHARDED ? a.n / a.world : a.n;
  const int blocks = pick_blocks(span / 8, a.max_blocks);
  // NVLS needs both multicast addresses (reduce through ld_reduce, publish through st)
  const bool nvls = k.grad_mc != nullptr && k.shadow_mc != nullptr;
  if (!nvls) { k.grad_mc = nullptr; k.shadow_mc = nullptr; }
#define LT_LAUNCH_COMM(W)                                                                           \
  do {                                                                                              \
    if (nvls) {                                                                                     \
      if (a.opt_kind == COMM_OPT_ADAMW) allreduce_adamw_kernel<0, COMM_OPT_ADAMW, true><<<blocks, THREADS, 0, stream>>>(k); \
      else allreduce_adamw_kernel<0, COMM_OPT_SGD, true><<<blocks, THREADS, 0, stream>>>(k);        \
    } else if (a.opt_kind == COMM_OPT_ADAMW) {                                                      \
      allreduce_adamw_kernel<W, COMM_OPT_ADAMW, false><<<blocks, THREADS, 0, stream>>>(k);          \
    } else {                                                                                        \
      allreduce_adamw_kernel<W, COMM_OPT_SGD, false><<<blocks, THREADS, 0, stream>>>(k);            \
    }                                                                                               \
  } while (0)
  switch (a.world) {
    case 2: LT_LAUNCH_COMM(2); break;
    case 4: LT_LAUNCH_COMM(4); break;
    case 8: LT_LAUNCH_COMM(8); break;
    default: LT_LAUNCH_COMM(0); break;
  }
#undef LT_LAUNCH_COMM
  g_comm_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t peer_broadcast(const uint64_t* buf_ptrs, const uint64_t* signal_ptrs, int rank,
                           int world, int root, int64_t byte_offset, int64_t nbytes,
                           uint32_t epoch, int* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_WORLD || root < 0 || root >= world) return cudaErrorInvalidValue;
  const int blocks = pick_blocks(nbytes / 16 + 1, 0);
  peer_broadcast_kernel<<<blocks, THREADS, 0, stream>>>(buf_ptrs, signal_ptrs, rank, world, root,
                                                       byte_offset, nbytes, epoch, DEFAULT_BUDGET,
                                                       status);
  g_comm_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t peer_allreduce(const uint64_t* buf_ptrs, const uint64_t* signal_ptrs, int rank,
                           int world, int64_t elem_offset, int64_t n, int dtype, float scale,
                           uint32_t epoch, int* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_WORLD) return cudaErrorInvalidValue;
  const int V = dtype == DT_F32 ? 4 : 8;
  if (n % ((int64_t)V * world) != 0 || elem_offset % V != 0) return cudaErrorInvalidValue;
  const int blocks = pick_blocks(n / world / V, 0);
  if (dtype == DT_F32)
    peer_allreduce_kernel<float><<<blocks, THREADS, 0, stream>>>(
        buf_ptrs, signal_ptrs, rank, world, elem_offset, n, scale, epoch, DEFAULT_BUDGET, status);
  else if (dtype == DT_BF16)
    peer_allreduce_kernel<__nv_bfloat16><<<blocks, THREADS, 0, stream>>>(
        buf_ptrs, signal_ptrs, rank, world, elem_offset, n, scale, epoch, DEFAULT_BUDGET, status);
  else
    return cudaErrorInvalidValue;
  g_comm_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t wait_flag_bounded(const uint32_t* flag, uint32_t expected, int64_t budget_cycles,
                              int* status, cudaStream_t stream) {
  wait_flag_kernel<<<1, 1, 0, stream>>>(flag, expected, budget_cycles, status);
  g_comm_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace lt
