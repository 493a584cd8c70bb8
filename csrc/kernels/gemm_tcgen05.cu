// bf16 GEMM on the 5th-generation tensor cores: tcgen05.mma issued by one thread per
// CTA, operands staged in shared memory by TMA (128-byte swizzle), fp32 accumulators
// in TMEM, epilogue read back with tcgen05.ld.
//
// Structure: persistent kernels, one CTA per SM, 64 + 32 * EPI_WARPS (= 576) threads:
//   warp 0       TMA producer (one lane issues the tiled loads of each pipeline stage)
//   warp 1       TMEM owner + MMA issuer (one lane)
//   warps 2..9   epilogue: two warps per 32-lane TMEM quadrant of the 128-row tile, each
//                taking half of the tile's columns
// The TMEM accumulator is double buffered (2 x BN columns) so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Two kernels share that structure and the epilogue:
//   gemm_tcgen05_kernel<BN>       one CTA per 128 x BN tile
//   gemm_tcgen05_pair_kernel<BN>  a cluster of two CTAs (cta_group::2) per 256 x BN tile: each
//                                 CTA loads its own 128 rows of A and half of B, the even CTA
//                                 issues the MMAs for both, each CTA drains its own TMEM half
// choose_tile() picks kernel and width from a cost model measured on the part; K may be split
// into slices that run as batches into an fp32 workspace (choose_split, splitk_reduce_kernel);
// the pair kernel can also pull remote row shards of B over NVLink while it multiplies the
// local ones (GemmGather).  A SIMT kernel covers the shapes TMA cannot address.
//
// This kernel stands in for the reference's cublasSgemm / cublasSgemmStridedBatched
// (csrc/cuda/ops/matmul.cu:121-133, 177-187) and for its add_broadcast / gelu_bias
// kernels (csrc/cuda/ops/arithmetic.cu:478-484, csrc/cuda/ops/fused.cu:26-35), which
// become epilogue options here.
#include "gemm.h"
#include "sm100_ptx.cuh"
#include "common.cuh"

#include <cuda.h>
#include <atomic>
#include <mutex>
#include <stdio.h>
#include <stdlib.h>

namespace lt {

using namespace ptx;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;              // 64 bf16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
// Sixteen epilogue warps (four per scheduler): with K = 768 a 256-wide tile's main loop lasts
// about 6000 cycles and a GELU / dGELU epilogue of 128 x 256 outputs per CTA needs that many
// issue slots, so with eight warps (two per scheduler, low IPC) the epilogue was the longer
// side of the pipeline: measured 58.9 -> 50.1 us for [8192,768]x[768,3072]^T with dGELU.
#ifndef LT_EPI_WARPS
#define LT_EPI_WARPS 16
#endif
constexpr int EPI_WARPS = LT_EPI_WARPS;     // EPI_WARPS/4 warps per TMEM lane quadrant share the columns
constexpr int EPI_SPLIT = EPI_WARPS / 4;
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
#ifndef LT_SMEM_BUDGET_KB
#define LT_SMEM_BUDGET_KB 200
#endif
constexpr int SMEM_BUDGET = LT_SMEM_BUDGET_KB * 1024;   // operand ring per CTA

// A pipeline stage holds KSUB 64-wide k blocks of both operands: one barrier round trip then
// covers KSUB x 4 MMAs.  (Measured: a stage costs about 0.17 us of hand-off on top of its
// bytes, so narrow tiles, whose stages are small, gain from two blocks per stage.)
template <int BN>
struct TileCfg {
  static constexpr int KSUB = BN <= 128 ? 2 : 1;
  static constexpr int B_SUB_BYTES = BN * BK * 2;
  static constexpr int A_STAGE = A_STAGE_BYTES * KSUB;
  static constexpr int B_STAGE_BYTES = B_SUB_BYTES * KSUB;
  static constexpr int STAGE_BYTES = A_STAGE + B_STAGE_BYTES;
  static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES;   // 4 at BN=256 and at BN=128
  static constexpr int TMEM_COLS = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);  // power of two
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ int g_gemm_error = 0;

struct KernelParams {
  int M, N, K;
  int tiles_m, tiles_n, batch_inner, batch_total;
  int a_mn, b_mn;
  void* C;
  long long ldc, c_stride_inner, c_stride_outer;
  float alpha;
  int c_fp32, accumulate;
  const void* bias;
  int bias_fp32;
  int act;
  const __nv_bfloat16* residual;
  long long ldr;
  __nv_bfloat16* aux_out;
  const __nv_bfloat16* aux_in;
  long long ld_aux;
  int causal_tiles;
  int causal_k;
  int vec_ok;  // C / residual / aux rows allow 16-byte vector access
  int vec32_ok;  // ... and 32-byte (256-bit) access (bf16 output, residual, aux)
  int c32_ok;    // fp32 output rows allow 32-byte access
  // all-gather of B fused into the kernel (g_world <= 1: off)
  const uint64_t* g_b_ptrs;
  const uint64_t* g_signal_ptrs;
  uint32_t* g_flags;
  int* g_status;
  long long g_ldb;
  int g_rank, g_world, g_rows_per_shard, g_done;
  uint32_t g_epoch;
  int late_wait;   // GemmArgs::overlap_prev: wait for the previous kernel before exit, not before work
};

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_f(float x) {
  const float k0 = 0.7978845608f, k1 = 0.044715f;
  float t = tanh_fast(k0 * (x + k1 * x * x * x));
  return 0.5f * x * (1.0f + t);
}
__device__ __forceinline__ float dgelu_f(float x) {
  const float k0 = 0.7978845608f, k1 = 0.044715f;
  float t = tanh_fast(k0 * (x + k1 * x * x * x));
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * k0 * (1.0f + 3.0f * k1 * x * x);
}

// The same two functions on a pair of values with packed f32x2 arithmetic (one instruction
// per two elements; the tanh stays one MUFU each).  The epilogue of a K = 768 product is bound
// by instruction issue, so the vector path uses these.
//   gelu(x)  = h + h t,                  h = x / 2, t = tanh(x (k0 + k0 k1 x^2))
//   gelu'(x) = s + s r (1 - s) 2,        s = (1 + t) / 2, r = x (k0 + 3 k0 k1 x^2)
__device__ __forceinline__ float2 tanh_arg2(float2 x, float2 x2) {
  const float k0 = 0.7978845608f, k0k1 = 0.7978845608f * 0.044715f;
  return fmul2(x, ffma2(x2, make_float2(k0k1, k0k1), make_float2(k0, k0)));
}
__device__ __forceinline__ float2 gelu2(float2 x) {
  const float2 u = tanh_arg2(x, fmul2(x, x));
  const float2 t = make_float2(tanh_fast(u.x), tanh_fast(u.y));
  const float2 h = fmul2(x, make_float2(0.5f, 0.5f));
  return ffma2(h, t, h);
}
// returns v * gelu'(x)
__device__ __forceinline__ float2 dgelu_mul2(float2 v, float2 x) {
  const float k0 = 0.7978845608f, k0k1 = 0.7978845608f * 0.044715f;
  const float2 x2 = fmul2(x, x);
  const float2 u = tanh_arg2(x, x2);
  const float2 t = make_float2(tanh_fast(u.x), tanh_fast(u.y));
  const float2 s = ffma2(t, make_float2(0.5f, 0.5f), make_float2(0.5f, 0.5f));
  // r2 = 2 x (k0 + 3 k0 k1 x^2)
  const float2 r2 = fmul2(x, ffma2(x2, make_float2(6.0f * k0k1, 6.0f * k0k1), make_float2(2.0f * k0, 2.0f * k0)));
  const float2 z = ffma2(fmul2(r2, s), make_float2(-1.0f, -1.0f), r2);      // r2 (1 - s)
  return fmul2(v, ffma2(s, z, s));
}

// Scalar epilogue for one element, shared by the tensor-core tail path and the SIMT
// fallback kernel.
__device__ __forceinline__ void epilogue_store_scalar(const KernelParams& p, char* c_base,
                                                      long long row, int col, float acc) {
  float v = acc * p.alpha;
  if (p.bias) {
    v += p.bias_fp32 ? ((const float*)p.bias)[col]
                     : __bfloat162float(((const __nv_bfloat16*)p.bias)[col]);
  }
  if (p.act == GEMM_ACT_GELU) {
    if (p.aux_out) p.aux_out[row * p.ldc + col] = __float2bfloat16(v);
    v = gelu_f(v);
  } else if (p.act == GEMM_ACT_RELU) {
    if (p.aux_out) p.aux_out[row * p.ldc + col] = __float2bfloat16(v);
    v = fmaxf(v, 0.0f);
  } else if (p.act == GEMM_ACT_DGELU) {
    v *= dgelu_f(__bfloat162float(p.aux_in[row * p.ld_aux + col]));
  } else if (p.act == GEMM_ACT_DRELU) {
    v = __bfloat162float(p.aux_in[row * p.ld_aux + col]) > 0.0f ? v : 0.0f;
  }
  if (p.residual) v += __bfloat162float(p.residual[row * p.ldr + col]);
  if (p.c_fp32) {
    float* c = (float*)c_base + row * p.ldc + col;
    if (p.accumulate) v += *c;
    *c = v;
  } else {
    __nv_bfloat16* c = (__nv_bfloat16*)c_base + row * p.ldc + col;
    if (p.accumulate) v += __bfloat162float(*c);
    *c = __float2bfloat16(v);
  }
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// 32 consecutive bf16 (64 bytes) of one output row: two 256-bit accesses when the address is
// 32-byte aligned (full sectors per instruction), else four 128-bit ones.
__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float* v, int vec32) {
  if (vec32) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint4 a = pack8(v + 16 * h), b = pack8(v + 16 * h + 8);
      asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 16 * h),
                   "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                   : "memory");
    }
  } else {
    uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = pack8(v + 8 * i);
  }
}
__device__ __forceinline__ void load_bf16x32(const __nv_bfloat16* src, float* v, int vec32) {
  if (vec32) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint4 a, b;
      asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                   : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z),
                     "=r"(b.w)
                   : "l"(src + 16 * h)
                   : "memory");
      float f[8];
      unpack8(a, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[16 * h + j] = f[j];
      unpack8(b, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[16 * h + 8 + j] = f[j];
    }
  } else {
    const uint4* sp = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
      unpack8(sp[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[8 * i + j] = f[j];
    }
  }
}

// Epilogue of one 128 x BN accumulator tile: this warp's 32 rows (TMEM lane quadrant `quad`)
// and every EPI_SPLIT-th 32-column chunk starting at chunk `half`, read from TMEM address
// `t_row`, written to C.  (Round robin: BN = 192 gives two of the four warps of a quadrant two
// chunks and the others one; BN = 64 leaves two of them idle.)
template <int BN>
__device__ __forceinline__ void epilogue_tile(const KernelParams& p, uint32_t t_row, int m0, int n0,
                                              int bi, int bo, int quad, int half, int lane) {
  constexpr int EPI_CW = 32;
  const long long row = m0 + quad * 32 + lane;
  const bool row_ok = row < p.M;
  const size_t esz = p.c_fp32 ? 4 : 2;
  char* c_base = (char*)p.C + (size_t)(bi * p.c_stride_inner + bo * p.c_stride_outer) * esz;
#pragma unroll 1
  for (int cb = half * EPI_CW; cb < BN; cb += EPI_CW * EPI_SPLIT) {
    if (n0 + cb >= p.N) break;  // uniform across the warp
    uint32_t rr[EPI_CW];
#pragma unroll
    for (int s = 0; s < EPI_CW / 32; ++s)
      tmem_ld_32x32(t_row + cb + 32 * s, *reinterpret_cast<uint32_t(*)[32]>(&rr[32 * s]));
    tmem_ld_wait();
#pragma unroll
    for (int s = 0; s < EPI_CW / 32; ++s) {
    const int c0 = cb + 32 * s;
    const int col0 = n0 + c0;
    if (col0 >= p.N) break;
    const uint32_t* r = &rr[32 * s];
    if (!row_ok) continue;
    if (p.vec_ok && col0 + 32 <= p.N) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
      if (p.alpha != 1.0f) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
      }
      if (p.bias) {
        if (p.bias_fp32) {
          const float4* bp = reinterpret_cast<const float4*>((const float*)p.bias + col0);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 bv = __ldg(bp + i);
            const float2 s0 = fadd2(make_float2(v[4 * i], v[4 * i + 1]), make_float2(bv.x, bv.y));
            const float2 s1 = fadd2(make_float2(v[4 * i + 2], v[4 * i + 3]), make_float2(bv.z, bv.w));
            v[4 * i] = s0.x; v[4 * i + 1] = s0.y; v[4 * i + 2] = s1.x; v[4 * i + 3] = s1.y;
          }
        } else {
          const uint4* bp =
              reinterpret_cast<const uint4*>((const __nv_bfloat16*)p.bias + col0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float f[8];
            unpack8(__ldg(bp + i), f);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const float2 sj = fadd2(make_float2(v[8 * i + j], v[8 * i + j + 1]), make_float2(f[j], f[j + 1]));
              v[8 * i + j] = sj.x; v[8 * i + j + 1] = sj.y;
            }
          }
        }
      }
      if (p.act == GEMM_ACT_GELU || p.act == GEMM_ACT_RELU) {
        if (p.aux_out) {
          store_bf16x32(p.aux_out + row * p.ldc + col0, v, p.vec32_ok);
        }
        if (p.act == GEMM_ACT_GELU) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 g = gelu2(make_float2(v[i], v[i + 1]));
            v[i] = g.x; v[i + 1] = g.y;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.0f);
        }
      } else if (p.act == GEMM_ACT_DGELU || p.act == GEMM_ACT_DRELU) {
        float x[32];
        load_bf16x32(p.aux_in + row * p.ld_aux + col0, x, p.vec32_ok);
        if (p.act == GEMM_ACT_DGELU) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 g = dgelu_mul2(make_float2(v[i], v[i + 1]), make_float2(x[i], x[i + 1]));
            v[i] = g.x; v[i + 1] = g.y;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = x[i] > 0.0f ? v[i] : 0.0f;
        }
      }
      if (p.residual) {
        float x[32];
        load_bf16x32(p.residual + row * p.ldr + col0, x, p.vec32_ok);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 si = fadd2(make_float2(v[i], v[i + 1]), make_float2(x[i], x[i + 1]));
          v[i] = si.x; v[i + 1] = si.y;
        }
      }
      if (p.c_fp32) {
        float* cf = (float*)c_base + row * p.ldc + col0;
        if (p.c32_ok) {
          // 128 bytes per lane as four 256-bit accesses (the epilogue's cost follows the number
          // of 32-byte sectors an instruction touches: 16-byte accesses write each sector twice)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[8 * i + j];
            if (p.accumulate) {
              float q[8];
              asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                           : "=f"(q[0]), "=f"(q[1]), "=f"(q[2]), "=f"(q[3]), "=f"(q[4]), "=f"(q[5]),
                             "=f"(q[6]), "=f"(q[7])
                           : "l"(cf + 8 * i)
                           : "memory");
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] += q[j];
            }
            asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(cf + 8 * i),
                         "f"(o[0]), "f"(o[1]), "f"(o[2]), "f"(o[3]), "f"(o[4]), "f"(o[5]), "f"(o[6]),
                         "f"(o[7])
                         : "memory");
          }
        } else {
          float4* cp = reinterpret_cast<float4*>(cf);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            if (p.accumulate) {
              float4 old = cp[i];
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            cp[i] = o;
          }
        }
      } else {
        __nv_bfloat16* cp = (__nv_bfloat16*)c_base + row * p.ldc + col0;
        if (p.accumulate) {
          float x[32];
          load_bf16x32(cp, x, p.vec32_ok);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += x[i];
        }
        store_bf16x32(cp, v, p.vec32_ok);
      }
    } else {
      // fully unrolled so the accumulator registers are only ever indexed statically
      // (a dynamic index would force the whole batch into local memory)
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int col = col0 + i;
        if (col < p.N) epilogue_store_scalar(p, c_base, row, col, __uint_as_float(r[i]));
      }
    }
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b, const KernelParams p) {
  using Cfg = TileCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows x 128 B.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * Cfg::A_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + STAGES;          // [STAGES]
  uint64_t* tmem_full_bar = bars + 2 * STAGES;  // [2]
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_base_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_holder + 1);

  const int warp_idx = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 32 * EPI_WARPS);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp_idx == 1) {
    tmem_alloc(smem_u32(tmem_base_holder), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_holder;
  // Everything above overlapped the previous kernel's tail; after the wait its results are
  // final.  The trigger comes AFTER the wait, so whenever a dependent kernel runs, everything
  // before this kernel is complete: that is what lets a kernel marked `late_wait` (independent
  // of its predecessor) start working at once and wait only before it exits.
  if (!p.late_wait) pdl_wait();
  pdl_trigger();

  const int num_kb = (p.K + BK * Cfg::KSUB - 1) / (BK * Cfg::KSUB);
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int total_tiles = tiles_per_batch * p.batch_total;

  auto tile_skipped = [&](int m0, int n0) -> bool {
    if (p.causal_tiles == 1) return n0 > m0 + BM - 1;
    if (p.causal_tiles == 2) return m0 > n0 + BN - 1;
    return false;
  };
  // pipeline stages of the k loop for the tile at row m0 (shortened for block-triangular A)
  auto tile_stages = [&](int m0) -> int {
    if (!p.causal_k) return num_kb;
    int k_end = m0 + BM;
    if (k_end > p.K) k_end = p.K;
    return (k_end + BK * Cfg::KSUB - 1) / (BK * Cfg::KSUB);
  };

  if (warp_idx == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int b = tile / tiles_per_batch;
        const int t = tile - b * tiles_per_batch;
        const int m0 = (t % p.tiles_m) * BM;
        const int n0 = (t / p.tiles_m) * BN;
        if (tile_skipped(m0, n0)) continue;
        const int bi = b % p.batch_inner, bo = b / p.batch_inner;
        const int nkb = tile_stages(m0);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag,
                                 &g_gemm_error, 1)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_arrive_expect_tx(fb, Cfg::STAGE_BYTES);
#pragma unroll
          for (int sub = 0; sub < Cfg::KSUB; ++sub) {
            const uint32_t sa = smem_u32(smem_a + stage * Cfg::A_STAGE + sub * A_STAGE_BYTES);
            const uint32_t sb = smem_u32(smem_b + stage * Cfg::B_STAGE_BYTES + sub * Cfg::B_SUB_BYTES);
            const int k0 = (kb * Cfg::KSUB + sub) * BK;   // past K: the load returns zeros
            if (!p.a_mn) {
              tma_load_4d(sa, &tmap_a, fb, k0, m0, bi, bo);
            } else {
#pragma unroll
              for (int c = 0; c < BM / 64; ++c)
                tma_load_4d(sa + c * (64 * BK * 2), &tmap_a, fb, m0 + 64 * c, k0, bi, bo);
            }
            if (!p.b_mn) {
              tma_load_4d(sb, &tmap_b, fb, k0, n0, bi, bo);
            } else {
#pragma unroll
              for (int c = 0; c < BN / 64; ++c)
                tma_load_4d(sb + c * (64 * BK * 2), &tmap_b, fb, n0 + 64 * c, k0, bi, bo);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // Tail: the last commits onto the "empty" barriers land asynchronously; wait for them
      // so nothing is still on its way when the CTA exits.
      for (int s = 0; ok && s < STAGES; ++s) {
        if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, &g_gemm_error, 5))
          ok = false;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) {
        // Give loads already in flight time to land before the CTA releases its
        // shared memory.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp_idx == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn, p.b_mn);
      // K-major: 8-row groups 1024 B apart, k-step of 16 elements = 32 B inside the span.
      // MN-major: 64-element chunks 64*BK*2 B apart (LBO), 8-k groups 1024 B apart (SBO),
      //           k-step of 16 = two groups = 2048 B.
      const uint32_t a_lbo = p.a_mn ? 64 * BK * 2 : 16, b_lbo = p.b_mn ? 64 * BK * 2 : 16;
      const uint32_t a_step = p.a_mn ? (2048 >> 4) : (32 >> 4);
      const uint32_t b_step = p.b_mn ? (2048 >> 4) : (32 >> 4);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int b = tile / tiles_per_batch;
        const int t = tile - b * tiles_per_batch;
        const int m0 = (t % p.tiles_m) * BM;
        const int n0 = (t / p.tiles_m) * BN;
        if (tile_skipped(m0, n0)) continue;
        if (!mbar_wait_bounded(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag,
                               &g_gemm_error, 2)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int nkb = tile_stages(m0);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&full_bar[stage]), phase, abort_flag, &g_gemm_error,
                                 3)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < Cfg::KSUB; ++sub) {
            const uint64_t a_desc = make_smem_desc_sw128(
                smem_u32(smem_a + stage * Cfg::A_STAGE + sub * A_STAGE_BYTES), a_lbo, 1024);
            const uint64_t b_desc = make_smem_desc_sw128(
                smem_u32(smem_b + stage * Cfg::B_STAGE_BYTES + sub * Cfg::B_SUB_BYTES), b_lbo, 1024);
#pragma unroll
            for (int j = 0; j < BK / UMMA_K; ++j) {
              umma_bf16(d_tmem, a_desc + (uint64_t)(j * a_step), b_desc + (uint64_t)(j * b_step),
                        idesc, (kb > 0 || sub > 0 || j > 0) ? 1u : 0u);
            }
          }
          umma_commit(smem_u32(&empty_bar[stage]));  // frees the smem stage when MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&tmem_full_bar[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp_idx & 3;  // TMEM lane quadrant this warp may read
    const int half = (warp_idx - 2) >> 2;         // which slice of the tile's columns
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int b = tile / tiles_per_batch;
      const int t = tile - b * tiles_per_batch;
      const int m0 = (t % p.tiles_m) * BM;
      const int n0 = (t / p.tiles_m) * BN;
      if (tile_skipped(m0, n0)) continue;
      const int bi = b % p.batch_inner, bo = b / p.batch_inner;
      if (!mbar_wait_bounded_warp(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, &g_gemm_error,
                             4)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      epilogue_tile<BN>(p, tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN, m0, n0, bi, bo,
                        quad, half, lane);
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp_idx == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (p.late_wait) pdl_wait();   // this grid completes only after its predecessor has
}

// ------------------------------------------------------------------------------
// All-gather of B fused into the pair kernel (see GemmGather in gemm.h).
// ------------------------------------------------------------------------------
#ifndef LT_PAIR_KSUB
#define LT_PAIR_KSUB 2
#endif
constexpr int GS_START = 0, GS_DONE = 16;        // signal-pad slots, as in csrc/comm/comm_kernels.cu
constexpr long long GATHER_BUDGET = 6000000000ll;  // about three seconds of SM clocks

__device__ __forceinline__ void g_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t g_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t g_ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 g_ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void epi_bar() {
  asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
}
__device__ void g_report(int* status, int code, int rank, uint32_t epoch, int phase, int peer,
                         uint32_t seen) {
  if (!status) return;
  if (atomicCAS(&status[0], 0, code) == 0) {
    status[1] = rank; status[2] = (int)epoch; status[3] = phase; status[4] = peer;
    status[5] = (int)seen;
  }
}
// Bounded wait until *flag (signed distance) reaches `target`; acquire at gpu or system scope.
template <bool SYS>
__device__ bool g_wait_flag(const uint32_t* flag, uint32_t target, const KernelParams& p, int phase,
                            int peer) {
  const long long t0 = clock64();
  unsigned spins = 0;
  while (true) {
    const uint32_t seen = SYS ? g_ld_acquire_sys(flag) : g_ld_acquire_gpu(flag);
    if ((int32_t)(seen - target) >= 0) return true;
    if ((++spins & 0xff) == 0) {
      if (p.g_status && ((volatile int*)p.g_status)[0] != 0) return false;
      if (clock64() - t0 > GATHER_BUDGET) {
        g_report(p.g_status, 2, p.g_rank, p.g_epoch, phase, peer, seen);
        return false;
      }
    }
    __nanosleep(64);
  }
}

// Run by the 32 * EPI_WARPS epilogue threads of every CTA before their first tile.
__device__ void gather_remote_shards(const KernelParams& p, int t, int* sh_fail) {
  const int W = p.g_world, rank = p.g_rank;
  if (t == 0) *sh_fail = 0;
  if (blockIdx.x == 0 && t < W) {
    __threadfence_system();   // the local shard was written by earlier kernels of this stream
    g_st_release_sys(reinterpret_cast<uint32_t*>(p.g_signal_ptrs[t]) + GS_START + rank, p.g_epoch);
  }
  epi_bar();
  if (t < W) {
    const uint32_t* my_pad = reinterpret_cast<const uint32_t*>(p.g_signal_ptrs[rank]);
    if (!g_wait_flag<true>(my_pad + GS_START + t, p.g_epoch, p, 1, t)) *sh_fail = 1;
  }
  epi_bar();
  const bool failed = *sh_fail != 0;
  const long long R = p.g_rows_per_shard, nv = p.N / 8;
  const long long total = R * nv;
  const long long stride = (long long)gridDim.x * (32 * EPI_WARPS);
  char* local = reinterpret_cast<char*>(p.g_b_ptrs[rank]);
  for (int s = 1; s < W; ++s) {
    const int peer = (rank + s) % W;
    if (!failed) {
      const char* src = reinterpret_cast<const char*>(p.g_b_ptrs[peer]);
      for (long long v0 = (long long)blockIdx.x * (32 * EPI_WARPS) + t; v0 < total; v0 += 4 * stride) {
        uint4 d[4];
        long long off[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const long long v = v0 + u * stride;
          off[u] = -1;
          if (v < total) {
            const long long row = (long long)peer * R + v / nv;
            off[u] = (row * p.g_ldb + (v % nv) * 8) * 2;
            d[u] = g_ld_peer16(src + off[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (off[u] >= 0) *reinterpret_cast<uint4*>(local + off[u]) = d[u];
      }
    }
    asm volatile("fence.proxy.async;" ::: "memory");   // these rows are read through TMA next
    __threadfence();
    epi_bar();
    // counted even after a failure, so that no producer waits for a shard in vain (the error
    // is already recorded in the status words)
    if (t == 0) atomicAdd(&p.g_flags[peer], 1u);
  }
  if (p.g_done && t == 0) {
    // the last CTA to finish its copies tells every peer that its shard is no longer read
    const unsigned ticket = atomicAdd(&p.g_flags[W], 1u);
    if (ticket == gridDim.x - 1) {
      for (int q = 0; q < W; ++q)
        g_st_release_sys(reinterpret_cast<uint32_t*>(p.g_signal_ptrs[q]) + GS_DONE + rank, p.g_epoch);
    }
  }
}

// ------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs (two SMs) owns one 256 x BN output tile.  CTA r holds
// rows [128 r, 128 r + 128) of the A tile, columns [r BN/2, (r+1) BN/2) of the B tile and the
// accumulator rows of its half; the even CTA issues tcgen05.mma.cta_group::2 for both.  Each SM
// therefore stages and reads only half of B, which halves the shared-memory traffic per FLOP
// relative to the single-CTA kernel.  Barrier protocol per stage:
//   full  (even CTA only): its producer arms it with the bytes of BOTH CTAs' loads; the odd
//          CTA's loads credit their bytes to the same barrier through its cluster address;
//   empty (both CTAs): the MMA thread commits to the local one and to the peer's, so each
//          producer refills its own stage when the MMAs that read it have retired;
//   tmem_full (both CTAs) / tmem_empty (even CTA, one arrive per epilogue warp of both CTAs).
// ------------------------------------------------------------------------------
template <int BN>
struct PairCfg {
  static constexpr int KSUB = LT_PAIR_KSUB;             // 64-wide k blocks per pipeline stage
  static constexpr int B_ROWS = BN / 2;                 // B-tile rows (n) held by one CTA
  static constexpr int B_SUB_BYTES = B_ROWS * BK * 2;
  static constexpr int A_STAGE = A_STAGE_BYTES * KSUB;
  static constexpr int B_STAGE_BYTES = B_SUB_BYTES * KSUB;
  static constexpr int STAGE_BYTES = A_STAGE + B_STAGE_BYTES;
  static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES;  // 3 at BN=256, 4 at BN=128
  static constexpr int TMEM_COLS = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b, const KernelParams p) {
  using Cfg = PairCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * Cfg::A_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full_bar = bars + 2 * STAGES;
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_base_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_holder + 1);
  int* gather_fail = reinterpret_cast<int*>(tmem_base_holder + 2);

  const int warp_idx = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_cta_rank();   // 0 = even CTA (issues the MMAs), 1 = odd
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 2 * EPI_WARPS);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp_idx == 1) {
    tmem_alloc_pair(smem_u32(tmem_base_holder), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();          // the peer's barriers exist before anything is sent to them
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_holder;
  if (!p.late_wait) pdl_wait();   // the previous kernel's results are final from here on
  pdl_trigger();                  // after the wait: see gemm_tcgen05_kernel

  const int num_kb = (p.K + BK * Cfg::KSUB - 1) / (BK * Cfg::KSUB);
  const int tiles_per_batch = p.tiles_m * p.tiles_n;     // tiles_m counts 256-row pair tiles
  const int total_tiles = tiles_per_batch * p.batch_total;

  if (warp_idx == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // fused all-gather: start every tile's k loop at the local shard and wait for a remote
      // shard only when its rows are first needed
      const bool gather = p.g_world > 1;
      const int kb_start = gather ? (p.g_rank * p.g_rows_per_shard) / (BK * Cfg::KSUB) : 0;
      uint32_t shard_ready = gather ? (1u << p.g_rank) : 0xffffffffu;
      for (int tile = cluster_id; ok && tile < total_tiles; tile += num_clusters) {
        const int b = tile / tiles_per_batch;
        const int t = tile - b * tiles_per_batch;
        const int m0 = (t % p.tiles_m) * (2 * BM) + (int)cta_rank * BM;
        const int n0 = (t / p.tiles_m) * BN + (int)cta_rank * Cfg::B_ROWS;
        const int bi = b % p.batch_inner, bo = b / p.batch_inner;
        for (int kbi = 0; kbi < num_kb; ++kbi) {
          int kb = kbi + kb_start;
          if (kb >= num_kb) kb -= num_kb;
          if (gather) {
            const int r_lo = kb * Cfg::KSUB * BK, r_hi = r_lo + Cfg::KSUB * BK - 1;
            int q_lo = r_lo / p.g_rows_per_shard, q_hi = r_hi / p.g_rows_per_shard;
            if (q_hi > p.g_world - 1) q_hi = p.g_world - 1;
            bool waited = false;
            for (int q = q_lo; ok && q <= q_hi; ++q) {
              if (!((shard_ready >> q) & 1u)) {
                if (!g_wait_flag<false>(p.g_flags + q, gridDim.x, p, 3, q)) {
                  *abort_flag = 1;
                  ok = false;
                }
                shard_ready |= 1u << q;
                waited = true;
              }
            }
            if (!ok) break;
            if (waited) asm volatile("fence.proxy.async;" ::: "memory");
          }
          if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag,
                                 &g_gemm_error, 11)) {
            ok = false;
            break;
          }
          // bytes of both CTAs land on the even CTA's barrier
          const uint32_t fb = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (cta_rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * Cfg::STAGE_BYTES);
#pragma unroll
          for (int sub = 0; sub < Cfg::KSUB; ++sub) {
            const uint32_t sa = smem_u32(smem_a + stage * Cfg::A_STAGE + sub * A_STAGE_BYTES);
            const uint32_t sb = smem_u32(smem_b + stage * Cfg::B_STAGE_BYTES + sub * Cfg::B_SUB_BYTES);
            const int k0 = (kb * Cfg::KSUB + sub) * BK;   // past K: the load returns zeros
            if (!p.a_mn) {
              tma_load_4d_pair(sa, &tmap_a, fb, k0, m0, bi, bo);
            } else {
#pragma unroll
              for (int c = 0; c < BM / 64; ++c)
                tma_load_4d_pair(sa + c * (64 * BK * 2), &tmap_a, fb, m0 + 64 * c, k0, bi, bo);
            }
            if (!p.b_mn) {
              tma_load_4d_pair(sb, &tmap_b, fb, k0, n0, bi, bo);
            } else {
#pragma unroll
              for (int c = 0; c < Cfg::B_ROWS / 64; ++c)
                tma_load_4d_pair(sb + c * (64 * BK * 2), &tmap_b, fb, n0 + 64 * c, k0, bi, bo);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // Tail: the MMA thread's commits reach this CTA's "empty" barriers asynchronously (for
      // the odd CTA from the other SM); nothing may still be on its way when the CTA exits
      // and its shared memory is handed to another block.
      for (int s = 0; ok && s < STAGES; ++s) {
        if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, &g_gemm_error, 15))
          ok = false;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp_idx == 1) {
    // ----------------------- MMA issuer (even CTA only) -----------------------
    if (lane == 0 && cta_rank == 0) {
      const uint32_t idesc = make_idesc_bf16(2 * BM, BN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? 64 * BK * 2 : 16, b_lbo = p.b_mn ? 64 * BK * 2 : 16;
      const uint32_t a_step = p.a_mn ? (2048 >> 4) : (32 >> 4);
      const uint32_t b_step = p.b_mn ? (2048 >> 4) : (32 >> 4);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; ok && tile < total_tiles; tile += num_clusters) {
        if (!mbar_wait_bounded(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag,
                               &g_gemm_error, 12)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&full_bar[stage]), phase, abort_flag, &g_gemm_error,
                                 13)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < Cfg::KSUB; ++sub) {
            const uint64_t a_desc = make_smem_desc_sw128(
                smem_u32(smem_a + stage * Cfg::A_STAGE + sub * A_STAGE_BYTES), a_lbo, 1024);
            const uint64_t b_desc = make_smem_desc_sw128(
                smem_u32(smem_b + stage * Cfg::B_STAGE_BYTES + sub * Cfg::B_SUB_BYTES), b_lbo, 1024);
#pragma unroll
            for (int j = 0; j < BK / UMMA_K; ++j) {
              umma_bf16_pair(d_tmem, a_desc + (uint64_t)(j * a_step),
                             b_desc + (uint64_t)(j * b_step), idesc,
                             (kb > 0 || sub > 0 || j > 0) ? 1u : 0u);
            }
          }
          // the stage is free in both CTAs once these MMAs have retired
          umma_commit_pair(smem_u32(&empty_bar[stage]));
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(smem_u32(&tmem_full_bar[acc]));
        umma_commit_pair(map_to_cta(smem_u32(&tmem_full_bar[acc]), 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp_idx & 3;
    const int half = (warp_idx - 2) >> 2;
    if (p.g_world > 1) gather_remote_shards(p, (int)threadIdx.x - 64, gather_fail);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = cluster_id; ok && tile < total_tiles; tile += num_clusters) {
      const int b = tile / tiles_per_batch;
      const int t = tile - b * tiles_per_batch;
      const int m0 = (t % p.tiles_m) * (2 * BM) + (int)cta_rank * BM;
      const int n0 = (t / p.tiles_m) * BN;
      const int bi = b % p.batch_inner, bo = b / p.batch_inner;
      if (!mbar_wait_bounded_warp(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, &g_gemm_error,
                             14)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      epilogue_tile<BN>(p, tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN, m0, n0, bi, bo,
                        quad, half, lane);
      tc_fence_before_sync();
      __syncwarp();
      // relaxed: the barrier only hands the accumulator columns back, and this warp's TMEM
      // reads are complete (tcgen05.wait::ld, tcgen05 fence above); a release at cluster scope
      // would first wait for the tile's global stores to reach L2 (2-3 us per launch)
      if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (p.g_world > 1 && p.g_done && (int)threadIdx.x - 64 < p.g_world) {
      // our shard may be rewritten after this kernel: wait until no peer reads it any more
      const int q = (int)threadIdx.x - 64;
      const uint32_t* my_pad = reinterpret_cast<const uint32_t*>(p.g_signal_ptrs[p.g_rank]);
      g_wait_flag<true>(my_pad + GS_DONE + q, p.g_epoch, p, 2, q);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();          // neither CTA frees TMEM or leaves while the other still works
  cluster_wait();
  if (warp_idx == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
  if (p.late_wait) pdl_wait();
}

// ------------------------------------------------------------------------------
// SIMT fallback: any stride / alignment, same epilogue. Only meant for the small or
// misaligned shapes TMA cannot address (e.g. a [256, 10] classifier head).
// ------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ B,
                 long long a_sm, long long a_sk, long long b_sk, long long b_sn,
                 long long a_stride_inner, long long a_stride_outer, long long b_stride_inner,
                 long long b_stride_outer, KernelParams p) {
  constexpr int T = 32, KT = 32;
  __shared__ float sa[KT][T + 1];
  __shared__ float sb[KT][T + 1];
  const int b = blockIdx.z;
  const int bi = b % p.batch_inner, bo = b / p.batch_inner;
  A += bi * a_stride_inner + bo * a_stride_outer;
  B += bi * b_stride_inner + bo * b_stride_outer;
  const size_t esz = p.c_fp32 ? 4 : 2;
  char* c_base = (char*)p.C + (size_t)(bi * p.c_stride_inner + bo * p.c_stride_outer) * esz;
  const int m0 = blockIdx.y * T, n0 = blockIdx.x * T;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 2x2 outputs each
  float acc[2][2] = {{0, 0}, {0, 0}};
  for (int k0 = 0; k0 < p.K; k0 += KT) {
    for (int i = threadIdx.x; i < T * KT; i += 256) {
      int kk, mm;
      if (a_sk == 1) { kk = i % KT; mm = i / KT; } else { mm = i % T; kk = i / T; }
      int m = m0 + mm, k = k0 + kk;
      sa[kk][mm] = (m < p.M && k < p.K) ? __bfloat162float(A[m * a_sm + k * a_sk]) : 0.0f;
      int nn;
      if (b_sk == 1) { kk = i % KT; nn = i / KT; } else { nn = i % T; kk = i / T; }
      int n = n0 + nn;
      k = k0 + kk;
      sb[kk][nn] = (n < p.N && k < p.K) ? __bfloat162float(B[k * b_sk + n * b_sn]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < KT; ++kk) {
      float a0 = sa[kk][ty], a1 = sa[kk][ty + 16];
      float b0 = sb[kk][tx], b1 = sb[kk][tx + 16];
      acc[0][0] += a0 * b0; acc[0][1] += a0 * b1;
      acc[1][0] += a1 * b0; acc[1][1] += a1 * b1;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
      if (m < p.M && n < p.N) epilogue_store_scalar(p, c_base, m, n, acc[i][j]);
    }
}

// ------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault,
                                         &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 4-D bf16 tensor map: (inner, rows, batch_inner, batch_outer), 128-byte swizzle.
bool encode_operand_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows,
                        uint64_t nbi, uint64_t nbo, int64_t ld, int64_t stride_bi,
                        int64_t stride_bo, uint32_t box_inner, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  if (stride_bi <= 0) stride_bi = ld * (int64_t)rows;
  if (stride_bo <= 0) stride_bo = stride_bi * (int64_t)nbi;
  cuuint64_t dims[4] = {inner, rows, nbi, nbo};
  cuuint64_t strides[3] = {(cuuint64_t)ld * 2, (cuuint64_t)stride_bi * 2,
                           (cuuint64_t)stride_bo * 2};
  cuuint32_t box[4] = {box_inner, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

std::atomic<uint64_t> g_launches{0};

int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

KernelParams make_params(const GemmArgs& a) {
  KernelParams p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.tiles_m = 0; p.tiles_n = 0;
  p.batch_inner = a.batch_inner < 1 ? 1 : a.batch_inner;
  p.batch_total = p.batch_inner * (a.batch_outer < 1 ? 1 : a.batch_outer);
  p.a_mn = a.a_mn_major; p.b_mn = a.b_mn_major;
  p.C = a.C; p.ldc = a.ldc;
  p.c_stride_inner = a.c_stride_inner; p.c_stride_outer = a.c_stride_outer;
  p.alpha = a.alpha; p.c_fp32 = a.c_fp32; p.accumulate = a.accumulate;
  p.bias = a.bias; p.bias_fp32 = a.bias_fp32; p.act = a.act;
  p.residual = (const __nv_bfloat16*)a.residual; p.ldr = a.ldr;
  p.aux_out = (__nv_bfloat16*)a.aux_out;
  p.aux_in = (const __nv_bfloat16*)a.aux_in; p.ld_aux = a.ld_aux;
  p.causal_tiles = a.causal_tiles;
  p.causal_k = a.causal_k;
  const int cvec = a.c_fp32 ? 4 : 8;
  bool v = aligned16(a.C) && (a.ldc % cvec == 0) && (a.c_stride_inner % cvec == 0) &&
           (a.c_stride_outer % cvec == 0);
  if (a.bias) v = v && aligned16(a.bias);
  if (a.residual) v = v && aligned16(a.residual) && (a.ldr % 8 == 0);
  if (a.aux_out) v = v && aligned16(a.aux_out) && (a.ldc % 8 == 0);
  if (a.aux_in) v = v && aligned16(a.aux_in) && (a.ld_aux % 8 == 0);
  p.vec_ok = v ? 1 : 0;
  auto a32 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31) == 0; };
  bool w = v && !a.c_fp32 && a32(a.C) && a.ldc % 16 == 0 && a.c_stride_inner % 16 == 0 &&
           a.c_stride_outer % 16 == 0;
  if (a.residual) w = w && a32(a.residual) && a.ldr % 16 == 0;
  if (a.aux_out) w = w && a32(a.aux_out);
  if (a.aux_in) w = w && a32(a.aux_in) && a.ld_aux % 16 == 0;
  p.vec32_ok = w ? 1 : 0;
  p.c32_ok = (v && a.c_fp32 && a32(a.C) && a.ldc % 8 == 0 && a.c_stride_inner % 8 == 0 &&
              a.c_stride_outer % 8 == 0) ? 1 : 0;
  p.late_wait = 0;   // set by the launcher (launch_late)
  p.g_b_ptrs = nullptr; p.g_signal_ptrs = nullptr; p.g_flags = nullptr; p.g_status = nullptr;
  p.g_ldb = 0; p.g_rank = 0; p.g_world = 1; p.g_rows_per_shard = 0; p.g_done = 0; p.g_epoch = 0;
  if (a.gather && a.gather->world > 1) {
    const GemmGather& g = *a.gather;
    p.g_b_ptrs = g.b_ptrs; p.g_signal_ptrs = g.signal_ptrs; p.g_flags = g.flags;
    p.g_status = g.status; p.g_ldb = a.ldb; p.g_rank = g.rank; p.g_world = g.world;
    p.g_rows_per_shard = a.K / g.world; p.g_done = g.done_barrier; p.g_epoch = g.epoch;
  }
  return p;
}

template <int BN>
cudaError_t launch_tc(const GemmArgs& a, cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  KernelParams p = make_params(a);
  p.tiles_m = (a.M + BM - 1) / BM;
  p.tiles_n = (a.N + BN - 1) / BN;
  CUtensorMap ta, tb;
  const uint64_t nbi = p.batch_inner, nbo = p.batch_total / p.batch_inner;
  bool ok;
  if (!a.a_mn_major)
    ok = encode_operand_map(&ta, a.A, a.K, a.M, nbi, nbo, a.lda, a.a_stride_inner,
                            a.a_stride_outer, BK, BM);
  else
    ok = encode_operand_map(&ta, a.A, a.M, a.K, nbi, nbo, a.lda, a.a_stride_inner,
                            a.a_stride_outer, 64, BK);
  if (!a.b_mn_major)
    ok = ok && encode_operand_map(&tb, a.B, a.K, a.N, nbi, nbo, a.ldb, a.b_stride_inner,
                                  a.b_stride_outer, BK, BN);
  else
    ok = ok && encode_operand_map(&tb, a.B, a.N, a.K, nbi, nbo, a.ldb, a.b_stride_inner,
                                  a.b_stride_outer, 64, BK);
  if (!ok) return cudaErrorInvalidValue;
  const long long total = (long long)p.tiles_m * p.tiles_n * p.batch_total;
  const int grid = (int)(total < num_sms() ? total : num_sms());
  const LateWait lw = late_wait_begin(a.overlap_prev);
  p.late_wait = lw.on;
  cudaError_t le = launch_pdl(gemm_tcgen05_kernel<BN>, dim3(grid), dim3(NUM_THREADS), Cfg::SMEM_BYTES, stream, ta, tb, p);
  late_wait_commit(lw);
  if (le != cudaSuccess) return le;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

// Number of CTA pairs the device can keep resident at once for the pair kernel.
template <int BN>
int pair_clusters() {
  static int n = -1;
  if (n < 0) {
    cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         PairCfg<BN>::SMEM_BYTES);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * num_sms());
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = PairCfg<BN>::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int c = 0;
    if (cudaOccupancyMaxActiveClusters(&c, gemm_tcgen05_pair_kernel<BN>, &cfg) != cudaSuccess || c <= 0) {
      cudaGetLastError();
      c = 0;
    }
    if (getenv("LT_GEMM_DEBUG")) fprintf(stderr, "pair_clusters<%d> = %d\n", BN, c);
    n = c;
  }
  return n;
}

template <int BN>
cudaError_t launch_pair(const GemmArgs& a, cudaStream_t stream) {
  using Cfg = PairCfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int clusters = pair_clusters<BN>();
  if (clusters <= 0) return cudaErrorNotSupported;
  KernelParams p = make_params(a);
  p.tiles_m = (a.M + 2 * BM - 1) / (2 * BM);
  p.tiles_n = (a.N + BN - 1) / BN;
  CUtensorMap ta, tb;
  const uint64_t nbi = p.batch_inner, nbo = p.batch_total / p.batch_inner;
  bool ok;
  if (!a.a_mn_major)
    ok = encode_operand_map(&ta, a.A, a.K, a.M, nbi, nbo, a.lda, a.a_stride_inner,
                            a.a_stride_outer, BK, BM);
  else
    ok = encode_operand_map(&ta, a.A, a.M, a.K, nbi, nbo, a.lda, a.a_stride_inner,
                            a.a_stride_outer, 64, BK);
  if (!a.b_mn_major)
    ok = ok && encode_operand_map(&tb, a.B, a.K, a.N, nbi, nbo, a.ldb, a.b_stride_inner,
                                  a.b_stride_outer, BK, Cfg::B_ROWS);
  else
    ok = ok && encode_operand_map(&tb, a.B, a.N, a.K, nbi, nbo, a.ldb, a.b_stride_inner,
                                  a.b_stride_outer, 64, BK);
  if (!ok) return cudaErrorInvalidValue;
  const long long total = (long long)p.tiles_m * p.tiles_n * p.batch_total;
  const int grid = 2 * (int)(total < clusters ? total : clusters);
  const LateWait lw = late_wait_begin(a.overlap_prev);
  p.late_wait = lw.on;
  cudaError_t le = launch_pdl(gemm_tcgen05_pair_kernel<BN>, dim3(grid), dim3(NUM_THREADS), Cfg::SMEM_BYTES, stream, ta, tb, p);
  late_wait_commit(lw);
  if (le != cudaSuccess) return le;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

// 0 = single-CTA kernels only, 1 = CTA pairs where the shape allows (default); the
// LT_GEMM_PAIR environment variable overrides, LT_GEMM_BN forces a tile width (tuning aids).
int pair_mode() {
  static int m = -1;
  if (m < 0) {
    const char* e = getenv("LT_GEMM_PAIR");
    m = e ? atoi(e) : 1;
  }
  return m;
}
int forced_bn() {
  static int m = -1;
  if (m < 0) {
    const char* e = getenv("LT_GEMM_BN");
    m = e ? atoi(e) : 0;
  }
  return m;
}

cudaError_t launch_simt(const GemmArgs& a, cudaStream_t stream) {
  KernelParams p = make_params(a);
  p.vec_ok = 0;
  long long a_sm = a.a_mn_major ? 1 : a.lda, a_sk = a.a_mn_major ? a.lda : 1;
  long long b_sk = a.b_mn_major ? a.ldb : 1, b_sn = a.b_mn_major ? 1 : a.ldb;
  dim3 grid((a.N + 31) / 32, (a.M + 31) / 32, p.batch_total);
  gemm_simt_kernel<<<grid, 256, 0, stream>>>(
      (const __nv_bfloat16*)a.A, (const __nv_bfloat16*)a.B, a_sm, a_sk, b_sk, b_sn,
      a.a_stride_inner, a.a_stride_outer, a.b_stride_inner, a.b_stride_outer, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace

bool gemm_uses_tensor_cores(const GemmArgs& a) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return false;
  if (!aligned16(a.A) || !aligned16(a.B)) return false;
  if (a.lda % 8 || a.ldb % 8) return false;
  if (a.a_stride_inner % 8 || a.a_stride_outer % 8 || a.b_stride_inner % 8 ||
      a.b_stride_outer % 8)
    return false;
  // Tiny problems are not worth a 128-row tile (a small output with a long K is not tiny:
  // convolution weight gradients have K = batch x pixels).
  if ((long long)a.M * a.N < 64 * 64 && a.K < 1024 && a.batch_inner * a.batch_outer == 1) return false;
  if (a.N < 8) return false;
  return true;
}

namespace {

struct TileChoice { int pair = 0, bn = 128; double cost = 1e30; };

// Candidates: CTA-pair tiles (256 x BN over two SMs) and single-CTA tiles (128 x BN).  Each is
// costed with a small model fitted to measurements on B200: a tile takes the longest of
//   its pipeline stages (per stage the slower of the MMAs, BN/2 cycles each, and the operand
//                     feed: about 0.17 us of barrier hand-off plus the bytes at the ~140 GB/s one
//                     SM pulls through TMA),
//   the chip-wide L2 -> SM traffic of the wave at about 12.5 TB/s,
//   its epilogue     (128 x BN outputs per CTA, about 3 TB/s of stores over the chip),
// tiles run in waves over the resident CTAs / CTA pairs, and a launch costs a fixed few
// microseconds (more for cluster launches).
TileChoice choose_tile(const GemmArgs& a, int K, long long batch, bool c_fp32, bool pair_only = false) {
  struct Cand { int pair, bn; };
  const Cand cands[7] = {{1, 256}, {1, 192}, {1, 128}, {0, 256}, {0, 192}, {0, 128}, {0, 64}};
  const int sms = num_sms();
  const bool pair_ok = pair_mode() != 0 && a.causal_tiles == 0 && a.causal_k == 0 && a.M > BM;
  const int force = forced_bn();
  const int clusters = pair_ok ? pair_clusters<256>() : 0;
  TileChoice best;
  for (int i = 0; i < 7; ++i) {
    const Cand& c = cands[i];
    const int bn = c.bn;
    if (force && bn != force) continue;
    if (pair_only && !c.pair) continue;
    if (c.pair) {
      if (clusters <= 0) continue;
      if (a.b_mn_major && (bn / 2) % 64 != 0) continue;   // MN-major B arrives in 64-column chunks
    }
    if (bn > 64 && a.N <= bn / 2) continue;
    const int rows = c.pair ? 2 * BM : BM;
    const long long units = c.pair ? clusters : sms;
    const long long tiles = ((a.M + rows - 1) / rows) * ((a.N + bn - 1) / bn) * batch;
    const double ctas = (double)(c.pair ? 2 * units : units);
    const int ksub = c.pair ? PairCfg<256>::KSUB : (bn <= 128 ? 2 : 1);
    const double stages = (double)((K + BK * ksub - 1) / (BK * ksub));
    const double b_rows = c.pair ? bn / 2.0 : (double)bn;
    const double stage_bytes = ksub * (128.0 + b_rows) * BK * 2.0;
    // per stage: the MMAs, or the hand-off plus the bytes at what one SM pulls through TMA
    const double s_mma = ksub * 4.0 * (bn / 2.0) / 1.7e9 * 1.1;
    const double s_feed = 0.175e-6 + stage_bytes / 142.0e9;
    const double t_cta = stages * (s_mma > s_feed ? s_mma : s_feed) + 0.4e-6;
    // time of one wave in which a fraction `f` of the chip is busy
    auto wave_time = [&](double f) {
      const double t_l2 = ctas * f * stages * stage_bytes / 12.5e12;
      const double t_epi = ctas * f * 128.0 * bn * (c_fp32 ? 4.0 : 2.0) / 3.0e12;
      double t = t_cta > t_l2 ? t_cta : t_l2;
      return t_epi > t ? t_epi : t;
    };
    const long long full = tiles / units, rem = tiles % units;
    const double cost = (c.pair ? 8.5e-6 : 5.5e-6) + (double)full * wave_time(1.0) +
                        (rem ? wave_time((double)rem / (double)units) : 0.0);
    if (cost < best.cost) { best.cost = cost; best.bn = bn; best.pair = c.pair; }
  }
  return best;
}

// Split-K factor for `a` (1 = none) and the tile to use for the slices.
int choose_split(const GemmArgs& a, TileChoice* slice_tile) {
  const long long batch = (long long)(a.batch_inner < 1 ? 1 : a.batch_inner) *
                          (a.batch_outer < 1 ? 1 : a.batch_outer);
  TileChoice whole = choose_tile(a, a.K, batch, a.c_fp32 != 0);
  *slice_tile = whole;
  if (batch != 1 || a.act != GEMM_ACT_NONE || a.residual || a.aux_out || a.aux_in ||
      a.causal_tiles || a.causal_k || a.K < 2048 || getenv("LT_GEMM_NO_SPLIT"))
    return 1;
  // LT_GEMM_SPLIT=n forces a split factor (tuning aid): the slice tile still comes from the model
  static int forced_split = -1;
  if (forced_split < 0) {
    const char* e = getenv("LT_GEMM_SPLIT");
    forced_split = e ? atoi(e) : 0;
  }
  if (forced_split > 1 && a.K % (forced_split * BK) == 0) {
    *slice_tile = choose_tile(a, a.K / forced_split, forced_split, true);
    return forced_split;
  }
  int best_s = 1;
  double best_cost = whole.cost;
  const int splits[14] = {2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 148};
  for (int i = 0; i < 14; ++i) {
    const int s = splits[i];
    if (a.K % (s * BK) != 0 || a.K / s < 8 * BK) continue;
    TileChoice t = choose_tile(a, a.K / s, s, true);
    // the second pass reads S fp32 slices and writes C; it mostly hits in L2
    const double reduce = 4.0e-6 + ((double)s * 4.0 + 4.0) * (double)a.M * (double)a.N / 4.0e12;
    const double cost = t.cost + reduce;
    if (cost < best_cost * 0.9) { best_cost = cost; best_s = s; *slice_tile = t; }
  }
  return best_s;
}

cudaError_t launch_choice(const TileChoice& t, const GemmArgs& a, cudaStream_t stream) {
  if (t.pair) {
    switch (t.bn) {
      case 256: return launch_pair<256>(a, stream);
      case 192: return launch_pair<192>(a, stream);
      default: return launch_pair<128>(a, stream);
    }
  }
  switch (t.bn) {
    case 256: return launch_tc<256>(a, stream);
    case 192: return launch_tc<192>(a, stream);
    case 64: return launch_tc<64>(a, stream);
    default: return launch_tc<128>(a, stream);
  }
}

// C = sum_s ws[s] (+ bias) (+ C), four elements per thread; slices are added in index order.
// The workspace rows are `ws_ld` floats apart (N rounded up to 4); C is written with 16-byte
// accesses when `vec` says its rows allow it, element by element otherwise (N = 27 ...).
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, int splits, long long slice, int M, int N,
                     int ws_ld, void* C, long long ldc, int c_fp32, int accumulate,
                     const void* __restrict__ bias, int bias_fp32, int vec) {
  pdl_enter();
  const int qpr = ws_ld / 4;
  const long long quads = (long long)M * qpr;
  for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q < quads;
       q += (long long)gridDim.x * blockDim.x) {
    const long long row = q / qpr;
    const int col = (int)(q - row * qpr) * 4;
    const float* src = ws + row * ws_ld + col;
    float4 acc = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(src + s * slice);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float r[4] = {acc.x, acc.y, acc.z, acc.w};
    if (bias) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (col + j < N)
          r[j] += bias_fp32 ? ((const float*)bias)[col + j]
                            : __bfloat162float(((const __nv_bfloat16*)bias)[col + j]);
    }
    if (vec) {
      if (c_fp32) {
        float4* dst = reinterpret_cast<float4*>((float*)C + row * ldc + col);
        if (accumulate) { const float4 o = *dst; r[0] += o.x; r[1] += o.y; r[2] += o.z; r[3] += o.w; }
        *dst = make_float4(r[0], r[1], r[2], r[3]);
      } else {
        __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>((__nv_bfloat16*)C + row * ldc + col);
        if (accumulate) {
          const float2 o0 = __bfloat1622float2(dst[0]), o1 = __bfloat1622float2(dst[1]);
          r[0] += o0.x; r[1] += o0.y; r[2] += o1.x; r[3] += o1.y;
        }
        dst[0] = __floats2bfloat162_rn(r[0], r[1]);
        dst[1] = __floats2bfloat162_rn(r[2], r[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (col + j >= N) break;
        if (c_fp32) {
          float* d = (float*)C + row * ldc + col + j;
          *d = accumulate ? *d + r[j] : r[j];
        } else {
          __nv_bfloat16* d = (__nv_bfloat16*)C + row * ldc + col + j;
          *d = __float2bfloat16(accumulate ? __bfloat162float(*d) + r[j] : r[j]);
        }
      }
    }
  }
}

// every output shape can be split; the workspace rows are padded to four floats
bool split_k_shape_ok(const GemmArgs&) { return true; }
inline int ws_ld_of(const GemmArgs& a) { return (a.N + 3) & ~3; }
inline bool reduce_vec_ok(const GemmArgs& a) {
  return a.N % 4 == 0 && a.ldc % 4 == 0 && (reinterpret_cast<uintptr_t>(a.C) & 15) == 0;
}

}  // namespace

size_t gemm_split_k_workspace_bytes(const GemmArgs& a) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || !gemm_uses_tensor_cores(a) || !split_k_shape_ok(a)) return 0;
  TileChoice t;
  const int s = choose_split(a, &t);
  return s > 1 ? (size_t)s * (size_t)a.M * (size_t)ws_ld_of(a) * sizeof(float) : 0;
}

// True while the kernel launched last by gemm_bf16 is a split-K reduction (it reads the
// workspace): a split-K GEMM that follows may then not start before that kernel has finished.
static thread_local bool g_prev_reads_workspace = false;

cudaError_t gemm_bf16(const GemmArgs& args, cudaStream_t stream) {
  if (args.M <= 0 || args.N <= 0) return cudaSuccess;
  if (args.K <= 0) return cudaErrorInvalidValue;
  GemmArgs a = args;
  if (a.gather && a.gather->world > 1) a.overlap_prev = 0;
  if (a.gather && a.gather->world > 1) {
    // B is gathered inside the kernel: CTA-pair path only
    const GemmGather& g = *a.gather;
    const bool ok = gemm_uses_tensor_cores(a) && a.b_mn_major == 1 && a.K % g.world == 0 &&
                    a.N % 8 == 0 && a.batch_inner <= 1 && a.batch_outer <= 1 &&
                    a.causal_tiles == 0 && a.M > BM && g.world <= 16 && g.b_ptrs &&
                    g.signal_ptrs && g.flags;
    if (!ok) return cudaErrorNotSupported;
    TileChoice t = choose_tile(a, a.K, 1, a.c_fp32 != 0, true);
    if (t.cost >= 1e29 || !t.pair) return cudaErrorNotSupported;
    return launch_choice(t, a, stream);
  }
  if (!gemm_uses_tensor_cores(a)) return launch_simt(a, stream);
  TileChoice tile;
  int splits = choose_split(a, &tile);
  const size_t need = (size_t)splits * (size_t)a.M * (size_t)ws_ld_of(a) * sizeof(float);
  if (splits > 1 && (!a.workspace || a.workspace_bytes < need || !split_k_shape_ok(a))) {
    splits = 1;
    tile = choose_tile(a, a.K, 1, a.c_fp32 != 0);
  }
  if (getenv("LT_GEMM_DEBUG"))
    fprintf(stderr, "gemm %dx%dx%d -> %s BN=%d split %d (model %.1f us)\n", a.M, a.N, a.K,
            tile.pair ? "pair" : "single", tile.bn, splits, tile.cost * 1e6);
  if (splits == 1) {
    g_prev_reads_workspace = false;
    return launch_choice(tile, a, stream);
  }
  // K slices as batches into the fp32 workspace, then one deterministic reduction
  if (g_prev_reads_workspace) a.overlap_prev = 0;
  g_prev_reads_workspace = true;
  GemmArgs g = a;
  const int ks = a.K / splits;
  g.K = ks;
  g.batch_inner = splits;
  g.batch_outer = 1;
  g.a_stride_inner = a.a_mn_major ? (int64_t)ks * a.lda : ks;
  g.b_stride_inner = a.b_mn_major ? (int64_t)ks * a.ldb : ks;
  g.a_stride_outer = g.b_stride_outer = 0;
  const int ws_ld = ws_ld_of(a);
  g.C = a.workspace;
  g.ldc = ws_ld;
  g.c_stride_inner = (int64_t)a.M * ws_ld;
  g.bias = nullptr;       // added by the reduction
  g.c_stride_outer = 0;
  g.c_fp32 = 1;
  g.accumulate = 0;
  g.workspace = nullptr;
  cudaError_t e = launch_choice(tile, g, stream);
  if (e != cudaSuccess) return e;
  const long long quads = (long long)a.M * (ws_ld / 4);
  int blocks = (int)((quads + 255) / 256);
  if (blocks > 8 * num_sms()) blocks = 8 * num_sms();
  cudaError_t re = launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream,
                              (const float*)a.workspace, splits, (long long)a.M * ws_ld, a.M, a.N,
                              ws_ld, a.C, (long long)a.ldc, a.c_fp32, a.accumulate, a.bias,
                              a.bias_fp32, reduce_vec_ok(a) ? 1 : 0);
  if (re != cudaSuccess) return re;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

int gemm_last_device_error() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int));
  return v;
}
void gemm_clear_device_error() {
  int v = 0;
  cudaMemcpyToSymbol(g_gemm_error, &v, sizeof(int));
}
uint64_t gemm_launch_count() { return g_launches.load(); }

}  // namespace lt
