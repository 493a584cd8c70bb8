// Flash attention backward on tcgen05 (no counterpart in the reference, which has no
// attention backward at all: lua/luatorch/nn/flash_attention.lua:52-108 never records one).
//
// Three launches, no floating-point atomics, bitwise reproducible:
//   1. delta[b,h,i] = sum_d dO[i,d] * O[i,d]
//   2. dK/dV kernel: one CTA per 128-key tile, loops over the query tiles that see it.
//        S = Q K^T and dP = dO V^T go to TMEM; thread r (query row r) rebuilds
//        P = exp(scale*S - lse) and dS = P * (dP - delta) * scale and stores both as bf16 in
//        the swizzled shared-memory layout; then dV += P^T dO and dK += dS^T Q accumulate in
//        TMEM (the transposes are free: the same shared-memory bytes are described to the
//        tensor core as an MN-major operand).
//   3. dQ kernel: one CTA per 128-query tile, loops over its key tiles, recomputes S / dP,
//        dQ += dS K accumulates in TMEM.
//      When the caller lends a dS scratch buffer (the default at head dim 128), launch 2
//      also stores dS there and dQ = dS K runs as one batched GEMM that skips the key blocks
//      above the causal diagonal (gemm_bf16 with causal_k) instead of launch 3.
#include "attention.h"
#include "sm100_ptx.cuh"
#include "common.cuh"
#include "gemm.h"

#include <cuda.h>
#include <stdio.h>
#include <atomic>

namespace lt {

using namespace ptx;

extern std::atomic<uint64_t> g_attn_launches;
// Status word of the backward kernels (device symbols are per translation unit).
static __device__ int g_attn_error = 0;
int attention_bwd_device_error() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int));
  return v;
}

namespace attn_detail {
bool make_qkv_map(CUtensorMap* map, const void* base, int D, int S, int H, int B, int64_t ss,
                  int64_t sh, int64_t sb, int box_rows);
}

namespace {

constexpr int BT = 128;                  // tile edge (queries and keys)
constexpr int CHUNK_BYTES = 128 * 128;   // 128 rows x 64 bf16
constexpr int COMPUTE_WARPS = 8;          // two per TMEM lane quadrant: each takes half of the key columns
constexpr int NUM_THREADS = 64 + 32 * COMPUTE_WARPS;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct BwdParams {
  int S, H, causal;
  float scale, scale_log2;
  const float* lse;
  const float* delta;
  __nv_bfloat16* out0;  // dK (kernel 2) or dQ (kernel 3)
  long long o0_sb, o0_ss, o0_sh;
  __nv_bfloat16* out1;  // dV (kernel 2)
  long long o1_sb, o1_ss, o1_sh;
  __nv_bfloat16* ds_out;  // optional [B, H, S, S]: dS tiles for the dQ GEMM (dK/dV kernel only)
  int late_wait = 0;      // independent of the previous kernel: wait for it before exit (common.cuh)
};

// ------------------------------------------------------------------ delta = rowsum(dO * O)
// One thread per (batch, position, head) row: D contiguous bf16 of O and dO, 16-byte loads;
// neighbouring threads take neighbouring heads, which are adjacent in memory.
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                  float* __restrict__ delta, int B, int H, int S, int D, long long o_sb,
                  long long o_ss, long long o_sh, long long do_sb, long long do_ss,
                  long long do_sh) {
  pdl_enter();
  const long long r = blockIdx.x * 256ll + threadIdx.x;  // over B*S*H, head fastest
  if (r >= (long long)B * H * S) return;
  const int h = r % H, s = (r / H) % S, b = r / ((long long)S * H);
  const uint4* op = reinterpret_cast<const uint4*>(o + b * o_sb + s * o_ss + h * o_sh);
  const uint4* dp = reinterpret_cast<const uint4*>(d_o + b * do_sb + s * do_ss + h * do_sh);
  float acc = 0.0f;
  for (int i = 0; i < D / 8; ++i) {
    const uint4 x = op[i], y = dp[i];
    const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&x);
    const __nv_bfloat162* yh = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __bfloat1622float2(xh[j]), c = __bfloat1622float2(yh[j]);
      acc += a.x * c.x + a.y * c.y;
    }
  }
  delta[((long long)b * H + h) * S + s] = acc;
}

// Rebuild P and dS for one query row from the S / dP accumulators in TMEM and store them
// (bf16) into the swizzled [query row][key] shared-memory tiles.
template <bool WRITE_P, bool MASKED>
__device__ __forceinline__ void rebuild_chunk(const uint32_t (&s)[32], const uint32_t (&dp)[32],
                                              int valid, float lse_l2, float delta, float c,
                                              float scale, uint8_t* p_dst, uint8_t* ds_dst,
                                              int c32, int row, __nv_bfloat16* ds_global) {
  uint32_t pp[16], dd[16];
  // two scores per instruction on the FMA pipe: x = s c - lse, g = dp scale - delta scale
  const float2 cc = make_float2(c, c), ll = make_float2(-lse_l2, -lse_l2);
  const float2 ss = make_float2(scale, scale), dl = make_float2(-delta * scale, -delta * scale);
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const float2 x = ffma2(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), cc, ll);
    float2 pv = make_float2(ex2(x.x), ex2(x.y));
    if (MASKED) {
      pv.x = (i < valid) ? pv.x : 0.0f;
      pv.y = (i + 1 < valid) ? pv.y : 0.0f;
    }
    const float2 g = ffma2(make_float2(__uint_as_float(dp[i]), __uint_as_float(dp[i + 1])), ss, dl);
    const float2 dv = fmul2(pv, g);
    __nv_bfloat162 hp = __floats2bfloat162_rn(pv.x, pv.y), hd = __floats2bfloat162_rn(dv.x, dv.y);
    pp[i >> 1] = *reinterpret_cast<uint32_t*>(&hp);
    dd[i >> 1] = *reinterpret_cast<uint32_t*>(&hd);
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int chunk16 = (((c32 & 1) * 4 + t) ^ (row & 7)) * 16;
    if (WRITE_P)
      *reinterpret_cast<uint4*>(p_dst + chunk16) =
          make_uint4(pp[4 * t], pp[4 * t + 1], pp[4 * t + 2], pp[4 * t + 3]);
    *reinterpret_cast<uint4*>(ds_dst + chunk16) =
        make_uint4(dd[4 * t], dd[4 * t + 1], dd[4 * t + 2], dd[4 * t + 3]);
  }
  if (ds_global) {   // the same 32 values, row-major, for the dQ GEMM
#pragma unroll
    for (int t = 0; t < 4; ++t)
      *reinterpret_cast<uint4*>(ds_global + 8 * t) =
          make_uint4(dd[4 * t], dd[4 * t + 1], dd[4 * t + 2], dd[4 * t + 3]);
  }
}

// This warp's half (`col_half`) of one query row: two 32-column chunks of S and dP.  No
// reduction across columns is needed in backward, so the halves are independent.  The second
// chunk's TMEM reads are in flight while the first is processed.
template <bool WRITE_P>
__device__ __forceinline__ void rebuild_row(uint32_t tmem_s, uint32_t tmem_dp, uint32_t lane_base,
                                            int row, int valid, bool masked, float lse_l2,
                                            float delta, float c, float scale, uint8_t* p_tile,
                                            uint8_t* ds_tile, int col_half,
                                            __nv_bfloat16* ds_row_global) {
  const int row_off = (row >> 3) * 1024 + (row & 7) * 128 + col_half * CHUNK_BYTES;
  const int col0 = col_half * 64;
  uint32_t s0[32], d0[32], s1[32], d1[32];
  tmem_ld_32x32(tmem_s + lane_base + col0, s0);
  tmem_ld_32x32(tmem_dp + lane_base + col0, d0);
  tmem_ld_wait();
  tmem_ld_32x32(tmem_s + lane_base + col0 + 32, s1);
  tmem_ld_32x32(tmem_dp + lane_base + col0 + 32, d1);
  if (masked) {
    rebuild_chunk<WRITE_P, true>(s0, d0, valid - col0, lse_l2, delta, c, scale, p_tile + row_off,
                                 ds_tile + row_off, 0, row, ds_row_global ? ds_row_global + col0 : nullptr);
    tmem_ld_wait();
    rebuild_chunk<WRITE_P, true>(s1, d1, valid - col0 - 32, lse_l2, delta, c, scale,
                                 p_tile + row_off, ds_tile + row_off, 1, row, ds_row_global ? ds_row_global + col0 + 32 : nullptr);
  } else {
    rebuild_chunk<WRITE_P, false>(s0, d0, 32, lse_l2, delta, c, scale, p_tile + row_off,
                                  ds_tile + row_off, 0, row, ds_row_global ? ds_row_global + col0 : nullptr);
    tmem_ld_wait();
    rebuild_chunk<WRITE_P, false>(s1, d1, 32, lse_l2, delta, c, scale, p_tile + row_off,
                                  ds_tile + row_off, 1, row, ds_row_global ? ds_row_global + col0 + 32 : nullptr);
  }
}

// Store one accumulator row (D fp32 columns in TMEM) as bf16.
template <int D>
__device__ __forceinline__ void store_acc_row(uint32_t taddr, __nv_bfloat16* dst, int first) {
  // the two warps that share a lane quadrant take alternate 32-column chunks
#pragma unroll 1
  for (int c32 = first; c32 < D / 32; c32 += 2) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + c32 * 32, r);
    tmem_ld_wait();
    if (dst) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 u;
        __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int t = 0; t < 4; ++t)
          hb[t] = __floats2bfloat162_rn(__uint_as_float(r[i + 2 * t]),
                                        __uint_as_float(r[i + 2 * t + 1]));
        *reinterpret_cast<uint4*>(dst + c32 * 32 + i) = u;
      }
    }
  }
}

template <int D, bool DKDV>
struct BwdSmem {
  static constexpr int DC = D / 64;
  static constexpr int TILE = DC * CHUNK_BYTES;          // one [128 x D] operand
  static constexpr int STAGES = D == 64 ? 2 : 1;         // streamed operand pair ring depth
  static constexpr int OFF_FIX0 = 0;                     // stationary operand 0 (K or Q)
  static constexpr int OFF_FIX1 = TILE;                  // stationary operand 1 (V or dO)
  static constexpr int OFF_STR = 2 * TILE;               // streamed pairs: [stage][2][TILE]
  static constexpr int OFF_P = OFF_STR + STAGES * 2 * TILE;
  static constexpr int OFF_DS = OFF_P + (DKDV ? 2 * CHUNK_BYTES : 0);
  static constexpr int OFF_BAR = OFF_DS + 2 * CHUNK_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

// DKDV = true : stationary (K_j, V_j), streamed (Q_i, dO_i), outputs dK_j, dV_j
// DKDV = false: stationary (Q_i, dO_i), streamed (K_j, V_j), output dQ_i
template <int D, bool DKDV>
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                 const BwdParams p) {
  using L = BwdSmem<D, DKDV>;
  constexpr int DC = L::DC, ST = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* fix_full = bars;        // 1
  uint64_t* str_full = bars + 1;    // ST
  uint64_t* str_empty = bars + 3;   // ST
  uint64_t* s_full = bars + 5;      // 1  (S and dP ready in TMEM)
  uint64_t* s_empty = bars + 6;     // 1  (compute warps done reading S / dP)
  uint64_t* pds_full = bars + 7;    // 1  (P / dS tiles written)
  uint64_t* pds_empty = bars + 8;   // 1  (MMAs reading P / dS retired)
  uint64_t* acc_full = bars + 9;    // 1  (final accumulators ready)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp_idx = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int n_tiles = (p.S + BT - 1) / BT;
  // DKDV: this CTA owns key tile `own`, streams query tiles [first, n_tiles)
  // dQ  : this CTA owns query tile `own`, streams key tiles [0, last]
  const int own = DKDV ? (int)blockIdx.z : (int)gridDim.z - 1 - (int)blockIdx.z;
  const int it_begin = DKDV ? (p.causal ? own : 0) : 0;
  const int it_end = DKDV ? n_tiles : (p.causal ? own + 1 : n_tiles);
  const int n_it = it_end - it_begin;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(fix_full), 1);
    for (int i = 0; i < ST; ++i) {
      mbar_init(smem_u32(&str_full[i]), 1);
      mbar_init(smem_u32(&str_empty[i]), 1);
    }
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(s_empty), 32 * COMPUTE_WARPS);
    mbar_init(smem_u32(pds_full), 32 * COMPUTE_WARPS);
    mbar_init(smem_u32(pds_empty), 1);
    mbar_init(smem_u32(acc_full), 1);
    fence_mbar_init();
  }
  if (warp_idx == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  pdl_enter();   // operands come from earlier kernels of the stream
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 128;
  const uint32_t tmem_acc0 = tmem_base + 256;        // dK or dQ
  const uint32_t tmem_acc1 = tmem_base + 256 + D;    // dV

  // shared-memory operand tiles; in both kernels "A-side" = the query-indexed pair (Q, dO)
  // and "B-side" = the key-indexed pair (K, V)
  auto fix0 = [&]() { return smem + L::OFF_FIX0; };
  auto fix1 = [&]() { return smem + L::OFF_FIX1; };
  auto str0 = [&](int st) { return smem + L::OFF_STR + st * 2 * L::TILE; };
  auto str1 = [&](int st) { return smem + L::OFF_STR + st * 2 * L::TILE + L::TILE; };

  if (warp_idx == 0) {
    if (lane == 0) {
      const uint32_t fb = smem_u32(fix_full);
      mbar_arrive_expect_tx(fb, 2 * L::TILE);
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        tma_load_4d(smem_u32(fix0() + c * CHUNK_BYTES), DKDV ? &tm_k : &tm_q, fb, 64 * c, own * BT,
                    h, b);
        tma_load_4d(smem_u32(fix1() + c * CHUNK_BYTES), DKDV ? &tm_v : &tm_do, fb, 64 * c,
                    own * BT, h, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % ST, use = it / ST, t = it_begin + it;
        if (!mbar_wait_bounded(smem_u32(&str_empty[st]), (use & 1) ^ 1, abort_flag, &g_attn_error,
                               31))
          break;
        const uint32_t sb = smem_u32(&str_full[st]);
        mbar_arrive_expect_tx(sb, 2 * L::TILE);
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          tma_load_4d(smem_u32(str0(st) + c * CHUNK_BYTES), DKDV ? &tm_q : &tm_k, sb, 64 * c,
                      t * BT, h, b);
          tma_load_4d(smem_u32(str1(st) + c * CHUNK_BYTES), DKDV ? &tm_do : &tm_v, sb, 64 * c,
                      t * BT, h, b);
        }
      }
    }
  } else if (warp_idx == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(BT, BT, 0, 0);
      const uint32_t idesc_kv = make_idesc_bf16(BT, D, 1, 1);  // P^T dO, dS^T Q
      const uint32_t idesc_q = make_idesc_bf16(BT, D, 0, 1);   // dS K
      bool ok = mbar_wait_bounded(smem_u32(fix_full), 0, abort_flag, &g_attn_error, 32);
      // S = Q K^T and dP = dO V^T for iteration `it`
      auto issue_scores = [&](int it) -> bool {
        const int st = it % ST, use = it / ST;
        if (!mbar_wait_bounded(smem_u32(&str_full[st]), use & 1, abort_flag, &g_attn_error, 33))
          return false;
        if (!mbar_wait_bounded(smem_u32(s_empty), (it & 1) ^ 1, abort_flag, &g_attn_error, 34))
          return false;
        tc_fence_after_sync();
        uint8_t* q_t = DKDV ? str0(st) : fix0();
        uint8_t* do_t = DKDV ? str1(st) : fix1();
        uint8_t* k_t = DKDV ? fix0() : str0(st);
        uint8_t* v_t = DKDV ? fix1() : str1(st);
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          const uint64_t qd = make_smem_desc_sw128(smem_u32(q_t + c * CHUNK_BYTES), 16, 1024);
          const uint64_t kd = make_smem_desc_sw128(smem_u32(k_t + c * CHUNK_BYTES), 16, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16(tmem_s, qd + (uint64_t)(ks * 2), kd + (uint64_t)(ks * 2), idesc_s,
                      (c > 0 || ks > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          const uint64_t dd = make_smem_desc_sw128(smem_u32(do_t + c * CHUNK_BYTES), 16, 1024);
          const uint64_t vd = make_smem_desc_sw128(smem_u32(v_t + c * CHUNK_BYTES), 16, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16(tmem_dp, dd + (uint64_t)(ks * 2), vd + (uint64_t)(ks * 2), idesc_s,
                      (c > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(s_full));
        return true;
      };
      if (ok && n_it > 0) ok = issue_scores(0);
      for (int it = 0; ok && it < n_it; ++it) {
        const int st = it % ST;
        if (!mbar_wait_bounded(smem_u32(pds_full), it & 1, abort_flag, &g_attn_error, 35)) {
          ok = false;
          break;
        }
        // with a 2-deep ring the next tile's scores go first so the compute warps restart
        // while the accumulating MMAs below run
        if (ST == 2 && it + 1 < n_it) {
          if (!issue_scores(it + 1)) { ok = false; break; }
        }
        tc_fence_after_sync();
        uint8_t* p_t = smem + L::OFF_P;
        uint8_t* ds_t = smem + L::OFF_DS;
        if (DKDV) {
          uint8_t* q_t = str0(st);
          uint8_t* do_t = str1(st);
          // dV[keys x D] += P^T dO ; dK[keys x D] += dS^T Q.  K dimension = 128 queries:
          // rows of the P / dS / dO / Q tiles, 16 queries = 2048 B per step.
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t pd =
                make_smem_desc_sw128(smem_u32(p_t) + ks * 2048, CHUNK_BYTES, 1024);
            const uint64_t od =
                make_smem_desc_sw128(smem_u32(do_t) + ks * 2048, CHUNK_BYTES, 1024);
            umma_bf16(tmem_acc1, pd, od, idesc_kv, (it > 0 || ks > 0) ? 1u : 0u);
          }
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t sd =
                make_smem_desc_sw128(smem_u32(ds_t) + ks * 2048, CHUNK_BYTES, 1024);
            const uint64_t qd =
                make_smem_desc_sw128(smem_u32(q_t) + ks * 2048, CHUNK_BYTES, 1024);
            umma_bf16(tmem_acc0, sd, qd, idesc_kv, (it > 0 || ks > 0) ? 1u : 0u);
          }
        } else {
          uint8_t* k_t = str0(st);
          // dQ[queries x D] += dS[queries x keys] K[keys x D]; K dimension = 128 keys
#pragma unroll
          for (int kc = 0; kc < 2; ++kc) {
            const uint64_t sd =
                make_smem_desc_sw128(smem_u32(ds_t + kc * CHUNK_BYTES), 16, 1024);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const uint64_t kd = make_smem_desc_sw128(
                  smem_u32(k_t) + (kc * 64 + ks * 16) * 128, CHUNK_BYTES, 1024);
              umma_bf16(tmem_acc0, sd + (uint64_t)(ks * 2), kd, idesc_q,
                        (it > 0 || kc > 0 || ks > 0) ? 1u : 0u);
            }
          }
        }
        umma_commit(smem_u32(pds_empty));
        umma_commit(smem_u32(&str_empty[st]));
        if (ST == 1 && it + 1 < n_it) {
          if (!issue_scores(it + 1)) { ok = false; break; }
        }
      }
      if (ok) umma_commit(smem_u32(acc_full));
    }
  } else {
    const int quad = warp_idx & 3;
    const int col_half = (warp_idx - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = ((uint32_t)(quad * 32)) << 16;
    bool ok = true;
    for (int it = 0; ok && it < n_it; ++it) {
      const int t = it_begin + it;
      const int q_tile = DKDV ? t : own, k_tile = DKDV ? own : t;
      const int qi = q_tile * BT + row, k0 = k_tile * BT;
      int valid = 0;
      float lse_l2 = 0.0f, delta = 0.0f;
      // uniform per tile: does any element of this (query tile, key tile) pair need masking?
      const bool tile_masked = (p.causal && k0 + BT - 1 > q_tile * BT) || (k0 + BT > p.S) ||
                               (q_tile * BT + BT > p.S);
      if (qi < p.S) {
        int lim = p.S - k0;
        if (p.causal) { int cl = qi - k0 + 1; lim = cl < lim ? cl : lim; }
        valid = lim < 0 ? 0 : (lim > BT ? BT : lim);
        const long long idx = ((long long)b * p.H + h) * p.S + qi;
        lse_l2 = p.lse[idx] * LOG2E;
        delta = p.delta[idx];
      }
      if (!mbar_wait_bounded_warp(smem_u32(s_full), it & 1, abort_flag, &g_attn_error, 36) ||
          !mbar_wait_bounded_warp(smem_u32(pds_empty), (it & 1) ^ 1, abort_flag, &g_attn_error, 37)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      __nv_bfloat16* ds_row = nullptr;
      if (DKDV && p.ds_out && qi < p.S)
        ds_row = p.ds_out + (((long long)b * p.H + h) * p.S + qi) * p.S + k0;
      rebuild_row<DKDV>(tmem_s, tmem_dp, lane_base, row, valid, tile_masked, lse_l2, delta,
                        p.scale_log2, p.scale, smem + L::OFF_P, smem + L::OFF_DS, col_half, ds_row);
      tc_fence_before_sync();
      mbar_arrive(smem_u32(s_empty));
      fence_proxy_async();
      mbar_arrive(smem_u32(pds_full));
    }
    if (ok && n_it > 0 &&
        mbar_wait_bounded_warp(smem_u32(acc_full), 0, abort_flag, &g_attn_error, 38)) {
      tc_fence_after_sync();
      const int gi = own * BT + row;  // key index (DKDV) or query index
      const bool in_range = gi < p.S;
      __nv_bfloat16* d0 = in_range ? p.out0 + (long long)b * p.o0_sb + (long long)gi * p.o0_ss +
                                         (long long)h * p.o0_sh
                                   : nullptr;
      store_acc_row<D>(tmem_acc0 + lane_base, d0, col_half);
      if (DKDV) {
        __nv_bfloat16* d1 = in_range ? p.out1 + (long long)b * p.o1_sb + (long long)gi * p.o1_ss +
                                           (long long)h * p.o1_sh
                                     : nullptr;
        store_acc_row<D>(tmem_acc1 + lane_base, d1, col_half);
      }
    } else if (ok && n_it == 0) {
      // a key tile no query attends to (cannot happen for causal self-attention): zero output
      const int gi = own * BT + row;
      if (gi < p.S && col_half == 0) {
        __nv_bfloat16* d0 = p.out0 + (long long)b * p.o0_sb + (long long)gi * p.o0_ss +
                            (long long)h * p.o0_sh;
        for (int i = 0; i < D; ++i) d0[i] = __float2bfloat16(0.0f);
        if (DKDV) {
          __nv_bfloat16* d1 = p.out1 + (long long)b * p.o1_sb + (long long)gi * p.o1_ss +
                              (long long)h * p.o1_sh;
          for (int i = 0; i < D; ++i) d1[i] = __float2bfloat16(0.0f);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp_idx == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// =====================================================================================
// Second-generation backward kernels (head dim 64, sequence length a multiple of 128).
//
// The row index of the STATIONARY operand sits on the TMEM lanes, the streamed operand arrives
// in sub-tiles of 64 rows that become the columns:
//   DKDV = true : lanes = 128 keys of this CTA, columns = 64 queries per step
//                 S^T = K Q^T, dP^T = V dO^T; thread (key) rebuilds P^T and dS^T for its row;
//                 dV += P^T dO and dK += dS^T Q
//   DKDV = false: lanes = 128 queries of this CTA, columns = 64 keys per step
//                 S = Q K^T, dP = dO V^T; thread (query) rebuilds dS; dQ += dS K
// In both cases the rebuilt P / dS tile is exactly the A operand (M = lanes, K = the 64
// streamed rows) of the accumulating MMAs, so it is written back to tensor memory as packed
// bf16 (over the columns its fp32 source occupied) and read from there by tcgen05.mma: no
// shared-memory staging of P or dS, no proxy fences.  A CTA needs 128 + 2 x 64 TMEM columns
// and 80 KB of shared memory, so two CTAs share an SM and one CTA's exponentials run under
// the other's MMAs.
// =====================================================================================
constexpr int SUB = 64;                         // streamed rows per step
constexpr int SUB_CHUNK = SUB * 128;            // 64 rows x 64 bf16
constexpr int B2_THREADS = 64 + 32 * COMPUTE_WARPS;

template <int D>
struct Bwd2Smem {
  static constexpr int DC = D / 64;
  static constexpr int FIX = DC * CHUNK_BYTES;            // one [128 x D] stationary operand
  static constexpr int STR = DC * SUB_CHUNK;              // one [64 x D] streamed operand
  static constexpr int STAGES = 3;
  static constexpr int OFF_FIX0 = 0;
  static constexpr int OFF_FIX1 = FIX;
  static constexpr int OFF_STR = 2 * FIX;                 // [stage][2][STR]
  static constexpr int OFF_SCAL = OFF_STR + STAGES * 2 * STR;   // [stage][2][64] floats: lse, delta
  static constexpr int OFF_BAR = OFF_SCAL + STAGES * 2 * SUB * 4;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 128 + 2 * D <= 256 ? 256 : 512;
};

// 16 columns of one lane's row: scores s and dp (fp32 from TMEM) -> packed bf16 P and dS.
// lse2 / dsc: log2-domain log-sum-exp and delta * scale, per column (COLV) or for the lane.
template <bool COLV, bool MASKED>
__device__ __forceinline__ void rebuild16(const uint32_t (&s)[16], const uint32_t (&dp)[16],
                                          const float* lse2_c, const float* dsc_c, float lse2_l,
                                          float dsc_l, float c, float scale, int lo, int hi,
                                          uint32_t (&pp)[8], uint32_t (&dd)[8]) {
  // columns j with lo <= j < hi are inside the causal / sequence bounds (only when MASKED)
  const float2 cc = make_float2(c, c), ss = make_float2(scale, scale);
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const float2 ll = COLV ? make_float2(-lse2_c[i], -lse2_c[i + 1]) : make_float2(-lse2_l, -lse2_l);
    const float2 dl = COLV ? make_float2(-dsc_c[i], -dsc_c[i + 1]) : make_float2(-dsc_l, -dsc_l);
    const float2 x = ffma2(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), cc, ll);
    float2 pv = make_float2(ex2(x.x), ex2(x.y));
    if (MASKED) {
      pv.x = (i >= lo && i < hi) ? pv.x : 0.0f;
      pv.y = (i + 1 >= lo && i + 1 < hi) ? pv.y : 0.0f;
    }
    const float2 g = ffma2(make_float2(__uint_as_float(dp[i]), __uint_as_float(dp[i + 1])), ss, dl);
    const float2 dv = fmul2(pv, g);
    __nv_bfloat162 hp = __floats2bfloat162_rn(pv.x, pv.y), hd = __floats2bfloat162_rn(dv.x, dv.y);
    pp[i >> 1] = *reinterpret_cast<uint32_t*>(&hp);
    dd[i >> 1] = *reinterpret_cast<uint32_t*>(&hd);
  }
}

template <int D, bool DKDV>
__global__ void __launch_bounds__(B2_THREADS, (D == 64 ? 2 : 1))
flash_bwd2_kernel(const __grid_constant__ CUtensorMap tm_fix0, const __grid_constant__ CUtensorMap tm_fix1,
                  const __grid_constant__ CUtensorMap tm_str0, const __grid_constant__ CUtensorMap tm_str1,
                  const BwdParams p) {
  // DKDV: fix0 = K, fix1 = V (128-row boxes), str0 = Q, str1 = dO (64-row boxes)
  // dQ  : fix0 = Q, fix1 = dO,                 str0 = K, str1 = V
  using L = Bwd2Smem<D>;
  constexpr int DC = L::DC, ST = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* fix_full = bars;           // 1
  uint64_t* str_full = bars + 1;       // ST
  uint64_t* str_empty = bars + 1 + ST; // ST
  uint64_t* s_full = bars + 1 + 2 * ST;    // S and dP of a step are in TMEM
  uint64_t* pds_full = bars + 2 + 2 * ST;  // P / dS of a step are back in TMEM
  uint64_t* acc_full = bars + 3 + 2 * ST;  // final accumulators
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 4 + 2 * ST);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp_idx = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int n_sub = p.S / SUB;
  const int own = DKDV ? (int)blockIdx.z : (int)gridDim.z - 1 - (int)blockIdx.z;  // longest first
  const int it_begin = DKDV ? (p.causal ? 2 * own : 0) : 0;
  const int it_end = DKDV ? n_sub : (p.causal ? 2 * own + 2 : n_sub);
  const int n_it = it_end - it_begin;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(fix_full), 1);
    for (int i = 0; i < ST; ++i) {
      mbar_init(smem_u32(&str_full[i]), 1);
      mbar_init(smem_u32(&str_empty[i]), 1);
    }
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(pds_full), 32 * COMPUTE_WARPS);
    mbar_init(smem_u32(acc_full), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tm_fix0);
    tma_prefetch_desc(&tm_fix1);
    tma_prefetch_desc(&tm_str0);
    tma_prefetch_desc(&tm_str1);
  }
  if (warp_idx == 1) {
    tmem_alloc(smem_u32(tmem_holder), L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  // operands come from kernels before the previous one when `late_wait` is set (the dQ kernel
  // after the dK / dV kernel: both read q, k, v, dO, lse, delta and write disjoint outputs)
  pdl_enter(p.late_wait != 0);
  const uint32_t tmem_s = tmem_base;             // 64 fp32 score columns; packed P lands in them
  const uint32_t tmem_dp = tmem_base + 64;       // 64 fp32 dP columns; packed dS lands in them
  const uint32_t tmem_acc0 = tmem_base + 128;    // dK (DKDV) or dQ: from dS
  const uint32_t tmem_acc1 = tmem_base + 128 + D;  // dV (DKDV only): from P
  // packed bf16 operand columns: the 32 columns owned by compute half hh keep 16 packed
  // columns at the start of their own fp32 range (so the two halves never touch each other's)
  auto packed_col = [](int ks) { return (ks >> 1) * 32 + (ks & 1) * 8; };  // 16 rows of K per step

  auto str0 = [&](int st) { return smem + L::OFF_STR + st * 2 * L::STR; };
  auto str1 = [&](int st) { return smem + L::OFF_STR + st * 2 * L::STR + L::STR; };

  if (warp_idx == 0) {
    if (lane == 0) {
      const uint32_t fb = smem_u32(fix_full);
      mbar_arrive_expect_tx(fb, 2 * L::FIX);
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        tma_load_4d(smem_u32(smem + L::OFF_FIX0 + c * CHUNK_BYTES), &tm_fix0, fb, 64 * c, own * BT, h, b);
        tma_load_4d(smem_u32(smem + L::OFF_FIX1 + c * CHUNK_BYTES), &tm_fix1, fb, 64 * c, own * BT, h, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % ST, use = it / ST, t = it_begin + it;
        if (!mbar_wait_bounded(smem_u32(&str_empty[st]), (use & 1) ^ 1, abort_flag, &g_attn_error, 71))
          break;
        const uint32_t sb = smem_u32(&str_full[st]);
        mbar_arrive_expect_tx(sb, 2 * L::STR + (DKDV ? 2 * SUB * 4 : 0));
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          tma_load_4d(smem_u32(str0(st) + c * SUB_CHUNK), &tm_str0, sb, 64 * c, t * SUB, h, b);
          tma_load_4d(smem_u32(str1(st) + c * SUB_CHUNK), &tm_str1, sb, 64 * c, t * SUB, h, b);
        }
        if (DKDV) {
          // the 64 streamed queries' log-sum-exp and delta ride on the same barrier: every
          // compute thread needs all of them, and reads them as shared-memory broadcasts
          const long long row0 = ((long long)b * p.H + h) * p.S + (long long)t * SUB;
          float* sc = reinterpret_cast<float*>(smem + L::OFF_SCAL) + st * 2 * SUB;
          bulk_load(smem_u32(sc), p.lse + row0, SUB * 4, sb);
          bulk_load(smem_u32(sc + SUB), p.delta + row0, SUB * 4, sb);
        }
      }
    }
  } else if (warp_idx == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(BT, SUB, 0, 0);   // [128 lanes] x [64 streamed rows]
      const uint32_t idesc_acc = make_idesc_bf16(BT, D, 0, 1);   // A from TMEM, B = streamed tile, rows as K
      bool ok = mbar_wait_bounded(smem_u32(fix_full), 0, abort_flag, &g_attn_error, 72);
      for (int it = 0; ok && it < n_it; ++it) {
        const int st = it % ST, use = it / ST;
        if (!mbar_wait_bounded(smem_u32(&str_full[st]), use & 1, abort_flag, &g_attn_error, 73)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // scores: lanes x streamed rows, contraction over the head dim.  They overwrite the
        // packed operands of the previous step, which the in-order tensor pipe has consumed
        // by then (the accumulating MMAs below were issued before these).
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          const uint64_t f0 = make_smem_desc_sw128(smem_u32(smem + L::OFF_FIX0 + c * CHUNK_BYTES), 16, 1024);
          const uint64_t s0 = make_smem_desc_sw128(smem_u32(str0(st) + c * SUB_CHUNK), 16, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16(tmem_s, f0 + (uint64_t)(ks * 2), s0 + (uint64_t)(ks * 2), idesc_s,
                      (c > 0 || ks > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          const uint64_t f1 = make_smem_desc_sw128(smem_u32(smem + L::OFF_FIX1 + c * CHUNK_BYTES), 16, 1024);
          const uint64_t s1 = make_smem_desc_sw128(smem_u32(str1(st) + c * SUB_CHUNK), 16, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16(tmem_dp, f1 + (uint64_t)(ks * 2), s1 + (uint64_t)(ks * 2), idesc_s,
                      (c > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(s_full));
        if (!mbar_wait_bounded(smem_u32(pds_full), it & 1, abort_flag, &g_attn_error, 74)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // accumulate over the 64 streamed rows (K), 16 rows = 2048 bytes of the tile per step
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // dS-based product: B = streamed operand 0 (Q for dK, K for dQ), its rows as K
          const uint64_t bd = make_smem_desc_sw128(smem_u32(str0(st)) + ks * 2048, SUB_CHUNK, 1024);
          umma_bf16_ts(tmem_acc0, tmem_dp + packed_col(ks), bd, idesc_acc, (it > 0 || ks > 0) ? 1u : 0u);
        }
        if (DKDV) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t bd = make_smem_desc_sw128(smem_u32(str1(st)) + ks * 2048, SUB_CHUNK, 1024);
            umma_bf16_ts(tmem_acc1, tmem_s + packed_col(ks), bd, idesc_acc, (it > 0 || ks > 0) ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(&str_empty[st]));
      }
      if (ok) umma_commit(smem_u32(acc_full));
    }
  } else {
    const int quad = warp_idx & 3;
    const int hh = (warp_idx - 2) >> 2;          // which 32 of the 64 columns
    const int row = quad * 32 + lane;
    const uint32_t lane_base = ((uint32_t)(quad * 32)) << 16;
    const int row_g = own * BT + row;            // key index (DKDV) or query index
    const long long bh = ((long long)b * p.H + h) * p.S;
    float lse2_l = 0.0f, dsc_l = 0.0f;
    if (!DKDV) {
      lse2_l = p.lse[bh + row_g] * LOG2E;
      dsc_l = p.delta[bh + row_g] * p.scale;
    }
    bool ok = true;
    for (int it = 0; ok && it < n_it; ++it) {
      const int t = it_begin + it;
      const int c0 = t * SUB + hh * 32;          // global index of this thread's first column
      // causal bounds in units of this thread's 32 columns
      int lo = 0, hi = 32;
      bool masked = false;
      if (p.causal && (t >> 1) == own) {
        masked = true;
        if (DKDV) lo = row_g - c0;               // query >= key
        else hi = row_g - c0 + 1;                // key <= query
      }
      float lse2_c[16], dsc_c[16];
      const float* sc = reinterpret_cast<const float*>(smem + L::OFF_SCAL) + (it % ST) * 2 * SUB + hh * 32;
      auto load_cols = [&](int off) {   // broadcast reads: every lane takes the same 16 columns
        const float4* l4 = reinterpret_cast<const float4*>(sc + off);
        const float4* d4 = reinterpret_cast<const float4*>(sc + SUB + off);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 a = l4[q], d = d4[q];
          lse2_c[4 * q] = a.x * LOG2E; lse2_c[4 * q + 1] = a.y * LOG2E;
          lse2_c[4 * q + 2] = a.z * LOG2E; lse2_c[4 * q + 3] = a.w * LOG2E;
          dsc_c[4 * q] = d.x * p.scale; dsc_c[4 * q + 1] = d.y * p.scale;
          dsc_c[4 * q + 2] = d.z * p.scale; dsc_c[4 * q + 3] = d.w * p.scale;
        }
      };
      if (!mbar_wait_bounded_warp(smem_u32(s_full), it & 1, abort_flag, &g_attn_error, 75)) {
        ok = false;
        break;
      }
      // the stage's barrier completed long ago (the MMAs waited for it); observing it here
      // makes the bulk-copied scalars visible to this thread
      if (DKDV && !mbar_wait_bounded_warp(smem_u32(&str_full[it % ST]), (it / ST) & 1, abort_flag,
                                          &g_attn_error, 77)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t s_addr = tmem_s + lane_base + hh * 32;
      const uint32_t d_addr = tmem_dp + lane_base + hh * 32;
      // two chunks of 16 columns; the packed bf16 results of chunk k go to columns [8 k, 8 k + 8)
      // of this thread's own 32-column range, which holds fp32 values it has already read
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        uint32_t sv[16], dv[16], pp[8], dd[8];
        tmem_ld_32x16(s_addr + 16 * k, sv);
        tmem_ld_32x16(d_addr + 16 * k, dv);
        if (DKDV) load_cols(16 * k);      // the stage (s_full follows str_full) is complete
        tmem_ld_wait();
        if (masked)
          rebuild16<DKDV, true>(sv, dv, lse2_c, dsc_c, lse2_l, dsc_l, p.scale_log2, p.scale,
                                lo - 16 * k, hi - 16 * k, pp, dd);
        else
          rebuild16<DKDV, false>(sv, dv, lse2_c, dsc_c, lse2_l, dsc_l, p.scale_log2, p.scale, 0, 16, pp, dd);
        if (DKDV) tmem_st_32x8(s_addr + 8 * k, pp);
        tmem_st_32x8(d_addr + 8 * k, dd);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(pds_full));
    }
    if (ok && n_it > 0 &&
        mbar_wait_bounded_warp(smem_u32(acc_full), 0, abort_flag, &g_attn_error, 76)) {
      tc_fence_after_sync();
      const bool in_range = row_g < p.S;
      __nv_bfloat16* d0p = in_range ? p.out0 + (long long)b * p.o0_sb + (long long)row_g * p.o0_ss +
                                          (long long)h * p.o0_sh
                                    : nullptr;
      store_acc_row<D>(tmem_acc0 + lane_base, d0p, hh);
      if (DKDV) {
        __nv_bfloat16* d1p = in_range ? p.out1 + (long long)b * p.o1_sb + (long long)row_g * p.o1_ss +
                                            (long long)h * p.o1_sh
                                      : nullptr;
        store_acc_row<D>(tmem_acc1 + lane_base, d1p, hh);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp_idx == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
  pdl_leave(p.late_wait != 0);
}

template <int D, bool DKDV>
cudaError_t launch_bwd2(const CUtensorMap& f0, const CUtensorMap& f1, const CUtensorMap& s0,
                        const CUtensorMap& s1, const BwdParams& p, dim3 grid, cudaStream_t s) {
  using L = Bwd2Smem<D>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd2_kernel<D, DKDV>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaError_t le = launch_pdl(flash_bwd2_kernel<D, DKDV>, grid, dim3(B2_THREADS), L::TOTAL, s, f0, f1, s0, s1, p);
  if (le != cudaSuccess) return le;
  g_attn_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

// LT_FLASH_BWD2_D128=1: the second-generation kernels at head dim 128 as well (one CTA per SM)
bool use_bwd2_d128() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LT_FLASH_BWD2_D128");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v != 0;
}
// LT_FLASH_BWD_V1=1 keeps the first-generation kernels (comparison runs)
bool use_bwd_v1() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LT_FLASH_BWD_V1");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v != 0;
}

template <int D, bool DKDV>
cudaError_t launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                       const CUtensorMap& tdo, const BwdParams& p, dim3 grid, cudaStream_t s) {
  using L = BwdSmem<D, DKDV>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd_kernel<D, DKDV>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaError_t le = launch_pdl(flash_bwd_kernel<D, DKDV>, grid, dim3(NUM_THREADS), L::TOTAL, s, tq, tk, tv, tdo, p);
  if (le != cudaSuccess) return le;
  g_attn_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

bool ok8(int64_t a, int64_t b, int64_t c) { return a % 8 == 0 && b % 8 == 0 && c % 8 == 0; }

}  // namespace

cudaError_t flash_attention_backward(const AttnArgs& a, const AttnBwdArgs& g, cudaStream_t stream) {
  if (a.B <= 0 || a.H <= 0 || a.S <= 0) return cudaSuccess;
  if (a.D != 64 && a.D != 128) return cudaErrorInvalidValue;
  if (!ok8(a.q_ss, a.q_sh, a.q_sb) || !ok8(a.k_ss, a.k_sh, a.k_sb) || !ok8(a.v_ss, a.v_sh, a.v_sb) ||
      !ok8(g.do_ss, g.do_sh, g.do_sb) || !ok8(g.dq_ss, g.dq_sh, g.dq_sb) ||
      !ok8(g.dk_ss, g.dk_sh, g.dk_sb) || !ok8(g.dv_ss, g.dv_sh, g.dv_sb))
    return cudaErrorInvalidValue;

  const long long rows = (long long)a.B * a.H * a.S;
  cudaError_t de = launch_pdl(attn_delta_kernel, dim3((unsigned)((rows + 255) / 256)), dim3(256), 0, stream,
                              (const __nv_bfloat16*)a.o, (const __nv_bfloat16*)g.d_o, g.delta, a.B, a.H,
                              a.S, a.D, (long long)a.o_sb, (long long)a.o_ss, (long long)a.o_sh,
                              (long long)g.do_sb, (long long)g.do_ss, (long long)g.do_sh);
  if (de != cudaSuccess) return de;
  g_attn_launches.fetch_add(1, std::memory_order_relaxed);

  if ((a.D == 64 || (a.D == 128 && use_bwd2_d128())) && a.S % BT == 0 && !use_bwd_v1() &&
      ((reinterpret_cast<uintptr_t>(a.lse) | reinterpret_cast<uintptr_t>(g.delta)) & 15) == 0) {
    // second-generation kernels: P / dS stay in tensor memory, two CTAs per SM
    CUtensorMap q128, k128, v128, do128, q64, k64, v64, do64;
    if (!attn_detail::make_qkv_map(&q128, a.q, a.D, a.S, a.H, a.B, a.q_ss, a.q_sh, a.q_sb, BT) ||
        !attn_detail::make_qkv_map(&k128, a.k, a.D, a.S, a.H, a.B, a.k_ss, a.k_sh, a.k_sb, BT) ||
        !attn_detail::make_qkv_map(&v128, a.v, a.D, a.S, a.H, a.B, a.v_ss, a.v_sh, a.v_sb, BT) ||
        !attn_detail::make_qkv_map(&do128, g.d_o, a.D, a.S, a.H, a.B, g.do_ss, g.do_sh, g.do_sb, BT) ||
        !attn_detail::make_qkv_map(&q64, a.q, a.D, a.S, a.H, a.B, a.q_ss, a.q_sh, a.q_sb, SUB) ||
        !attn_detail::make_qkv_map(&k64, a.k, a.D, a.S, a.H, a.B, a.k_ss, a.k_sh, a.k_sb, SUB) ||
        !attn_detail::make_qkv_map(&v64, a.v, a.D, a.S, a.H, a.B, a.v_ss, a.v_sh, a.v_sb, SUB) ||
        !attn_detail::make_qkv_map(&do64, g.d_o, a.D, a.S, a.H, a.B, g.do_ss, g.do_sh, g.do_sb, SUB))
      return cudaErrorInvalidValue;
    BwdParams p2;
    p2.S = a.S; p2.H = a.H; p2.causal = a.causal;
    p2.scale = a.scale; p2.scale_log2 = a.scale * LOG2E;
    p2.lse = a.lse; p2.delta = g.delta; p2.ds_out = nullptr;
    dim3 grid2(a.H, a.B, a.S / BT);   // tile index slowest: longest CTAs of every head go first
    p2.out0 = (__nv_bfloat16*)g.dk; p2.o0_sb = g.dk_sb; p2.o0_ss = g.dk_ss; p2.o0_sh = g.dk_sh;
    p2.out1 = (__nv_bfloat16*)g.dv; p2.o1_sb = g.dv_sb; p2.o1_ss = g.dv_ss; p2.o1_sh = g.dv_sh;
    cudaError_t e2 = a.D == 64 ? launch_bwd2<64, true>(k128, v128, q64, do64, p2, grid2, stream)
                               : launch_bwd2<128, true>(k128, v128, q64, do64, p2, grid2, stream);
    if (e2 != cudaSuccess) return e2;
    p2.out0 = (__nv_bfloat16*)g.dq; p2.o0_sb = g.dq_sb; p2.o0_ss = g.dq_ss; p2.o0_sh = g.dq_sh;
    p2.out1 = nullptr; p2.o1_sb = p2.o1_ss = p2.o1_sh = 0;
    const LateWait lw = late_wait_begin(1);   // independent of the dK / dV kernel: runs in its tail
    p2.late_wait = lw.on;
    e2 = a.D == 64 ? launch_bwd2<64, false>(q128, do128, k64, v64, p2, grid2, stream)
                   : launch_bwd2<128, false>(q128, do128, k64, v64, p2, grid2, stream);
    late_wait_commit(lw);
    return e2;
  }

  CUtensorMap tq, tk, tv, tdo;
  if (!attn_detail::make_qkv_map(&tq, a.q, a.D, a.S, a.H, a.B, a.q_ss, a.q_sh, a.q_sb, BT) ||
      !attn_detail::make_qkv_map(&tk, a.k, a.D, a.S, a.H, a.B, a.k_ss, a.k_sh, a.k_sb, BT) ||
      !attn_detail::make_qkv_map(&tv, a.v, a.D, a.S, a.H, a.B, a.v_ss, a.v_sh, a.v_sb, BT) ||
      !attn_detail::make_qkv_map(&tdo, g.d_o, a.D, a.S, a.H, a.B, g.do_ss, g.do_sh, g.do_sb, BT))
    return cudaErrorInvalidValue;

  BwdParams p;
  p.S = a.S; p.H = a.H; p.causal = a.causal;
  p.scale = a.scale; p.scale_log2 = a.scale * LOG2E;
  p.lse = a.lse; p.delta = g.delta;
  dim3 grid(a.H, a.B, (a.S + BT - 1) / BT);

  p.out0 = (__nv_bfloat16*)g.dk; p.o0_sb = g.dk_sb; p.o0_ss = g.dk_ss; p.o0_sh = g.dk_sh;
  p.out1 = (__nv_bfloat16*)g.dv; p.o1_sb = g.dv_sb; p.o1_ss = g.dv_ss; p.o1_sh = g.dv_sh;
  const bool dq_by_gemm = g.ds_scratch != nullptr && a.S % BT == 0;
  p.ds_out = dq_by_gemm ? (__nv_bfloat16*)g.ds_scratch : nullptr;
  cudaError_t e = a.D == 64 ? launch_bwd<64, true>(tq, tk, tv, tdo, p, grid, stream)
                            : launch_bwd<128, true>(tq, tk, tv, tdo, p, grid, stream);
  if (e != cudaSuccess) return e;
  p.ds_out = nullptr;
  if (dq_by_gemm) {
    // dQ[b, h] = dS[b, h] (S x S, the scale already folded in) @ K[b, h] (S x D); with a causal
    // mask the k loop of a query tile stops at its own diagonal (nothing was written beyond it)
    GemmArgs m;
    m.M = a.S; m.N = a.D; m.K = a.S;
    m.A = g.ds_scratch; m.lda = a.S; m.a_mn_major = 0;
    m.a_stride_inner = (int64_t)a.S * a.S; m.a_stride_outer = (int64_t)a.H * a.S * a.S;
    m.B = a.k; m.ldb = a.k_ss; m.b_mn_major = 1;
    m.b_stride_inner = a.k_sh; m.b_stride_outer = a.k_sb;
    m.C = g.dq; m.ldc = g.dq_ss; m.c_stride_inner = g.dq_sh; m.c_stride_outer = g.dq_sb;
    m.batch_inner = a.H; m.batch_outer = a.B;
    m.causal_k = a.causal ? 1 : 0;
    return gemm_bf16(m, stream);
  }

  p.out0 = (__nv_bfloat16*)g.dq; p.o0_sb = g.dq_sb; p.o0_ss = g.dq_ss; p.o0_sh = g.dq_sh;
  p.out1 = nullptr; p.o1_sb = p.o1_ss = p.o1_sh = 0;
  return a.D == 64 ? launch_bwd<64, false>(tq, tk, tv, tdo, p, grid, stream)
                   : launch_bwd<128, false>(tq, tk, tv, tdo, p, grid, stream);
}

}  // namespace lt
