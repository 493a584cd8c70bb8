// Causal / non-causal flash attention forward on tcgen05.  Two kernels: the first generation
// described here (kept for comparison runs) and the second generation further down, which is
// the default for head dims 64 and 128.
//
// First generation: one CTA per (128-query tile, head, batch); 192 threads:
//   warp 0      TMA producer: Q once, then K/V tiles through a 2-stage ring
//   warp 1      MMA issuer: S = Q K^T into one of two TMEM score buffers, O_tile = P V
//   warps 2..5  softmax: thread r owns query row r; reads S from TMEM, keeps the running
//               max / sum and the output row in registers, writes P (bf16) into shared
//               memory in the 128-byte-swizzled layout the tensor core expects as operand A
// S for tile j+1 is issued before P V of tile j, so the tensor core works while the softmax
// warps are busy with exponentials.  Tiles above the causal diagonal are never loaded.
#include "attention.h"
#include "sm100_ptx.cuh"
#include "common.cuh"

#include <cuda.h>
#include <atomic>
#include <mutex>

namespace lt {

using namespace ptx;

std::atomic<uint64_t> g_attn_launches{0};
__device__ int g_attn_error = 0;

int attention_bwd_device_error();  // attention_bwd.cu
int attention_last_device_error() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int));
  return v != 0 ? v : attention_bwd_device_error();
}
uint64_t attention_launch_count() { return g_attn_launches.load(); }

namespace attn_detail {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
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

// (head_dim, seq, head, batch) bf16 map with a (64, rows, 1, 1) box and 128-byte swizzle.
bool make_qkv_map(CUtensorMap* map, const void* base, int D, int S, int H, int B, int64_t ss,
                  int64_t sh, int64_t sb, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace attn_detail

namespace {

constexpr int BM = 128;       // queries per CTA
constexpr int BN = 128;       // keys per tile
constexpr int CHUNK_BYTES = 128 * 128;  // 128 rows x 64 bf16, one swizzled operand chunk
constexpr int NUM_THREADS = 192;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// Row maximum over one 32-column chunk; `valid` = number of leading columns of this chunk
// that are inside the causal / sequence bounds (only consulted when `masked`).
__device__ __forceinline__ float chunk_max(const uint32_t (&r)[32], float mx, bool masked,
                                           int valid) {
  if (!masked) {
#pragma unroll
    for (int i = 0; i < 32; i += 2)
      mx = fmaxf(mx, fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) mx = fmaxf(mx, __uint_as_float(r[i]));
  }
  return mx;
}

// p = 2^(s*c - mc) for one chunk, written as bf16 into the swizzled operand-A tile; returns
// the chunk's row sum.
__device__ __forceinline__ float chunk_exp_store(const uint32_t (&r)[32], float c, float mc,
                                                 bool masked, int valid, uint8_t* p_row, int c32,
                                                 int row) {
  uint32_t packed[16];
  float sum0 = 0.0f, sum1 = 0.0f;
  if (!masked) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const float p0 = ex2(fmaf(__uint_as_float(r[i]), c, -mc));
      const float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), c, -mc));
      sum0 += p0;
      sum1 += p1;
      __nv_bfloat162 hb = __floats2bfloat162_rn(p0, p1);
      packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hb);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const float p0 = (i < valid) ? ex2(fmaf(__uint_as_float(r[i]), c, -mc)) : 0.0f;
      const float p1 = (i + 1 < valid) ? ex2(fmaf(__uint_as_float(r[i + 1]), c, -mc)) : 0.0f;
      sum0 += p0;
      sum1 += p1;
      __nv_bfloat162 hb = __floats2bfloat162_rn(p0, p1);
      packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hb);
    }
  }
  uint8_t* dst = p_row + (c32 >> 1) * CHUNK_BYTES;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int chunk16 = ((c32 & 1) * 4 + t) ^ (row & 7);
    *reinterpret_cast<uint4*>(dst + chunk16 * 16) =
        make_uint4(packed[4 * t], packed[4 * t + 1], packed[4 * t + 2], packed[4 * t + 3]);
  }
  return sum0 + sum1;
}

struct FwdParams {
  int S, H;
  int causal;
  float scale_log2;  // scale * log2(e)
  float scale;
  __nv_bfloat16* o;
  long long o_sb, o_ss, o_sh;
  float* lse;
  int tmem_p;        // keep P in tensor memory (A operand of P V read from TMEM)
};

template <int D>
struct FwdSmem {
  static constexpr int DC = D / 64;                 // 64-wide head_dim chunks
  static constexpr int Q_BYTES = DC * CHUNK_BYTES;
  static constexpr int KV_BYTES = DC * CHUNK_BYTES;
  static constexpr int P_BYTES = 2 * CHUNK_BYTES;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;          // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;     // 2 stages
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  // head_dim 64: one score buffer and 256 TMEM columns so that TWO CTAs share an SM (their
  // softmax and MMA phases interleave); head_dim 128 fills the SM with one CTA and double
  // buffers the scores instead.
  static constexpr int NSB = D == 64 ? 1 : 2;
  static constexpr int TMEM_COLS = D == 64 ? 256 : 512;
  static constexpr int TOTAL = OFF_BAR + 256;   // base must be 1024-byte aligned (checked)
};

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, (D == 64 ? 2 : 1))
flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using L = FwdSmem<D>;
  constexpr int DC = L::DC;
  constexpr int NSB = L::NSB;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023) {  // swizzled operand tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(&g_attn_error, 0, 40);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* v_full = bars + 3;        // 2
  uint64_t* kv_empty = bars + 5;      // 2
  uint64_t* s_full = bars + 7;        // 2
  uint64_t* s_empty = bars + 9;       // 2
  uint64_t* p_full = bars + 11;       // 1
  uint64_t* o_full = bars + 12;       // 1
  uint64_t* o_empty = bars + 13;      // 1
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp_idx = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // longest (most key tiles) query tiles first
  const int q_tile = (int)gridDim.z - 1 - (int)blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int q0 = q_tile * BM;
  const int n_kv_all = (p.S + BN - 1) / BN;
  const int n_kv = p.causal ? (q_tile + 1 < n_kv_all ? q_tile + 1 : n_kv_all) : n_kv_all;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&k_full[i]), 1);
      mbar_init(smem_u32(&v_full[i]), 1);
      mbar_init(smem_u32(&kv_empty[i]), 1);
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 128);
    }
    mbar_init(smem_u32(p_full), 128);
    mbar_init(smem_u32(o_full), 1);
    mbar_init(smem_u32(o_empty), 128);
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp_idx == 1) {
    tmem_alloc(smem_u32(tmem_holder), L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  pdl_enter();   // q, k, v come from the previous kernel
  const uint32_t tmem_s = tmem_base;                // NSB score buffers of 128 columns
  const uint32_t tmem_o = tmem_base + NSB * 128;    // D columns

  if (warp_idx == 0) {
    if (lane == 0) {
      const uint32_t qb = smem_u32(q_full);
      mbar_arrive_expect_tx(qb, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DC; ++c)
        tma_load_4d(smem_u32(smem + L::OFF_Q + c * CHUNK_BYTES), &tm_q, qb, 64 * c, q0, h, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait_bounded(smem_u32(&kv_empty[st]), ((j >> 1) & 1) ^ 1, abort_flag,
                               &g_attn_error, 11))
          break;
        const uint32_t kb = smem_u32(&k_full[st]), vb = smem_u32(&v_full[st]);
        mbar_arrive_expect_tx(kb, L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; ++c)
          tma_load_4d(smem_u32(smem + L::OFF_K + st * L::KV_BYTES + c * CHUNK_BYTES), &tm_k, kb,
                      64 * c, j * BN, h, b);
        mbar_arrive_expect_tx(vb, L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; ++c)
          tma_load_4d(smem_u32(smem + L::OFF_V + st * L::KV_BYTES + c * CHUNK_BYTES), &tm_v, vb,
                      64 * c, j * BN, h, b);
      }
    }
  } else if (warp_idx == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(BM, D, 0, 1);
      bool ok = mbar_wait_bounded(smem_u32(q_full), 0, abort_flag, &g_attn_error, 12);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const int sb = NSB == 2 ? st : 0;                 // score buffer
        const int su = NSB == 2 ? (j >> 1) : j;           // how often it has been used
        if (!mbar_wait_bounded(smem_u32(&k_full[st]), (j >> 1) & 1, abort_flag, &g_attn_error, 13))
          return false;
        if (!mbar_wait_bounded(smem_u32(&s_empty[sb]), (su & 1) ^ 1, abort_flag, &g_attn_error,
                               14))
          return false;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          const uint64_t qd =
              make_smem_desc_sw128(smem_u32(smem + L::OFF_Q + c * CHUNK_BYTES), 16, 1024);
          const uint64_t kd = make_smem_desc_sw128(
              smem_u32(smem + L::OFF_K + st * L::KV_BYTES + c * CHUNK_BYTES), 16, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16(tmem_s + sb * BN, qd + (uint64_t)(ks * 2), kd + (uint64_t)(ks * 2), idesc_s,
                      (c > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&s_full[sb]));
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j & 1;
        if (NSB == 2 && j + 1 < n_kv) {
          if (!issue_s(j + 1)) { ok = false; break; }
        }
        if (!mbar_wait_bounded(smem_u32(&v_full[st]), (j >> 1) & 1, abort_flag, &g_attn_error, 15) ||
            !mbar_wait_bounded(smem_u32(p_full), j & 1, abort_flag, &g_attn_error, 16) ||
            !mbar_wait_bounded(smem_u32(o_empty), (j & 1) ^ 1, abort_flag, &g_attn_error, 17)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // O_tile[128 x D] = P[128 x 128 keys] * V[128 keys x D]; keys are the K dimension:
        // two 64-key chunks of P, V rows 8-key groups 1024 B apart, 16 keys = 2048 B per step.
#pragma unroll
        for (int kc = 0; kc < 2; ++kc) {
          const uint64_t pd =
              make_smem_desc_sw128(smem_u32(smem + L::OFF_P + kc * CHUNK_BYTES), 16, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t v_addr = smem_u32(smem + L::OFF_V + st * L::KV_BYTES) +
                                    (kc * 64 + ks * 16) * 128;
            const uint64_t vd = make_smem_desc_sw128(v_addr, CHUNK_BYTES, 1024);
            umma_bf16(tmem_o, pd + (uint64_t)(ks * 2), vd, idesc_o, (kc > 0 || ks > 0) ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(o_full));
        umma_commit(smem_u32(&kv_empty[st]));
        if (NSB == 1 && j + 1 < n_kv) {
          // single score buffer: the softmax warps released it just before p_full
          if (!issue_s(j + 1)) { ok = false; break; }
        }
      }
    }
  } else {
    // ------------------------------ softmax / output ------------------------------
    const int quad = warp_idx & 3;
    const int row = quad * 32 + lane;      // query row inside the tile
    const int qi = q0 + row;               // global query index
    const uint32_t lane_base = ((uint32_t)(quad * 32)) << 16;
    float m = -INFINITY, l = 0.0f;
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.0f;
    const float c = p.scale_log2;
    bool ok = true;
    uint8_t* p_row = smem + L::OFF_P + (row >> 3) * 1024 + (row & 7) * 128;

    for (int j = 0; ok && j < n_kv; ++j) {
      const int st = NSB == 2 ? (j & 1) : 0;
      const int su = NSB == 2 ? (j >> 1) : j;
      if (!mbar_wait_bounded_warp(smem_u32(&s_full[st]), su & 1, abort_flag, &g_attn_error, 18)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int k0 = j * BN;
      const bool need_mask = (p.causal && k0 + BN - 1 > q0) || (k0 + BN > p.S);
      // number of valid key columns for this row inside the tile
      int valid = BN;
      if (need_mask) {
        int lim = p.S - k0;
        if (p.causal) { int cl = qi - k0 + 1; lim = cl < lim ? cl : lim; }
        valid = lim < 0 ? 0 : (lim > BN ? BN : lim);
      }
      // pass 1: row maximum.  TMEM reads are double buffered: the next 32-column chunk is in
      // flight while the current one is reduced.
      float mx = m;
      uint32_t ra[32], rb[32];
      const uint32_t s_addr = tmem_s + lane_base + st * BN;
      tmem_ld_32x32(s_addr, ra);
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 32, rb);
      mx = chunk_max(ra, mx, need_mask, valid);
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 64, ra);
      mx = chunk_max(rb, mx, need_mask, valid - 32);
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 96, rb);
      mx = chunk_max(ra, mx, need_mask, valid - 64);
      tmem_ld_wait();
      tmem_ld_32x32(s_addr, ra);            // first chunk of pass 2, lands during the O fold
      mx = chunk_max(rb, mx, need_mask, valid - 96);
      const float m_new = mx;
      const float alpha = (m == -INFINITY) ? 0.0f : ex2((m - m_new) * c);
      // fold in the previous tile's P V product, then rescale to the new maximum
      if (j > 0) {
        if (!mbar_wait_bounded_warp(smem_u32(o_full), (j - 1) & 1, abort_flag, &g_attn_error, 19)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int c32 = 0; c32 < D / 32; ++c32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_o + lane_base + c32 * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c32 * 32 + i] += __uint_as_float(r[i]);
        }
        tc_fence_before_sync();
        mbar_arrive(smem_u32(o_empty));
      }
#pragma unroll
      for (int i = 0; i < D; ++i) o_acc[i] *= alpha;
      l *= alpha;
      // pass 2: exponentials -> P (bf16, swizzled operand-A layout) + row sum
      const float mc = (m_new == -INFINITY) ? 0.0f : m_new * c;
      float rsum = 0.0f;
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 32, rb);
      rsum += chunk_exp_store(ra, c, mc, need_mask, valid, p_row, 0, row);
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 64, ra);
      rsum += chunk_exp_store(rb, c, mc, need_mask, valid - 32, p_row, 1, row);
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 96, rb);
      rsum += chunk_exp_store(ra, c, mc, need_mask, valid - 64, p_row, 2, row);
      tmem_ld_wait();
      rsum += chunk_exp_store(rb, c, mc, need_mask, valid - 96, p_row, 3, row);
      l += rsum;
      m = m_new;
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&s_empty[st]));
      fence_proxy_async();
      mbar_arrive(smem_u32(p_full));
    }
    if (ok && n_kv > 0) {
      if (mbar_wait_bounded_warp(smem_u32(o_full), (n_kv - 1) & 1, abort_flag, &g_attn_error, 20)) {
        tc_fence_after_sync();
#pragma unroll
        for (int c32 = 0; c32 < D / 32; ++c32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_o + lane_base + c32 * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c32 * 32 + i] += __uint_as_float(r[i]);
        }
        if (qi < p.S) {
          const float inv = l > 0.0f ? 1.0f / l : 0.0f;
          __nv_bfloat16* orow = p.o + (long long)b * p.o_sb + (long long)qi * p.o_ss +
                                (long long)h * p.o_sh;
#pragma unroll
          for (int i = 0; i < D; i += 8) {
            uint4 u;
            __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
            for (int t = 0; t < 4; ++t)
              hb[t] = __floats2bfloat162_rn(o_acc[i + 2 * t] * inv, o_acc[i + 2 * t + 1] * inv);
            *reinterpret_cast<uint4*>(orow + i) = u;
          }
          if (p.lse)
            p.lse[((long long)b * p.H + h) * p.S + qi] =
                (l > 0.0f) ? m * p.scale + __logf(l) : -INFINITY;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp_idx == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------
// Second generation (the default; 64.4 vs 77.0 us at B 8, S 1024, H 12, D 64 and 162 vs 181 us at
// B 4, S 2048, H 16, D 128).  Same data flow as above, rebuilt around what the first
// kernel's profile showed: it was bound by the instruction stream of its four softmax warps
// (about 7 instructions per score at two warps per scheduler), not by the tensor cores.
//   * eight softmax warps: warps w and w+4 share the TMEM lanes (query rows) of quadrant w&3
//     and split the 128 keys of a tile in halves; both take the row maximum over all 128
//     scores (so they agree without exchanging anything) and exponentiate their own 64;
//   * those 64 scores are copied to registers and the TMEM buffer is released BEFORE the
//     exponentials, so Q K^T of the next tile runs under them;
//   * O stays in TMEM and is accumulated by the tensor core across tiles; it is rescaled only
//     when a row's maximum grows by more than 2^8 (exponentials stay far inside fp32 / bf16
//     range), which after the first tiles is rare;
//   * packed fp32 math (fma / add on register pairs) and three-input max halve the FMA-pipe
//     instruction count.
// ------------------------------------------------------------------------------
constexpr int V2_SOFTMAX_WARPS = 8;
constexpr int V2_THREADS = 64 + 32 * V2_SOFTMAX_WARPS;
constexpr float V2_RESCALE_LOG2 = 8.0f;

// max over one 32-column chunk; `valid` = leading columns of the chunk inside the bounds
__device__ __forceinline__ float v2_chunk_max(const uint32_t (&r)[32], float mx, bool masked,
                                              int valid) {
  if (!masked) {
    float a = mx, b = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      a = max3f(a, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
      b = max3f(b, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
    }
    return fmaxf(a, b);
  }
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (i < valid) mx = fmaxf(mx, __uint_as_float(r[i]));
  return mx;
}

// p = 2^(s c - mc) for 32 scores -> bf16 into the swizzled P tile; adds the row sum to `sum2`
__device__ __forceinline__ void v2_chunk_exp_store(const uint32_t (&r)[32], float c, float mc,
                                                   bool masked, int valid, uint8_t* p_row,
                                                   int c32, int row, float2& sum2) {
  uint32_t packed[16];
  const float2 cc = make_float2(c, c), mm = make_float2(-mc, -mc);
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const float2 x = ffma2(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), cc, mm);
    float p0 = ex2(x.x), p1 = ex2(x.y);
    if (masked) {
      p0 = (i < valid) ? p0 : 0.0f;
      p1 = (i + 1 < valid) ? p1 : 0.0f;
    }
    sum2 = fadd2(sum2, make_float2(p0, p1));
    __nv_bfloat162 hb = __floats2bfloat162_rn(p0, p1);
    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hb);
  }
  uint8_t* dst = p_row + (c32 >> 1) * CHUNK_BYTES;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int chunk16 = ((c32 & 1) * 4 + t) ^ (row & 7);
    *reinterpret_cast<uint4*>(dst + chunk16 * 16) =
        make_uint4(packed[4 * t], packed[4 * t + 1], packed[4 * t + 2], packed[4 * t + 3]);
  }
}

// Same exponentials, but P goes to tensor memory (two bf16 keys per 32-bit column, the layout
// tcgen05.mma reads an A operand from): 32 scores -> 16 columns starting at `p_addr`.
__device__ __forceinline__ void v2_chunk_exp_tmem(const uint32_t (&r)[32], float c, float mc,
                                                  bool masked, int valid, uint32_t p_addr,
                                                  float2& sum2) {
  uint32_t packed[16];
  const float2 cc = make_float2(c, c), mm = make_float2(-mc, -mc);
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const float2 x = ffma2(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), cc, mm);
    float p0 = ex2(x.x), p1 = ex2(x.y);
    if (masked) {
      p0 = (i < valid) ? p0 : 0.0f;
      p1 = (i + 1 < valid) ? p1 : 0.0f;
    }
    sum2 = fadd2(sum2, make_float2(p0, p1));
    __nv_bfloat162 hb = __floats2bfloat162_rn(p0, p1);
    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hb);
  }
  tmem_st_32x16(p_addr, packed);
}

bool use_tmem_p() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LT_FLASH_TMEM_P");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v != 0;
}

template <int D>
struct Fwd2Smem {
  static constexpr int DC = D / 64;                          // 64-wide head-dim chunks
  static constexpr int TILE = DC * CHUNK_BYTES;              // one [128 x D] operand
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + TILE;                 // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * TILE;             // 2 stages
  static constexpr int OFF_P = OFF_V + 2 * TILE;             // 128 x 128 bf16 = 2 chunks
  static constexpr int OFF_BAR = OFF_P + 2 * CHUNK_BYTES;
  // 128 score columns + D output columns (+ 64 columns of bf16 P when P stays in tensor memory)
  static constexpr int TMEM_COLS = D == 64 ? 256 : 512;
  static constexpr int P_COL = 128 + D;
  static constexpr int TOTAL = OFF_BAR + 256;
};

template <int D>
__global__ void __launch_bounds__(V2_THREADS, (D == 64 ? 2 : 1))
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using L = Fwd2Smem<D>;
  constexpr int DC = L::DC;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(&g_attn_error, 0, 40);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* v_full = bars + 3;        // 2
  uint64_t* kv_empty = bars + 5;      // 2
  uint64_t* s_full = bars + 7;        // 1
  uint64_t* s_empty = bars + 8;       // 1
  uint64_t* p_full = bars + 9;        // 1
  uint64_t* o_full = bars + 10;       // 1
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp_idx = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = (int)gridDim.z - 1 - (int)blockIdx.z;   // longest tiles first, over the WHOLE grid
  const int h = blockIdx.x, b = blockIdx.y;
  const int q0 = q_tile * BM;
  const int n_kv_all = (p.S + BN - 1) / BN;
  const int n_kv = p.causal ? (q_tile + 1 < n_kv_all ? q_tile + 1 : n_kv_all) : n_kv_all;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&k_full[i]), 1);
      mbar_init(smem_u32(&v_full[i]), 1);
      mbar_init(smem_u32(&kv_empty[i]), 1);
    }
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(s_empty), 32 * V2_SOFTMAX_WARPS);
    mbar_init(smem_u32(p_full), 32 * V2_SOFTMAX_WARPS);
    mbar_init(smem_u32(o_full), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp_idx == 1) {
    tmem_alloc(smem_u32(tmem_holder), L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  pdl_enter();   // q, k, v come from the previous kernel
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 128;

  if (warp_idx == 0) {
    if (lane == 0) {
      const uint32_t qb = smem_u32(q_full);
      mbar_arrive_expect_tx(qb, L::TILE);
#pragma unroll
      for (int c = 0; c < DC; ++c)
        tma_load_4d(smem_u32(smem + L::OFF_Q + c * CHUNK_BYTES), &tm_q, qb, 64 * c, q0, h, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait_bounded(smem_u32(&kv_empty[st]), ((j >> 1) & 1) ^ 1, abort_flag,
                               &g_attn_error, 51))
          break;
        const uint32_t kb = smem_u32(&k_full[st]), vb = smem_u32(&v_full[st]);
        mbar_arrive_expect_tx(kb, L::TILE);
#pragma unroll
        for (int c = 0; c < DC; ++c)
          tma_load_4d(smem_u32(smem + L::OFF_K + st * L::TILE + c * CHUNK_BYTES), &tm_k, kb, 64 * c,
                      j * BN, h, b);
        mbar_arrive_expect_tx(vb, L::TILE);
#pragma unroll
        for (int c = 0; c < DC; ++c)
          tma_load_4d(smem_u32(smem + L::OFF_V + st * L::TILE + c * CHUNK_BYTES), &tm_v, vb, 64 * c,
                      j * BN, h, b);
      }
    }
  } else if (warp_idx == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(BM, D, 0, 1);
      bool ok = mbar_wait_bounded(smem_u32(q_full), 0, abort_flag, &g_attn_error, 52);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait_bounded(smem_u32(&k_full[st]), (j >> 1) & 1, abort_flag, &g_attn_error, 53))
          return false;
        // the softmax warps have copied the previous scores out of TMEM
        if (!mbar_wait_bounded(smem_u32(s_empty), (j & 1) ^ 1, abort_flag, &g_attn_error, 54))
          return false;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          const uint64_t qd = make_smem_desc_sw128(smem_u32(smem + L::OFF_Q + c * CHUNK_BYTES), 16, 1024);
          const uint64_t kd = make_smem_desc_sw128(
              smem_u32(smem + L::OFF_K + st * L::TILE + c * CHUNK_BYTES), 16, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16(tmem_s, qd + (uint64_t)(ks * 2), kd + (uint64_t)(ks * 2), idesc_s,
                      (c > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(s_full));
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j & 1;
        if (j + 1 < n_kv) {
          if (!issue_s(j + 1)) { ok = false; break; }
        }
        if (!mbar_wait_bounded(smem_u32(&v_full[st]), (j >> 1) & 1, abort_flag, &g_attn_error, 55) ||
            !mbar_wait_bounded(smem_u32(p_full), j & 1, abort_flag, &g_attn_error, 56)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // O[128 x D] (+)= P[128 x 128 keys] V[128 keys x D]
        if (p.tmem_p) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {     // 16 keys = 8 TMEM columns of P per step
            const uint32_t v_addr = smem_u32(smem + L::OFF_V + st * L::TILE) + (ks * 16) * 128;
            const uint64_t vd = make_smem_desc_sw128(v_addr, CHUNK_BYTES, 1024);
            umma_bf16_ts(tmem_o, tmem_base + L::P_COL + ks * 8, vd, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
          }
        } else
#pragma unroll
        for (int kc = 0; kc < 2; ++kc) {
          const uint64_t pd = make_smem_desc_sw128(smem_u32(smem + L::OFF_P + kc * CHUNK_BYTES), 16, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t v_addr = smem_u32(smem + L::OFF_V + st * L::TILE) + (kc * 64 + ks * 16) * 128;
            const uint64_t vd = make_smem_desc_sw128(v_addr, CHUNK_BYTES, 1024);
            umma_bf16(tmem_o, pd + (uint64_t)(ks * 2), vd, idesc_o, (j > 0 || kc > 0 || ks > 0) ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(o_full));
        umma_commit(smem_u32(&kv_empty[st]));
      }
    }
  } else {
    // ------------------------------ softmax / output ------------------------------
    const int quad = warp_idx & 3;
    const int half = (warp_idx - 2) >> 2;      // keys [64 half, 64 half + 64) of every tile
    const int row = quad * 32 + lane;
    const int qi = q0 + row;
    const uint32_t lane_base = ((uint32_t)(quad * 32)) << 16;
    const float c = p.scale_log2;
    float m_used = -INFINITY;
    float2 l2 = make_float2(0.0f, 0.0f);       // this thread's part of the row sum
    bool ok = true;
    uint8_t* p_row = smem + L::OFF_P + (row >> 3) * 1024 + (row & 7) * 128;

    for (int j = 0; ok && j < n_kv; ++j) {
      if (!mbar_wait_bounded_warp(smem_u32(s_full), j & 1, abort_flag, &g_attn_error, 57)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int k0 = j * BN;
      const bool need_mask = (p.causal && k0 + BN - 1 > q0) || (k0 + BN > p.S);
      int valid = BN;
      if (need_mask) {
        int lim = p.S - k0;
        if (p.causal) { int cl = qi - k0 + 1; lim = cl < lim ? cl : lim; }
        valid = lim < 0 ? 0 : (lim > BN ? BN : lim);
      }
      // pass 1: row maximum over all 128 scores, TMEM reads double buffered
      uint32_t ra[32], rb[32];
      const uint32_t s_addr = tmem_s + lane_base;
      const int own_c = half * 64;
      float mx = -INFINITY;
      tmem_ld_32x32(s_addr, ra);
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 32, rb);
      mx = v2_chunk_max(ra, mx, need_mask, valid);
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 64, ra);
      mx = v2_chunk_max(rb, mx, need_mask, valid - 32);
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 96, rb);
      mx = v2_chunk_max(ra, mx, need_mask, valid - 64);
      tmem_ld_wait();
      mx = v2_chunk_max(rb, mx, need_mask, valid - 96);

      float alpha = 1.0f;
      bool rescale = false;
      if (j == 0) {
        m_used = mx;
      } else if ((mx - m_used) * c > V2_RESCALE_LOG2) {
        alpha = ex2((m_used - mx) * c);
        m_used = mx;
        rescale = true;
      }
      if (j > 0) {
        // P V of the previous tile has finished: the P tile is free and O is settled
        if (!mbar_wait_bounded_warp(smem_u32(o_full), (j - 1) & 1, abort_flag, &g_attn_error, 58)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
          for (int oc = 0; oc < D / 64; ++oc) {     // this thread's D/2 output columns, 32 at a time
            const uint32_t o_addr = tmem_o + lane_base + half * (D / 2) + oc * 32;
            tmem_ld_32x32(o_addr, ra);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ra[i] = __float_as_uint(__uint_as_float(ra[i]) * alpha);
            tmem_st_32x16(o_addr, *reinterpret_cast<uint32_t(*)[16]>(&ra[0]));
            tmem_st_32x16(o_addr + 16, *reinterpret_cast<uint32_t(*)[16]>(&ra[16]));
          }
          tmem_st_wait();
          l2.x *= alpha;
          l2.y *= alpha;
        }
      }
      // pass 2: this thread's 64 scores -> exponentials -> P; the score buffer is handed back
      // to the tensor core as soon as both chunks are in registers
      tmem_ld_32x32(s_addr + own_c, ra);
      tmem_ld_32x32(s_addr + own_c + 32, rb);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(s_empty));
      const float mc = (m_used == -INFINITY) ? 0.0f : m_used * c;
      if (p.tmem_p) {
        const uint32_t p_addr = tmem_base + lane_base + L::P_COL + half * 32;
        v2_chunk_exp_tmem(ra, c, mc, need_mask, valid - own_c, p_addr, l2);
        v2_chunk_exp_tmem(rb, c, mc, need_mask, valid - own_c - 32, p_addr + 16, l2);
        tmem_st_wait();
      } else {
        v2_chunk_exp_store(ra, c, mc, need_mask, valid - own_c, p_row, half * 2, row, l2);
        v2_chunk_exp_store(rb, c, mc, need_mask, valid - own_c - 32, p_row, half * 2 + 1, row, l2);
      }
      tc_fence_before_sync();
      fence_proxy_async();
      mbar_arrive(smem_u32(p_full));
    }
    if (ok && n_kv > 0) {
      if (mbar_wait_bounded_warp(smem_u32(o_full), (n_kv - 1) & 1, abort_flag, &g_attn_error, 59)) {
        tc_fence_after_sync();
        // the P tile is free now: the two halves of a row meet there to add their sums
        float* lsum = reinterpret_cast<float*>(smem + L::OFF_P);
        const float l_mine = l2.x + l2.y;
        lsum[half * 128 + row] = l_mine;
        // all 256 threads meet on the (now unused) p_full barrier: a bounded wait, unlike bar.sync
        mbar_arrive(smem_u32(p_full));
        const bool met = mbar_wait_bounded_warp(smem_u32(p_full), n_kv & 1, abort_flag, &g_attn_error, 60);
        const float l = l_mine + lsum[(1 - half) * 128 + row];
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        __nv_bfloat16* orow = p.o + (long long)b * p.o_sb + (long long)qi * p.o_ss +
                              (long long)h * p.o_sh + half * (D / 2);
#pragma unroll
        for (int oc = 0; oc < D / 64; ++oc) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_o + lane_base + half * (D / 2) + oc * 32, r);
          tmem_ld_wait();
          if (met && qi < p.S) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 u;
              __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
              for (int t = 0; t < 4; ++t)
                hb[t] = __floats2bfloat162_rn(__uint_as_float(r[i + 2 * t]) * inv,
                                              __uint_as_float(r[i + 2 * t + 1]) * inv);
              *reinterpret_cast<uint4*>(orow + oc * 32 + i) = u;
            }
          }
        }
        if (met && qi < p.S) {
          if (p.lse && half == 0)
            p.lse[((long long)b * p.H + h) * p.S + qi] =
                (l > 0.0f) ? m_used * p.scale + __logf(l) : -INFINITY;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp_idx == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

template <int D>
cudaError_t launch_fwd_v2(const AttnArgs& a, cudaStream_t stream) {
  using L = Fwd2Smem<D>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd2_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  CUtensorMap tq, tk, tv;
  if (!attn_detail::make_qkv_map(&tq, a.q, a.D, a.S, a.H, a.B, a.q_ss, a.q_sh, a.q_sb, BM) ||
      !attn_detail::make_qkv_map(&tk, a.k, a.D, a.S, a.H, a.B, a.k_ss, a.k_sh, a.k_sb, BN) ||
      !attn_detail::make_qkv_map(&tv, a.v, a.D, a.S, a.H, a.B, a.v_ss, a.v_sh, a.v_sb, BN))
    return cudaErrorInvalidValue;
  FwdParams p;
  p.S = a.S; p.H = a.H; p.causal = a.causal;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.o = (__nv_bfloat16*)a.o;
  p.o_sb = a.o_sb; p.o_ss = a.o_ss; p.o_sh = a.o_sh;
  p.lse = a.lse;
  p.tmem_p = use_tmem_p() ? 1 : 0;
  dim3 grid(a.H, a.B, (a.S + BM - 1) / BM);   // tile index slowest: the hardware hands out the longest tiles of every head first
  cudaError_t le = launch_pdl(flash_fwd2_kernel<D>, grid, dim3(V2_THREADS), L::TOTAL, stream, tq, tk, tv, p);
  if (le != cudaSuccess) return le;
  g_attn_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

// LT_FLASH_FWD_V1=1 selects the first-generation kernel (comparison runs)
bool use_fwd_v1() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LT_FLASH_FWD_V1");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v != 0;
}

template <int D>
cudaError_t launch_fwd(const AttnArgs& a, cudaStream_t stream) {
  using L = FwdSmem<D>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  CUtensorMap tq, tk, tv;
  if (!attn_detail::make_qkv_map(&tq, a.q, a.D, a.S, a.H, a.B, a.q_ss, a.q_sh, a.q_sb, BM) ||
      !attn_detail::make_qkv_map(&tk, a.k, a.D, a.S, a.H, a.B, a.k_ss, a.k_sh, a.k_sb, BN) ||
      !attn_detail::make_qkv_map(&tv, a.v, a.D, a.S, a.H, a.B, a.v_ss, a.v_sh, a.v_sb, BN))
    return cudaErrorInvalidValue;
  FwdParams p;
  p.S = a.S; p.H = a.H; p.causal = a.causal;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.o = (__nv_bfloat16*)a.o;
  p.o_sb = a.o_sb; p.o_ss = a.o_ss; p.o_sh = a.o_sh;
  p.lse = a.lse;
  p.tmem_p = 0;
  dim3 grid(a.H, a.B, (a.S + BM - 1) / BM);   // tile index slowest: the hardware hands out the longest tiles of every head first
  cudaError_t le = launch_pdl(flash_fwd_kernel<D>, grid, dim3(NUM_THREADS), L::TOTAL, stream, tq, tk, tv, p);
  if (le != cudaSuccess) return le;
  g_attn_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

bool strides_ok(int64_t ss, int64_t sh, int64_t sb) {
  return ss % 8 == 0 && sh % 8 == 0 && sb % 8 == 0;
}

}  // namespace

cudaError_t flash_attention_forward(const AttnArgs& a, cudaStream_t stream) {
  if (a.B <= 0 || a.H <= 0 || a.S <= 0) return cudaSuccess;
  if (a.D != 64 && a.D != 128) return cudaErrorInvalidValue;
  if (!strides_ok(a.q_ss, a.q_sh, a.q_sb) || !strides_ok(a.k_ss, a.k_sh, a.k_sb) ||
      !strides_ok(a.v_ss, a.v_sh, a.v_sb) || !strides_ok(a.o_ss, a.o_sh, a.o_sb))
    return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) |
       reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.o)) & 15)
    return cudaErrorInvalidValue;
  if (a.D == 64) return use_fwd_v1() ? launch_fwd<64>(a, stream) : launch_fwd_v2<64>(a, stream);
  return use_fwd_v1() ? launch_fwd<128>(a, stream) : launch_fwd_v2<128>(a, stream);
}

}  // namespace lt
