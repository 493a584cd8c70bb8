// Host-side interface of the bf16 tensor-core GEMM (tcgen05 + TMEM + TMA).
//
// Replaces the reference's cuBLAS SGEMM call sites (csrc/cuda/ops/matmul.cu:92-195):
// one kernel covers matmul, bmm and every transposed form backward needs, so no
// transposed copy is ever materialised (the reference transposes in
// lua/luatorch/autograd.lua:105-114).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace lt {

enum GemmAct : int {
  GEMM_ACT_NONE = 0,
  GEMM_ACT_GELU = 1,    // out = gelu(acc + bias); optional aux_out receives acc + bias
  GEMM_ACT_DGELU = 2,   // out = acc * gelu'(aux_in)
  GEMM_ACT_RELU = 3,    // out = max(acc + bias, 0)
  GEMM_ACT_DRELU = 4,   // out = acc * (aux_in > 0)
};

// C[b] = act(alpha * op(A[b]) * op(B[b]) + bias) + residual (+ C[b] if accumulate)
//
// Operand layouts (bf16, innermost stride 1):
//   a_mn_major == 0 : A stored [M, K] with row stride lda      ("K-major")
//   a_mn_major == 1 : A stored [K, M] with row stride lda      ("M-major", i.e. A^T in memory)
//   b_mn_major == 0 : B stored [N, K] with row stride ldb      ("K-major", i.e. B^T in memory)
//   b_mn_major == 1 : B stored [K, N] with row stride ldb      ("N-major", plain row-major B)
// Batches are addressed with two nested batch indices (inner count `batch_inner`,
// outer count `batch_outer`) so that [B, S, H, d]-strided attention operands need
// no re-layout; element strides per operand.
struct GemmArgs {
  int M = 0, N = 0, K = 0;
  const void* A = nullptr;
  const void* B = nullptr;
  void* C = nullptr;
  int64_t lda = 0, ldb = 0, ldc = 0;
  int a_mn_major = 0, b_mn_major = 1;
  int batch_inner = 1, batch_outer = 1;
  int64_t a_stride_inner = 0, a_stride_outer = 0;
  int64_t b_stride_inner = 0, b_stride_outer = 0;
  int64_t c_stride_inner = 0, c_stride_outer = 0;
  float alpha = 1.0f;
  int c_fp32 = 0;        // output element type: 0 bf16, 1 fp32
  int accumulate = 0;    // C += result
  const void* bias = nullptr;  // [N]
  int bias_fp32 = 0;
  int act = GEMM_ACT_NONE;
  const void* residual = nullptr;  // bf16 [M, N], row stride ldr (unbatched use)
  int64_t ldr = 0;
  void* aux_out = nullptr;         // bf16 [M, N] pre-activation, row stride ldc
  const void* aux_in = nullptr;    // bf16 [M, N] pre-activation for DGELU/DRELU, row stride ld_aux
  int64_t ld_aux = 0;
  int causal_tiles = 0;  // 1: skip output tiles strictly above the diagonal (n0 > m0 + BM - 1);
                         // 2: skip tiles strictly below (m0 > n0 + BN - 1)
  int causal_k = 0;      // 1: the k loop of the output tile at row m0 stops at k = m0 + 128
                         //    (A is lower block-triangular in 128-blocks: attention dS / P)
  // n > 0: this product reads nothing that the n kernels launched just before it on `stream`
  // write and writes nothing they touch (n = 1: the weight-gradient GEMM after the
  // input-gradient GEMM of the same layer).  Under programmatic dependent launch it then works
  // in their tail and waits for them only before it exits; everything older is complete by
  // then (see the launch rules in common.cuh).  Without the launch attribute it does nothing.
  int overlap_prev = 0;
  // Optional scratch for split-K (fp32, device memory valid on `stream`).  When a long-K
  // product has too few output tiles to fill the chip (weight gradients: K = tokens), K is cut
  // into S slices that run as S batches into workspace[S][M][N], and a second kernel sums the
  // slices in fixed order (deterministic) into C.  Without a workspace no split is made.
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  // Optional: B is sharded by rows over `world` GPUs and gathered INSIDE the kernel
  // (parameter all-gather fused into the consuming GEMM), see GemmGather.
  const struct GemmGather* gather = nullptr;
};

// All-gather of B fused into the GEMM.  Every rank holds a full-size copy of B ([K, N], row
// stride ldb, b_mn_major = 1) in peer-mapped memory, of which only rows
// [p K/world, (p+1) K/world) are up to date on rank p.  The kernel
//   1. tells the peers that the local shard is final and waits (bounded) for theirs,
//   2. lets the epilogue warps of all CTAs pull the remote shards into the local copy with
//      16-byte peer loads, in the order (rank+1, rank+2, ...) and counts each finished shard in
//      `flags`,
//   3. runs the k loop of every tile starting at the local shard, the TMA producer waiting
//      (bounded) for a shard's flag only when it first needs rows of that shard,
// so each remote byte crosses NVLink once and the transfer hides behind the first tiles'
// math.  After the call the local copy of B is complete.  `flags` must be zero on entry.
struct GemmGather {
  const uint64_t* b_ptrs = nullptr;       // device table [world]: every rank's copy of B
  const uint64_t* signal_ptrs = nullptr;  // device table [world]: signal pads (as in csrc/comm)
  uint32_t* flags = nullptr;              // local device words [world + 1], zero on entry
  int rank = 0, world = 1;
  uint32_t epoch = 0;                     // same on every rank, increases per collective
  int* status = nullptr;                  // [8] device ints, zero when healthy
  int done_barrier = 1;                   // wait until every peer has finished copying our shard
};

// Bytes of workspace with which `args` would use split-K (0: it would not split).
size_t gemm_split_k_workspace_bytes(const GemmArgs& args);

// Returns cudaSuccess or the launch error. Uses the tensor-core path whenever the
// operands satisfy TMA alignment (base 16 B aligned, lda/ldb multiples of 8
// elements); otherwise a SIMT fallback handles the call.
cudaError_t gemm_bf16(const GemmArgs& args, cudaStream_t stream);

// True if `args` is eligible for the tcgen05 path.
bool gemm_uses_tensor_cores(const GemmArgs& args);

// Device-side status word written by bounded waits (0 = ok). Reading synchronises.
int gemm_last_device_error();
void gemm_clear_device_error();

// Number of kernel launches issued by this translation unit since process start.
uint64_t gemm_launch_count();

}  // namespace lt
