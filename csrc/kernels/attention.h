// Flash attention (forward and backward) on tcgen05 tensor cores.
//
// The reference has a forward-only kernel in which 32 threads load K/V tiles and ONE thread
// per query row does all the arithmetic (csrc/cuda/ops/flash_attention.cu:19-113), no
// log-sum-exp output and no backward; at head_dim 128 it cannot launch at all (66 KB of
// dynamic shared memory without the opt-in attribute, :130-136).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace lt {

// All tensors are bf16 with unit stride along head_dim and arbitrary element strides for
// batch (sb), sequence (ss) and head (sh), so the [B*S, 3*E] output of a fused QKV
// projection is consumed in place.  lse / delta are fp32 [B, H, S].
struct AttnArgs {
  int B = 0, H = 0, S = 0, D = 0;   // D in {64, 128}
  const void* q = nullptr; const void* k = nullptr; const void* v = nullptr;
  void* o = nullptr;
  float* lse = nullptr;
  int64_t q_sb = 0, q_ss = 0, q_sh = 0;
  int64_t k_sb = 0, k_ss = 0, k_sh = 0;
  int64_t v_sb = 0, v_ss = 0, v_sh = 0;
  int64_t o_sb = 0, o_ss = 0, o_sh = 0;
  int causal = 1;
  float scale = 1.0f;               // softmax(scale * Q K^T)
};

struct AttnBwdArgs {
  const void* d_o = nullptr;
  int64_t do_sb = 0, do_ss = 0, do_sh = 0;
  void* dq = nullptr; void* dk = nullptr; void* dv = nullptr;
  int64_t dq_sb = 0, dq_ss = 0, dq_sh = 0;
  int64_t dk_sb = 0, dk_ss = 0, dk_sh = 0;
  int64_t dv_sb = 0, dv_ss = 0, dv_sh = 0;
  float* delta = nullptr;           // scratch [B, H, S]: rowsum(dO * O)
  // Optional bf16 scratch [B, H, S, S].  When given (and S is a multiple of 128) the dK/dV
  // kernel also writes its dS tiles there and dQ = dS K runs as a batched tensor-core GEMM
  // over them instead of a third kernel that would rebuild S, dP and dS a second time.
  void* ds_scratch = nullptr;
};

cudaError_t flash_attention_forward(const AttnArgs& a, cudaStream_t stream);
cudaError_t flash_attention_backward(const AttnArgs& a, const AttnBwdArgs& b, cudaStream_t stream);

int attention_last_device_error();
uint64_t attention_launch_count();

}  // namespace lt
