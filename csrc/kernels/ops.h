// Raw-pointer launch interface of the memory-bound sm_100a kernels.  No framework
// types appear here: the PyTorch binding and the C ABI library both call these.
// All launchers enqueue on `stream`, never synchronise, and return the launch status.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace lt {

enum DType : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };

enum BinaryOp : int { BIN_ADD = 0, BIN_SUB = 1, BIN_MUL = 2, BIN_DIV = 3 };
enum ScalarOp : int { SC_ADD = 0, SC_MUL = 1, SC_DIV = 2, SC_POW = 3, SC_GT = 4 };
enum UnaryOp : int {
  UN_NEG = 0, UN_ABS = 1, UN_SQRT = 2, UN_LOG = 3, UN_EXP = 4,
  UN_RELU = 5, UN_SIGMOID = 6, UN_TANH = 7, UN_GELU = 8, UN_SILU = 9,
};
enum ReduceOp : int { RED_SUM = 0, RED_MAX = 1, RED_MIN = 2 };

uint64_t ops_launch_count();
// Programmatic dependent launch at run time: 0 = off, 1 = on, -1 = follow LT_PDL (default).
void set_pdl_override(int v);

// ---- elementwise family (reference: csrc/cuda/ops/arithmetic.cu:57-143, activation.cu:25-60)
cudaError_t binary_op(int op, int dtype, const void* a, const void* b, void* out, int64_t n,
                      cudaStream_t s);
cudaError_t scalar_op(int op, int dtype, const void* a, float scalar, void* out, int64_t n,
                      cudaStream_t s);
cudaError_t unary_op(int op, int dtype, const void* a, void* out, int64_t n, cudaStream_t s);
// dx = dy * f'(x) for the activations above (UN_RELU .. UN_SILU)
cudaError_t unary_backward(int op, int dtype, const void* x, const void* dy, void* dx, int64_t n,
                           cudaStream_t s);
cudaError_t add_broadcast(int dtype, const void* a, const void* bias, void* out, int64_t rows,
                          int64_t cols, cudaStream_t s);
// out[r, c] = a[r, c] * scale[c] + shift[c] (shift may be null)
cudaError_t affine_cols(int dtype, const void* a, const void* scale, const void* shift, void* out,
                        int64_t rows, int64_t cols, cudaStream_t s);
// out[c] = sum_r in[r, c]  (deterministic two-stage; `scratch` holds ceil(rows/128)*cols floats)
cudaError_t column_sum(int dtype, const void* in, int64_t ld, void* out, int out_dtype,
                       int accumulate, int64_t rows, int64_t cols, float* scratch, cudaStream_t s);
int64_t column_sum_scratch_floats(int64_t rows, int64_t cols);
cudaError_t cast(int src_dtype, const void* src, int dst_dtype, void* dst, int64_t n,
                 cudaStream_t s);
cudaError_t transpose2d(int dtype, const void* in, void* out, int64_t rows, int64_t cols,
                        cudaStream_t s);
cudaError_t fill_random(int dtype, void* out, int64_t n, uint64_t seed, uint64_t offset,
                        int normal, cudaStream_t s);
// out = x * mask / (1-p), mask ~ Bernoulli(1-p) regenerated from (seed, offset) in backward
// `dyn_offset` (device, optional) is added to `offset` inside the kernel: a replayed CUDA graph
// gets fresh masks by advancing that one word between replays.
cudaError_t dropout(int dtype, const void* x, void* out, int64_t n, float p, uint64_t seed,
                    uint64_t offset, cudaStream_t s, const uint64_t* dyn_offset = nullptr);
// fp32 a -> bf16 hi and lo parts (a ~= hi + lo) used by the fp32-accurate GEMM path
cudaError_t split_bf16(const float* a, void* hi, void* lo, int64_t n, cudaStream_t s);

// ---- reductions (reference: csrc/cuda/ops/arithmetic.cu:148-208, 339-448; matmul.cu:232-256)
// Single launch; the result is left in `out` (one fp32 on the device).  `scratch` needs
// reduce_scratch_bytes() and must be zero before the first use (the kernel re-zeroes it).
size_t reduce_scratch_bytes();
cudaError_t reduce_all(int op, int dtype, const void* a, int64_t n, float scale, float* out,
                       void* scratch, cudaStream_t s);
cudaError_t dot_all(int dtype, const void* a, const void* b, int64_t n, float* out, void* scratch,
                    cudaStream_t s);
// flag[0] |= any(!isfinite(a * inv_scale)); optionally writes a * inv_scale back in place
cudaError_t check_finite_scale(int dtype, void* a, int64_t n, float scale, int write_back,
                               int* flag, cudaStream_t s);

// ---- softmax and losses (reference: csrc/cuda/ops/activation.cu:65-112, loss.cu:27-125)
cudaError_t softmax_rows(int dtype, const void* in, void* out, int64_t rows, int64_t cols,
                         int64_t ld, cudaStream_t s);
// in-place scaled, optionally causally masked softmax over [batch, rows, cols] scores
cudaError_t softmax_scores(void* scores_bf16, int64_t batch, int64_t rows, int64_t cols,
                           int64_t ld, int causal, cudaStream_t s);
// ds = p * (dp - rowsum(dp * p)) * scale, in place over dp; p and dp are bf16 [n_rows, cols]
cudaError_t softmax_scores_backward(const void* p_bf16, void* dp_bf16, int64_t n_rows,
                                    int64_t cols, int64_t ld, float scale, int causal,
                                    int64_t rows_per_batch, cudaStream_t s);
// row_loss[r] = lse_r - logit[r, label_r]; lse[r] saved for backward.  The mean is a
// reduce_all over row_loss (fixed order, reproducible).
// labels: int64, int32 or fp32 (label_kind 0/1/2).  err_flag set on out-of-range label.
cudaError_t cross_entropy_forward(int dtype, const void* logits, int64_t ld, const void* labels,
                                  int label_kind, int64_t rows, int64_t cols, float* lse,
                                  float* row_loss, int* err_flag, cudaStream_t s);
// dlogits = (softmax - onehot) * grad_scale (grad_scale read from device if gs_dev != null)
// Forward + backward in one kernel: on return `logits` holds (softmax - onehot) * grad_scale.
cudaError_t cross_entropy_fused(int dtype, void* logits, int64_t ld, const void* labels,
                                int label_kind, int64_t rows, int64_t cols, float* lse,
                                float* row_loss, int* err_flag, float grad_scale, cudaStream_t s);
cudaError_t cross_entropy_backward(int dtype, const void* logits, int64_t ld, const void* labels,
                                   int label_kind, int64_t rows, int64_t cols, const float* lse,
                                   float grad_scale, const float* gs_dev, void* dlogits,
                                   int64_t ld_out, cudaStream_t s);
// mode 0: mse, 1: mae.  loss_out[0] = mean; scratch as reduce_all.
cudaError_t pointwise_loss(int mode, int dtype, const void* pred, const void* target, int64_t n,
                           float* loss_out, void* scratch, cudaStream_t s);
cudaError_t pointwise_loss_backward(int mode, int dtype, const void* pred, const void* target,
                                    int64_t n, float grad_scale, void* dpred, cudaStream_t s);

// ---- layernorm / gelu+bias (reference: csrc/cuda/ops/fused.cu:26-127; backward has none there)
cudaError_t layernorm_forward(int dtype, const void* x, const void* gamma, const void* beta,
                              int param_dtype, float eps, void* y, float* mean, float* rstd,
                              int64_t rows, int64_t cols, cudaStream_t s);
// dx (+= dx_add if given); dgamma/dbeta partial sums land in scratch then are reduced into
// dgamma/dbeta (dtype grad_dtype, accumulate flag).  `dxsum` (same dtype, own accumulate
// flag): when given and the fused path applies, the column sums of dx are produced by the same
// two launches (*dxsum_done = 1) - the bias gradient of a linear layer whose output, plus a
// residual, was this LayerNorm's input; otherwise *dxsum_done = 0 and the caller sums dx.
int64_t layernorm_backward_scratch_floats(int64_t rows, int64_t cols);
cudaError_t layernorm_backward(int dtype, const void* x, const void* dy, const void* gamma,
                               int param_dtype, const float* mean, const float* rstd,
                               const void* dx_add, void* dx, void* dgamma, void* dbeta,
                               int grad_dtype, int accumulate, float* scratch, int64_t rows,
                               int64_t cols, cudaStream_t s, void* dxsum = nullptr,
                               int dxsum_accumulate = 0, int* dxsum_done = nullptr,
                               int scratch_is_private = 0);
// `scratch_is_private`: the caller owns `scratch` outside the stream's caching allocator (it
// cannot be handed to the kernel launched next); the closing parameter reduction is then
// marked as a side kernel, so that a following GEMM may run beside it.
cudaError_t gelu_bias_forward(int dtype, const void* x, const void* bias, int bias_dtype,
                              void* out, int64_t rows, int64_t cols, cudaStream_t s);
// dx = dy * gelu'(x + bias)
cudaError_t gelu_bias_backward(int dtype, const void* x, const void* bias, int bias_dtype,
                               const void* dy, void* dx, int64_t rows, int64_t cols,
                               cudaStream_t s);

// ---- embedding (reference: lua/luatorch/nn/embedding.lua:34-82, positional.lua:109-145)
// out[t, :] = table[ids[t], :] (+ pos_table[t % seq_len, :]); ids int64/int32/fp32 (kind 0/1/2)
cudaError_t embedding_forward(int dtype, const void* table, const void* ids, int id_kind,
                              const void* pos_table, int64_t seq_len, void* out, int64_t n_tokens,
                              int64_t dim, int64_t vocab, int* err_flag, cudaStream_t s);
// Deterministic scatter-add: dtable[v, :] = sum_{t: ids[t]==v} dy[t, :] for every v (rows with
// no token are written as zero unless accumulate).  workspace: embedding_backward_workspace().
size_t embedding_backward_workspace(int64_t n_tokens, int64_t vocab);
cudaError_t embedding_backward(int dtype, const void* dy, const void* ids, int id_kind,
                               void* dtable, int grad_dtype, int accumulate, int64_t n_tokens,
                               int64_t dim, int64_t vocab, void* workspace, cudaStream_t s);
// dpos[p, :] = sum_b dy[b*seq_len + p, :]; rows >= seq_len zeroed unless accumulate
cudaError_t positional_backward(int dtype, const void* dy, void* dpos, int grad_dtype,
                                int accumulate, int64_t batch, int64_t seq_len, int64_t max_seq,
                                int64_t dim, cudaStream_t s);

// ---- im2col / col2im (reference: csrc/ops/conv2d.c:11-49, CPU only there)
cudaError_t im2col(int dtype, const void* in, void* cols, int batch, int C, int H, int W, int k,
                   int stride, int pad, int64_t ld_cols, cudaStream_t s);
cudaError_t col2im(int dtype, const void* cols, void* din, int batch, int C, int H, int W, int k,
                   int stride, int pad, int64_t ld_cols, cudaStream_t s);
// [B*oh*ow, C] (NHWC-flat) <-> [B, C, oh*ow] (NCHW-flat)
cudaError_t nhwc_to_nchw(int dtype, const void* in, void* out, int batch, int C, int hw,
                         int to_nchw, cudaStream_t s);

// ---- optimizers over flat arenas (reference: csrc/cuda/ops/fused.cu:132-174,
//      lua/luatorch/optim/sgd.lua:33-56)
struct AdamArgs {
  float lr, beta1, beta2, eps, bc1, bc2;
  float grad_scale;          // multiplied into the gradient before use (1/world, 1/loss-scale)
  const int* skip_flag;      // device flag: nonzero => leave everything untouched (overflow)
  // device {lr, bc1, bc2}: when set, these replace the by-value fields, so that a captured
  // CUDA graph can be replayed with the step-dependent scalars of each new step
  const float* dyn = nullptr;
};
// Segment table: seg_end[i] = exclusive end element of segment i, seg_wd[i] = its weight decay.
cudaError_t adamw_flat(float* master, void* shadow_bf16, const void* grad, int grad_dtype,
                       float* m, float* v, int64_t n, const int64_t* seg_end, const float* seg_wd,
                       int nseg, AdamArgs args, cudaStream_t s);
cudaError_t sgd_flat(float* master, void* shadow_bf16, const void* grad, int grad_dtype,
                     float* vel, int64_t n, float lr, float momentum, int nesterov,
                     float grad_scale, cudaStream_t s, const float* dyn_lr = nullptr);
// Writes the step-dependent scalars that a replayed CUDA graph reads from device memory:
// dyn = {lr, bc1, bc2} (AdamArgs::dyn, sgd_flat's dyn_lr) and the dropout offset word.
// Either pointer may be null.  One single-thread launch, ordered before the graph by the stream.
cudaError_t set_step_scalars(float* dyn, float lr, float bc1, float bc2, uint64_t* dyn_offset,
                             uint64_t offset, cudaStream_t s);

}  // namespace lt
