// PyTorch-facing binding of the sm_100a kernels (module `luatorch_b200._C`).
// Tensors are only used for their storage: every kernel launch goes through the raw-pointer
// interfaces in csrc/kernels/ops.h and csrc/kernels/gemm.h on the current CUDA stream.
#include <cstdlib>
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>

#include <map>
#include <mutex>

#include "../kernels/gemm.h"
#include "../kernels/ops.h"
#include "../kernels/attention.h"
#include "../comm/comm_kernels.h"

namespace {

using at::Tensor;
using OptT = c10::optional<Tensor>;

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

void check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "luatorch_b200: ", what, " failed: ", cudaGetErrorString(e));
}

int dt(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return lt::DT_F32;
    case at::kBFloat16: return lt::DT_BF16;
    case at::kHalf: return lt::DT_F16;
    default: TORCH_CHECK(false, "luatorch_b200: unsupported dtype ", t.scalar_type());
  }
  return -1;
}
int label_kind(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kLong: return 0;
    case at::kInt: return 1;
    case at::kFloat: return 2;
    default: TORCH_CHECK(false, "luatorch_b200: labels/ids must be int64, int32 or float32");
  }
  return -1;
}
void need_cuda_contig(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
const void* optptr(const OptT& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// Per (device, stream) scratch for the single-launch reductions (ticket must start at zero).
void* reduce_scratch() {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, Tensor> cache;
  std::lock_guard<std::mutex> lock(mu);
  int dev = 0;
  cudaGetDevice(&dev);
  auto key = std::make_pair(dev, cur_stream());
  auto it = cache.find(key);
  if (it == cache.end()) {
    Tensor t = at::zeros({(int64_t)lt::reduce_scratch_bytes()},
                         at::TensorOptions().dtype(at::kByte).device(at::kCUDA, dev));
    it = cache.emplace(key, t).first;
  }
  return it->second.data_ptr();
}

Tensor scratch_floats(int64_t n, const Tensor& like) {
  return at::empty({n > 0 ? n : 1}, like.options().dtype(at::kFloat));
}

// ------------------------------------------------------------------------------ GEMM
// One-shot hint consumed by the next gemm() call: that product is independent of the `n`
// kernels launched just before it (lt::GemmArgs::overlap_prev).
static int g_next_gemm_overlap = 0;
void gemm_next_overlaps_prev(int64_t n) { g_next_gemm_overlap = (int)n; }

void gemm(const Tensor& A, const Tensor& B, Tensor& C, int64_t M, int64_t N, int64_t K,
          int64_t lda, int64_t ldb, int64_t ldc, bool a_mn, bool b_mn, int64_t batch_inner,
          int64_t batch_outer, int64_t a_si, int64_t a_so, int64_t b_si, int64_t b_so,
          int64_t c_si, int64_t c_so, double alpha, bool accumulate, const OptT& bias,
          int64_t act, const OptT& residual, int64_t ldr, const OptT& aux_out,
          const OptT& aux_in, int64_t ld_aux, int64_t causal_tiles) {
  // the hint is for THIS call only: taken before anything can throw
  const int overlap_prev = g_next_gemm_overlap;
  g_next_gemm_overlap = 0;
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && C.is_cuda(), "gemm operands must be CUDA tensors");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16,
              "gemm operands must be bfloat16");
  TORCH_CHECK(C.scalar_type() == at::kBFloat16 || C.scalar_type() == at::kFloat,
              "gemm output must be bfloat16 or float32");
  c10::cuda::CUDAGuard guard(A.device());
  lt::GemmArgs g;
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.A = A.data_ptr(); g.B = B.data_ptr(); g.C = C.data_ptr();
  g.lda = lda; g.ldb = ldb; g.ldc = ldc;
  g.a_mn_major = a_mn; g.b_mn_major = b_mn;
  g.batch_inner = (int)batch_inner; g.batch_outer = (int)batch_outer;
  g.a_stride_inner = a_si; g.a_stride_outer = a_so;
  g.b_stride_inner = b_si; g.b_stride_outer = b_so;
  g.c_stride_inner = c_si; g.c_stride_outer = c_so;
  g.alpha = (float)alpha;
  g.c_fp32 = C.scalar_type() == at::kFloat;
  g.accumulate = accumulate;
  if (bias.has_value()) {
    g.bias = bias->data_ptr();
    g.bias_fp32 = bias->scalar_type() == at::kFloat;
    TORCH_CHECK(g.bias_fp32 || bias->scalar_type() == at::kBFloat16, "bias must be f32 or bf16");
  }
  g.act = (int)act;
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16, "residual must be bfloat16");
    g.residual = residual->data_ptr();
    g.ldr = ldr;
  }
  if (aux_out.has_value()) g.aux_out = aux_out->data_ptr();
  if (aux_in.has_value()) { g.aux_in = aux_in->data_ptr(); g.ld_aux = ld_aux; }
  g.causal_tiles = (int)causal_tiles;
  g.overlap_prev = overlap_prev;
  // scratch for split-K comes from torch's caching allocator, so it is stream-ordered
  Tensor ws;
  const size_t ws_bytes = lt::gemm_split_k_workspace_bytes(g);
  if (ws_bytes) {
    ws = torch::empty({(int64_t)(ws_bytes / 4)}, C.options().dtype(torch::kFloat32));
    g.workspace = ws.data_ptr();
    g.workspace_bytes = ws_bytes;
  }
  check(lt::gemm_bf16(g, cur_stream()), "gemm");
}

// C = act(A @ B + bias) where B's row shards live on `world` GPUs and are gathered inside the
// GEMM kernel (lt::GemmGather).  `b_byte_offset` locates B inside every rank's symmetric buffer;
// `flags` (world + 1 int32 words) is zeroed here on the launching stream.
void gemm_gather(const Tensor& A, const Tensor& B_local, Tensor& C, int64_t M, int64_t N, int64_t K,
                 int64_t lda, int64_t ldb, int64_t ldc, const OptT& bias, int64_t act,
                 const OptT& aux_out, const Tensor& b_ptrs, const Tensor& signal_ptrs, Tensor& flags,
                 int64_t rank, int64_t world, int64_t epoch, Tensor& status, bool done_barrier) {
  TORCH_CHECK(A.is_cuda() && B_local.is_cuda() && C.is_cuda(), "gemm_gather operands must be CUDA tensors");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B_local.scalar_type() == at::kBFloat16 &&
              C.scalar_type() == at::kBFloat16, "gemm_gather works on bfloat16");
  TORCH_CHECK(flags.numel() >= world + 1 && flags.scalar_type() == at::kInt, "flags: int32[world+1]");
  c10::cuda::CUDAGuard guard(A.device());
  lt::GemmArgs g;
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.A = A.data_ptr(); g.B = B_local.data_ptr(); g.C = C.data_ptr();
  g.lda = lda; g.ldb = ldb; g.ldc = ldc;
  g.a_mn_major = 0; g.b_mn_major = 1;
  if (bias.has_value()) {
    g.bias = bias->data_ptr();
    g.bias_fp32 = bias->scalar_type() == at::kFloat;
  }
  g.act = (int)act;
  if (aux_out.has_value()) g.aux_out = aux_out->data_ptr();
  lt::GemmGather gg;
  gg.b_ptrs = (const uint64_t*)b_ptrs.data_ptr<int64_t>();
  gg.signal_ptrs = (const uint64_t*)signal_ptrs.data_ptr<int64_t>();
  gg.flags = (uint32_t*)flags.data_ptr<int>();
  gg.rank = (int)rank; gg.world = (int)world; gg.epoch = (uint32_t)epoch;
  gg.status = status.data_ptr<int>();
  gg.done_barrier = done_barrier ? 1 : 0;
  g.gather = &gg;
  check(cudaMemsetAsync(flags.data_ptr(), 0, (size_t)flags.numel() * 4, cur_stream()), "gemm_gather flags");
  check(lt::gemm_bf16(g, cur_stream()), "gemm_gather");
}

int64_t gemm_device_error() { return lt::gemm_last_device_error(); }

// ------------------------------------------------------------------------------ elementwise
Tensor binary(int64_t op, const Tensor& a, const Tensor& b, bool inplace) {
  need_cuda_contig(a, "a"); need_cuda_contig(b, "b");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "binary op dtype mismatch");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = inplace ? a : at::empty_like(a);
  check(lt::binary_op((int)op, dt(a), a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(),
                      cur_stream()), "binary_op");
  return out;
}
Tensor scalar(int64_t op, const Tensor& a, double s, bool inplace) {
  need_cuda_contig(a, "a");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = inplace ? a : at::empty_like(a);
  check(lt::scalar_op((int)op, dt(a), a.data_ptr(), (float)s, out.data_ptr(), a.numel(),
                      cur_stream()), "scalar_op");
  return out;
}
Tensor unary(int64_t op, const Tensor& a) {
  need_cuda_contig(a, "a");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty_like(a);
  check(lt::unary_op((int)op, dt(a), a.data_ptr(), out.data_ptr(), a.numel(), cur_stream()),
        "unary_op");
  return out;
}
Tensor unary_backward(int64_t op, const Tensor& x, const Tensor& dy) {
  need_cuda_contig(x, "x"); need_cuda_contig(dy, "dy");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = at::empty_like(x);
  check(lt::unary_backward((int)op, dt(x), x.data_ptr(), dy.data_ptr(), out.data_ptr(), x.numel(),
                           cur_stream()), "unary_backward");
  return out;
}
Tensor add_broadcast(const Tensor& a, const Tensor& bias) {
  need_cuda_contig(a, "a"); need_cuda_contig(bias, "bias");
  TORCH_CHECK(a.dim() == 2 && bias.numel() == a.size(1) && a.scalar_type() == bias.scalar_type());
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty_like(a);
  check(lt::add_broadcast(dt(a), a.data_ptr(), bias.data_ptr(), out.data_ptr(), a.size(0),
                          a.size(1), cur_stream()), "add_broadcast");
  return out;
}
Tensor affine_cols(const Tensor& a, const Tensor& scale, const OptT& shift) {
  need_cuda_contig(a, "a"); need_cuda_contig(scale, "scale");
  TORCH_CHECK(a.dim() == 2 && scale.numel() == a.size(1) && scale.scalar_type() == a.scalar_type());
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty_like(a);
  check(lt::affine_cols(dt(a), a.data_ptr(), scale.data_ptr(), optptr(shift), out.data_ptr(),
                        a.size(0), a.size(1), cur_stream()), "affine_cols");
  return out;
}
// out (optional, [cols], any float dtype) receives / accumulates the column sums of in[rows, cols]
Tensor column_sum(const Tensor& in, const OptT& out_opt, bool accumulate) {
  TORCH_CHECK(in.is_cuda() && in.dim() == 2 && in.stride(1) == 1);
  c10::cuda::CUDAGuard guard(in.device());
  Tensor out = out_opt.has_value() ? *out_opt : at::empty({in.size(1)}, in.options());
  Tensor scratch = scratch_floats(lt::column_sum_scratch_floats(in.size(0), in.size(1)), in);
  check(lt::column_sum(dt(in), in.data_ptr(), in.stride(0), out.data_ptr(), dt(out), accumulate,
                       in.size(0), in.size(1), scratch.data_ptr<float>(), cur_stream()),
        "column_sum");
  return out;
}
Tensor cast(const Tensor& a, at::ScalarType to) {
  need_cuda_contig(a, "a");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty(a.sizes(), a.options().dtype(to));
  check(lt::cast(dt(a), a.data_ptr(), dt(out), out.data_ptr(), a.numel(), cur_stream()), "cast");
  return out;
}
void cast_into(const Tensor& a, Tensor& out) {
  need_cuda_contig(a, "a"); need_cuda_contig(out, "out");
  TORCH_CHECK(a.numel() == out.numel());
  c10::cuda::CUDAGuard guard(a.device());
  check(lt::cast(dt(a), a.data_ptr(), dt(out), out.data_ptr(), a.numel(), cur_stream()), "cast");
}
Tensor transpose2d(const Tensor& a) {
  need_cuda_contig(a, "a");
  TORCH_CHECK(a.dim() == 2);
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty({a.size(1), a.size(0)}, a.options());
  check(lt::transpose2d(dt(a), a.data_ptr(), out.data_ptr(), a.size(0), a.size(1), cur_stream()),
        "transpose2d");
  return out;
}
void fill_random(Tensor& out, int64_t seed, int64_t offset, bool normal) {
  need_cuda_contig(out, "out");
  c10::cuda::CUDAGuard guard(out.device());
  check(lt::fill_random(dt(out), out.data_ptr(), out.numel(), (uint64_t)seed, (uint64_t)offset,
                        normal, cur_stream()), "fill_random");
}
// `dyn_offset`: optional int64[1] on the device, added to `offset` inside the kernel (graph replay)
Tensor dropout_dyn(const Tensor& x, double p, int64_t seed, int64_t offset, const OptT& dyn_offset) {
  need_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const uint64_t* dyn = nullptr;
  if (dyn_offset.has_value()) {
    TORCH_CHECK(dyn_offset->is_cuda() && dyn_offset->scalar_type() == at::kLong &&
                dyn_offset->numel() >= 1, "dyn_offset: int64 CUDA tensor expected");
    dyn = reinterpret_cast<const uint64_t*>(dyn_offset->data_ptr<int64_t>());
  }
  Tensor out = at::empty_like(x);
  check(lt::dropout(dt(x), x.data_ptr(), out.data_ptr(), x.numel(), (float)p, (uint64_t)seed,
                    (uint64_t)offset, cur_stream(), dyn), "dropout");
  return out;
}
Tensor dropout(const Tensor& x, double p, int64_t seed, int64_t offset) {
  return dropout_dyn(x, p, seed, offset, c10::nullopt);
}
std::vector<Tensor> split_bf16(const Tensor& a) {
  need_cuda_contig(a, "a");
  TORCH_CHECK(a.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(a.device());
  Tensor hi = at::empty(a.sizes(), a.options().dtype(at::kBFloat16));
  Tensor lo = at::empty_like(hi);
  check(lt::split_bf16(a.data_ptr<float>(), hi.data_ptr(), lo.data_ptr(), a.numel(), cur_stream()),
        "split_bf16");
  return {hi, lo};
}

// ------------------------------------------------------------------------------ reductions
Tensor reduce(int64_t op, const Tensor& a, double scale) {
  need_cuda_contig(a, "a");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty({1}, a.options().dtype(at::kFloat));
  check(lt::reduce_all((int)op, dt(a), a.data_ptr(), a.numel(), (float)scale,
                       out.data_ptr<float>(), reduce_scratch(), cur_stream()), "reduce_all");
  return out;
}
Tensor dot(const Tensor& a, const Tensor& b) {
  need_cuda_contig(a, "a"); need_cuda_contig(b, "b");
  TORCH_CHECK(a.numel() == b.numel() && a.scalar_type() == b.scalar_type());
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty({1}, a.options().dtype(at::kFloat));
  check(lt::dot_all(dt(a), a.data_ptr(), b.data_ptr(), a.numel(), out.data_ptr<float>(),
                    reduce_scratch(), cur_stream()), "dot_all");
  return out;
}
void check_finite_scale(Tensor& a, double scale, bool write_back, Tensor& flag) {
  need_cuda_contig(a, "a");
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(a.device());
  check(lt::check_finite_scale(dt(a), a.data_ptr(), a.numel(), (float)scale, write_back,
                               flag.data_ptr<int>(), cur_stream()), "check_finite_scale");
}

// ------------------------------------------------------------------------------ softmax / losses
Tensor softmax(const Tensor& a) {
  need_cuda_contig(a, "a");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t cols = a.dim() >= 2 ? a.size(-1) : a.numel();
  const int64_t rows = a.numel() / (cols > 0 ? cols : 1);
  Tensor out = at::empty_like(a);
  check(lt::softmax_rows(dt(a), a.data_ptr(), out.data_ptr(), rows, cols, cols, cur_stream()),
        "softmax_rows");
  return out;
}
void softmax_scores(Tensor& sc, int64_t batch, int64_t rows, int64_t cols, bool causal) {
  need_cuda_contig(sc, "scores");
  TORCH_CHECK(sc.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(sc.device());
  check(lt::softmax_scores(sc.data_ptr(), batch, rows, cols, cols, causal, cur_stream()),
        "softmax_scores");
}
void softmax_scores_backward(const Tensor& p, Tensor& dp, int64_t rows_per_batch, double scale,
                             bool causal) {
  need_cuda_contig(p, "p"); need_cuda_contig(dp, "dp");
  c10::cuda::CUDAGuard guard(p.device());
  const int64_t cols = p.size(-1);
  check(lt::softmax_scores_backward(p.data_ptr(), dp.data_ptr(), p.numel() / cols, cols, cols,
                                    (float)scale, causal, rows_per_batch, cur_stream()),
        "softmax_scores_backward");
}
// logits [rows, ld] with `cols` valid columns -> (loss[1] fp32, lse[rows] fp32, err[4] int:
// flag, row, offending label of the first out-of-range label seen)
std::vector<Tensor> cross_entropy_forward(const Tensor& logits, int64_t cols, const Tensor& labels) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  need_cuda_contig(labels, "labels");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t rows = logits.size(0);
  auto fo = logits.options().dtype(at::kFloat);
  Tensor lse = at::empty({rows}, fo), row_loss = at::empty({rows}, fo), loss = at::empty({1}, fo);
  Tensor err = at::zeros({4}, logits.options().dtype(at::kInt));
  check(lt::cross_entropy_forward(dt(logits), logits.data_ptr(), logits.stride(0),
                                  labels.data_ptr(), label_kind(labels), rows, cols,
                                  lse.data_ptr<float>(), row_loss.data_ptr<float>(),
                                  err.data_ptr<int>(), cur_stream()), "cross_entropy_forward");
  check(lt::reduce_all(lt::RED_SUM, lt::DT_F32, row_loss.data_ptr(), rows, 1.0f / (float)rows,
                       loss.data_ptr<float>(), reduce_scratch(), cur_stream()), "reduce_all");
  return {loss, lse, err};
}
// as cross_entropy_forward, and `logits` is overwritten with (softmax - onehot) * grad_scale
std::vector<Tensor> cross_entropy_fused(Tensor& logits, int64_t cols, const Tensor& labels,
                                        double grad_scale) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  need_cuda_contig(labels, "labels");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t rows = logits.size(0);
  auto fo = logits.options().dtype(at::kFloat);
  Tensor lse = at::empty({rows}, fo), row_loss = at::empty({rows}, fo), loss = at::empty({1}, fo);
  Tensor err = at::zeros({4}, logits.options().dtype(at::kInt));
  check(lt::cross_entropy_fused(dt(logits), logits.data_ptr(), logits.stride(0), labels.data_ptr(),
                                label_kind(labels), rows, cols, lse.data_ptr<float>(),
                                row_loss.data_ptr<float>(), err.data_ptr<int>(), (float)grad_scale,
                                cur_stream()), "cross_entropy_fused");
  check(lt::reduce_all(lt::RED_SUM, lt::DT_F32, row_loss.data_ptr(), rows, 1.0f / (float)rows,
                       loss.data_ptr<float>(), reduce_scratch(), cur_stream()), "reduce_all");
  return {loss, lse, err};
}
// dlogits written into `out` (may alias logits)
void cross_entropy_backward(const Tensor& logits, int64_t cols, const Tensor& labels,
                            const Tensor& lse, double grad_scale, const OptT& gs_dev, Tensor& out) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.scalar_type() == logits.scalar_type());
  c10::cuda::CUDAGuard guard(logits.device());
  check(lt::cross_entropy_backward(dt(logits), logits.data_ptr(), logits.stride(0),
                                   labels.data_ptr(), label_kind(labels), logits.size(0), cols,
                                   lse.data_ptr<float>(), (float)grad_scale,
                                   gs_dev.has_value() ? gs_dev->data_ptr<float>() : nullptr,
                                   out.data_ptr(), out.stride(0), cur_stream()),
        "cross_entropy_backward");
}
Tensor pointwise_loss(int64_t mode, const Tensor& pred, const Tensor& target) {
  need_cuda_contig(pred, "pred"); need_cuda_contig(target, "target");
  TORCH_CHECK(pred.scalar_type() == target.scalar_type() && pred.numel() == target.numel());
  c10::cuda::CUDAGuard guard(pred.device());
  Tensor out = at::empty({1}, pred.options().dtype(at::kFloat));
  check(lt::pointwise_loss((int)mode, dt(pred), pred.data_ptr(), target.data_ptr(), pred.numel(),
                           out.data_ptr<float>(), reduce_scratch(), cur_stream()),
        "pointwise_loss");
  return out;
}
Tensor pointwise_loss_backward(int64_t mode, const Tensor& pred, const Tensor& target,
                               double grad_scale) {
  need_cuda_contig(pred, "pred"); need_cuda_contig(target, "target");
  c10::cuda::CUDAGuard guard(pred.device());
  Tensor out = at::empty_like(pred);
  check(lt::pointwise_loss_backward((int)mode, dt(pred), pred.data_ptr(), target.data_ptr(),
                                    pred.numel(), (float)grad_scale, out.data_ptr(), cur_stream()),
        "pointwise_loss_backward");
  return out;
}

// ------------------------------------------------------------------------------ layernorm / gelu
std::vector<Tensor> layernorm_forward(const Tensor& x, const Tensor& gamma, const Tensor& beta,
                                      double eps) {
  need_cuda_contig(x, "x"); need_cuda_contig(gamma, "gamma"); need_cuda_contig(beta, "beta");
  TORCH_CHECK(gamma.scalar_type() == beta.scalar_type());
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1), rows = x.numel() / cols;
  TORCH_CHECK(gamma.numel() == cols && beta.numel() == cols);
  auto fo = x.options().dtype(at::kFloat);
  Tensor y = at::empty_like(x), mean = at::empty({rows}, fo), rstd = at::empty({rows}, fo);
  check(lt::layernorm_forward(dt(x), x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), dt(gamma),
                              (float)eps, y.data_ptr(), mean.data_ptr<float>(),
                              rstd.data_ptr<float>(), rows, cols, cur_stream()),
        "layernorm_forward");
  return {y, mean, rstd};
}
// Partial rows of the LayerNorm backward: one buffer per device that lives outside the
// caching allocator's reuse (allocated once, grown when a larger one is asked for, never
// while a graph is being captured).  `*is_private` tells the launcher whether it got it.
Tensor ln_scratch(int64_t n, const Tensor& like, int* is_private) {
  static std::mutex mu;
  static std::map<int, Tensor> cache;
  std::lock_guard<std::mutex> lock(mu);
  const int dev = like.get_device();
  auto it = cache.find(dev);
  if (it == cache.end() || it->second.numel() < n) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(cur_stream(), &st);
    if (st != cudaStreamCaptureStatusNone) {
      *is_private = 0;
      return scratch_floats(n, like);
    }
    if (it != cache.end()) cache.erase(it);
    it = cache.emplace(dev, at::empty({n}, like.options().dtype(at::kFloat))).first;
  }
  *is_private = 1;
  return it->second;
}

// returns dx; dgamma / dbeta are written (or accumulated) into the given buffers
Tensor layernorm_backward(const Tensor& x, const Tensor& dy, const Tensor& gamma,
                          const Tensor& mean, const Tensor& rstd, const OptT& dx_add,
                          Tensor& dgamma, Tensor& dbeta, bool accumulate) {
  need_cuda_contig(x, "x"); need_cuda_contig(dy, "dy");
  TORCH_CHECK(dgamma.scalar_type() == dbeta.scalar_type());
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1), rows = x.numel() / cols;
  Tensor dx = at::empty_like(x);
  int priv = 0;
  Tensor scratch = ln_scratch(lt::layernorm_backward_scratch_floats(rows, cols), x, &priv);
  check(lt::layernorm_backward(dt(x), x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), dt(gamma),
                               mean.data_ptr<float>(), rstd.data_ptr<float>(), optptr(dx_add),
                               dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), dt(dgamma),
                               accumulate, scratch.data_ptr<float>(), rows, cols, cur_stream(),
                               nullptr, 0, nullptr, priv),
        "layernorm_backward");
  return dx;
}
// The same, and the column sums of dx go to `dxsum` (dtype of dgamma) when the fused kernels
// can produce them: returns (dx, done).
std::tuple<Tensor, bool> layernorm_backward_dxsum(const Tensor& x, const Tensor& dy,
                                                  const Tensor& gamma, const Tensor& mean,
                                                  const Tensor& rstd, const OptT& dx_add,
                                                  Tensor& dgamma, Tensor& dbeta, bool accumulate,
                                                  Tensor& dxsum, bool dxsum_accumulate) {
  need_cuda_contig(x, "x"); need_cuda_contig(dy, "dy");
  TORCH_CHECK(dgamma.scalar_type() == dbeta.scalar_type() && dxsum.scalar_type() == dgamma.scalar_type());
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1), rows = x.numel() / cols;
  TORCH_CHECK(dxsum.numel() == cols && dxsum.is_contiguous());
  Tensor dx = at::empty_like(x);
  int priv = 0;
  Tensor scratch = ln_scratch(lt::layernorm_backward_scratch_floats(rows, cols), x, &priv);
  int done = 0;
  check(lt::layernorm_backward(dt(x), x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), dt(gamma),
                               mean.data_ptr<float>(), rstd.data_ptr<float>(), optptr(dx_add),
                               dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), dt(dgamma),
                               accumulate, scratch.data_ptr<float>(), rows, cols, cur_stream(),
                               dxsum.data_ptr(), dxsum_accumulate ? 1 : 0, &done, priv),
        "layernorm_backward");
  return {dx, done != 0};
}
Tensor gelu_bias_forward(const Tensor& x, const OptT& bias) {
  need_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1), rows = x.numel() / cols;
  Tensor out = at::empty_like(x);
  check(lt::gelu_bias_forward(dt(x), x.data_ptr(), optptr(bias),
                              bias.has_value() ? dt(*bias) : dt(x), out.data_ptr(), rows, cols,
                              cur_stream()), "gelu_bias_forward");
  return out;
}
Tensor gelu_bias_backward(const Tensor& x, const OptT& bias, const Tensor& dy) {
  need_cuda_contig(x, "x"); need_cuda_contig(dy, "dy");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1), rows = x.numel() / cols;
  Tensor out = at::empty_like(x);
  check(lt::gelu_bias_backward(dt(x), x.data_ptr(), optptr(bias),
                               bias.has_value() ? dt(*bias) : dt(x), dy.data_ptr(),
                               out.data_ptr(), rows, cols, cur_stream()), "gelu_bias_backward");
  return out;
}

// ------------------------------------------------------------------------------ embedding
std::vector<Tensor> embedding_forward(const Tensor& table, const Tensor& ids, const OptT& pos_table,
                                      int64_t seq_len) {
  need_cuda_contig(table, "table"); need_cuda_contig(ids, "ids");
  c10::cuda::CUDAGuard guard(table.device());
  const int64_t n = ids.numel(), dim = table.size(1), vocab = table.size(0);
  Tensor out = at::empty({n, dim}, table.options());
  Tensor err = at::zeros({4}, table.options().dtype(at::kInt));
  check(lt::embedding_forward(dt(table), table.data_ptr(), ids.data_ptr(), label_kind(ids),
                              optptr(pos_table), seq_len > 0 ? seq_len : 1, out.data_ptr(), n, dim,
                              vocab, err.data_ptr<int>(), cur_stream()), "embedding_forward");
  return {out, err};
}
void embedding_backward(const Tensor& dy, const Tensor& ids, Tensor& dtable, bool accumulate) {
  need_cuda_contig(dy, "dy"); need_cuda_contig(ids, "ids"); need_cuda_contig(dtable, "dtable");
  c10::cuda::CUDAGuard guard(dy.device());
  const int64_t n = ids.numel(), dim = dtable.size(1), vocab = dtable.size(0);
  Tensor ws = at::empty({(int64_t)lt::embedding_backward_workspace(n, vocab)},
                        dy.options().dtype(at::kByte));
  check(lt::embedding_backward(dt(dy), dy.data_ptr(), ids.data_ptr(), label_kind(ids),
                               dtable.data_ptr(), dt(dtable), accumulate, n, dim, vocab,
                               ws.data_ptr(), cur_stream()), "embedding_backward");
}
void positional_backward(const Tensor& dy, Tensor& dpos, int64_t batch, int64_t seq_len,
                         bool accumulate) {
  need_cuda_contig(dy, "dy"); need_cuda_contig(dpos, "dpos");
  c10::cuda::CUDAGuard guard(dy.device());
  check(lt::positional_backward(dt(dy), dy.data_ptr(), dpos.data_ptr(), dt(dpos), accumulate,
                                batch, seq_len, dpos.size(0), dpos.size(1), cur_stream()),
        "positional_backward");
}

// ------------------------------------------------------------------------------ conv lowering
Tensor im2col(const Tensor& in, int64_t batch, int64_t C, int64_t H, int64_t W, int64_t k,
              int64_t stride, int64_t pad, int64_t ld) {
  need_cuda_contig(in, "input");
  c10::cuda::CUDAGuard guard(in.device());
  const int64_t oh = (H + 2 * pad - k) / stride + 1, ow = (W + 2 * pad - k) / stride + 1;
  const int64_t patch = C * k * k;
  if (ld < patch) ld = patch;
  // the 16-byte-store kernel writes the padding columns itself; the scalar one leaves them
  const bool vec = ld % (16 / (int64_t)in.element_size()) == 0;
  Tensor cols = (ld == patch || vec) ? at::empty({batch * oh * ow, ld}, in.options())
                                     : at::zeros({batch * oh * ow, ld}, in.options());
  check(lt::im2col(dt(in), in.data_ptr(), cols.data_ptr(), (int)batch, (int)C, (int)H, (int)W,
                   (int)k, (int)stride, (int)pad, ld, cur_stream()), "im2col");
  return cols;
}
Tensor col2im(const Tensor& cols, int64_t batch, int64_t C, int64_t H, int64_t W, int64_t k,
              int64_t stride, int64_t pad) {
  TORCH_CHECK(cols.is_cuda() && cols.dim() == 2 && cols.stride(1) == 1);
  c10::cuda::CUDAGuard guard(cols.device());
  Tensor din = at::empty({batch * C * H * W}, cols.options());
  check(lt::col2im(dt(cols), cols.data_ptr(), din.data_ptr(), (int)batch, (int)C, (int)H, (int)W,
                   (int)k, (int)stride, (int)pad, cols.stride(0), cur_stream()), "col2im");
  return din;
}
Tensor relayout(const Tensor& in, int64_t batch, int64_t C, int64_t hw, bool to_nchw) {
  need_cuda_contig(in, "input");
  c10::cuda::CUDAGuard guard(in.device());
  Tensor out = at::empty_like(in);
  check(lt::nhwc_to_nchw(dt(in), in.data_ptr(), out.data_ptr(), (int)batch, (int)C, (int)hw,
                         to_nchw, cur_stream()), "nhwc_to_nchw");
  return out;
}

// ------------------------------------------------------------------------------ optimizers
// `dyn`: optional fp32[3] on the device holding {lr, bc1, bc2}; when given it replaces the
// by-value scalars inside the kernel, so a captured graph can be replayed for later steps.
void adamw_flat_dyn(Tensor& master, const OptT& shadow, const Tensor& grad, Tensor& m, Tensor& v,
                    const OptT& seg_end, const OptT& seg_wd, double lr, double beta1, double beta2,
                    double eps, double bc1, double bc2, double grad_scale, const OptT& skip_flag,
                    const OptT& dyn) {
  need_cuda_contig(master, "master"); need_cuda_contig(grad, "grad");
  need_cuda_contig(m, "m"); need_cuda_contig(v, "v");
  TORCH_CHECK(master.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat &&
              v.scalar_type() == at::kFloat);
  TORCH_CHECK(grad.numel() == master.numel() && m.numel() == master.numel());
  c10::cuda::CUDAGuard guard(master.device());
  lt::AdamArgs a{(float)lr, (float)beta1, (float)beta2, (float)eps, (float)bc1, (float)bc2,
                 (float)grad_scale,
                 skip_flag.has_value() ? skip_flag->data_ptr<int>() : nullptr};
  if (dyn.has_value()) {
    TORCH_CHECK(dyn->is_cuda() && dyn->scalar_type() == at::kFloat && dyn->numel() >= 3,
                "dyn: fp32 CUDA tensor with {lr, bc1, bc2} expected");
    a.dyn = dyn->data_ptr<float>();
  }
  const int nseg = seg_end.has_value() ? (int)seg_end->numel() : 0;
  check(lt::adamw_flat(master.data_ptr<float>(), optptr(shadow) ? shadow->data_ptr() : nullptr,
                       grad.data_ptr(), dt(grad), m.data_ptr<float>(), v.data_ptr<float>(),
                       master.numel(), nseg ? seg_end->data_ptr<int64_t>() : nullptr,
                       nseg ? seg_wd->data_ptr<float>() : nullptr, nseg, a, cur_stream()),
        "adamw_flat");
}
void adamw_flat(Tensor& master, const OptT& shadow, const Tensor& grad, Tensor& m, Tensor& v,
                const OptT& seg_end, const OptT& seg_wd, double lr, double beta1, double beta2,
                double eps, double bc1, double bc2, double grad_scale, const OptT& skip_flag) {
  adamw_flat_dyn(master, shadow, grad, m, v, seg_end, seg_wd, lr, beta1, beta2, eps, bc1, bc2,
                 grad_scale, skip_flag, c10::nullopt);
}
// Step-dependent scalars of a replayed graph: dyn fp32[>=3] <- {lr, bc1, bc2}, dyn_offset int64[1].
void set_step_scalars(const OptT& dyn, double lr, double bc1, double bc2, const OptT& dyn_offset,
                      int64_t offset) {
  float* d = nullptr;
  uint64_t* o = nullptr;
  if (dyn.has_value()) {
    TORCH_CHECK(dyn->is_cuda() && dyn->scalar_type() == at::kFloat && dyn->numel() >= 3);
    d = dyn->data_ptr<float>();
  }
  if (dyn_offset.has_value()) {
    TORCH_CHECK(dyn_offset->is_cuda() && dyn_offset->scalar_type() == at::kLong);
    o = reinterpret_cast<uint64_t*>(dyn_offset->data_ptr<int64_t>());
  }
  if (!d && !o) return;
  c10::cuda::CUDAGuard guard(dyn.has_value() ? dyn->device() : dyn_offset->device());
  check(lt::set_step_scalars(d, (float)lr, (float)bc1, (float)bc2, o, (uint64_t)offset,
                             cur_stream()), "set_step_scalars");
}
void sgd_flat_dyn(Tensor& master, const OptT& shadow, const Tensor& grad, const OptT& vel,
                  double lr, double momentum, bool nesterov, double grad_scale, const OptT& dyn) {
  need_cuda_contig(master, "master"); need_cuda_contig(grad, "grad");
  c10::cuda::CUDAGuard guard(master.device());
  const float* dyn_lr = nullptr;
  if (dyn.has_value()) {
    TORCH_CHECK(dyn->is_cuda() && dyn->scalar_type() == at::kFloat && dyn->numel() >= 1);
    dyn_lr = dyn->data_ptr<float>();
  }
  check(lt::sgd_flat(master.data_ptr<float>(), shadow.has_value() ? shadow->data_ptr() : nullptr,
                     grad.data_ptr(), dt(grad), vel.has_value() ? vel->data_ptr<float>() : nullptr,
                     master.numel(), (float)lr, (float)momentum, nesterov, (float)grad_scale,
                     cur_stream(), dyn_lr), "sgd_flat");
}
void sgd_flat(Tensor& master, const OptT& shadow, const Tensor& grad, const OptT& vel, double lr,
              double momentum, bool nesterov, double grad_scale) {
  sgd_flat_dyn(master, shadow, grad, vel, lr, momentum, nesterov, grad_scale, c10::nullopt);
}

// ------------------------------------------------------------------------------ attention
// q, k, v: bf16 views [B, S, H, D] (any strides with stride(-1)==1). Returns (o [B,S,H,D], lse [B,H,S]).
std::vector<Tensor> flash_forward(const Tensor& q, const Tensor& k, const Tensor& v, bool causal,
                                  double scale) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 4 && q.scalar_type() == at::kBFloat16);
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1);
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3);
  Tensor o = at::empty({B, S, H, D}, q.options());
  Tensor lse = at::empty({B, H, S}, q.options().dtype(at::kFloat));
  lt::AttnArgs a;
  a.B = (int)B; a.H = (int)H; a.S = (int)S; a.D = (int)D;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr();
  a.lse = lse.data_ptr<float>();
  a.q_sb = q.stride(0); a.q_ss = q.stride(1); a.q_sh = q.stride(2);
  a.k_sb = k.stride(0); a.k_ss = k.stride(1); a.k_sh = k.stride(2);
  a.v_sb = v.stride(0); a.v_ss = v.stride(1); a.v_sh = v.stride(2);
  a.o_sb = o.stride(0); a.o_ss = o.stride(1); a.o_sh = o.stride(2);
  a.causal = causal; a.scale = (float)scale;
  check(lt::flash_attention_forward(a, cur_stream()), "flash_attention_forward");
  return {o, lse};
}
// returns (dq, dk, dv) each [B, S, H, D] contiguous
std::vector<Tensor> flash_backward(const Tensor& q, const Tensor& k, const Tensor& v,
                                   const Tensor& o, const Tensor& lse, const Tensor& d_o,
                                   bool causal, double scale, const OptT& dqkv_out) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 4 && d_o.stride(3) == 1 && o.stride(3) == 1);
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3);
  Tensor dq, dk, dv;
  if (dqkv_out.has_value()) {
    // packed [B, S, 3, H, D] gradient buffer laid out like a fused qkv activation
    Tensor g = *dqkv_out;
    dq = g.select(2, 0); dk = g.select(2, 1); dv = g.select(2, 2);
  } else {
    dq = at::empty({B, S, H, D}, q.options());
    dk = at::empty({B, S, H, D}, q.options());
    dv = at::empty({B, S, H, D}, q.options());
  }
  Tensor delta = at::empty({B, H, S}, q.options().dtype(at::kFloat));
  lt::AttnArgs a;
  a.B = (int)B; a.H = (int)H; a.S = (int)S; a.D = (int)D;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = (void*)o.data_ptr();
  a.lse = (float*)lse.data_ptr<float>();
  a.q_sb = q.stride(0); a.q_ss = q.stride(1); a.q_sh = q.stride(2);
  a.k_sb = k.stride(0); a.k_ss = k.stride(1); a.k_sh = k.stride(2);
  a.v_sb = v.stride(0); a.v_ss = v.stride(1); a.v_sh = v.stride(2);
  a.o_sb = o.stride(0); a.o_ss = o.stride(1); a.o_sh = o.stride(2);
  a.causal = causal; a.scale = (float)scale;
  lt::AttnBwdArgs b;
  b.d_o = d_o.data_ptr(); b.do_sb = d_o.stride(0); b.do_ss = d_o.stride(1); b.do_sh = d_o.stride(2);
  b.dq = dq.data_ptr(); b.dk = dk.data_ptr(); b.dv = dv.data_ptr();
  b.dq_sb = dq.stride(0); b.dq_ss = dq.stride(1); b.dq_sh = dq.stride(2);
  b.dk_sb = dk.stride(0); b.dk_ss = dk.stride(1); b.dk_sh = dk.stride(2);
  b.dv_sb = dv.stride(0); b.dv_ss = dv.stride(1); b.dv_sh = dv.stride(2);
  b.delta = delta.data_ptr<float>();
  // scratch for the dS tiles (dQ = dS K as a GEMM).  Measured: worth it at head dim 128 (0.456
  // vs 0.526 ms at B 4, S 2048, H 16), a wash at head dim 64 where writing and re-reading dS costs
  // what the third kernel's recomputation costs.  LT_FLASH_DQ_GEMM=0 / 1 forces it off / on.
  Tensor ds;
  static const int dq_gemm = [] { const char* e = getenv("LT_FLASH_DQ_GEMM"); return e ? (e[0] == '0' ? 0 : 2) : 1; }();
  if ((dq_gemm == 2 || (dq_gemm == 1 && D == 128)) && S % 128 == 0) {
    ds = at::empty({B, H, S, S}, q.options());
    b.ds_scratch = ds.data_ptr();
  }
  check(lt::flash_attention_backward(a, b, cur_stream()), "flash_attention_backward");
  return {dq, dk, dv};
}
int64_t attention_device_error() { return lt::attention_last_device_error(); }

// ------------------------------------------------------------------------------ comm kernels
// Pointer tables are int64 CUDA tensors holding peer-mapped device addresses.
void allreduce_adamw(const Tensor& grad_ptrs, const Tensor& signal_ptrs, int64_t rank,
                     int64_t world, int64_t elem_offset, int64_t n, Tensor& master,
                     const OptT& shadow_ptrs, const OptT& m, const OptT& v, const OptT& seg_end,
                     const OptT& seg_wd, double lr, double beta1, double beta2, double eps,
                     double bc1, double bc2, double grad_scale, int64_t epoch, int64_t mode,
                     int64_t max_blocks, Tensor& status, int64_t state_base, int64_t opt_kind,
                     double momentum, bool nesterov, int64_t grad_mc, int64_t shadow_mc,
                     const OptT& skip_flag, const OptT& dyn) {
  c10::cuda::CUDAGuard guard(master.device());
  lt::CommAdamArgs a;
  a.grad_ptrs = (const uint64_t*)grad_ptrs.data_ptr<int64_t>();
  a.signal_ptrs = (const uint64_t*)signal_ptrs.data_ptr<int64_t>();
  a.shadow_ptrs = shadow_ptrs.has_value() ? (const uint64_t*)shadow_ptrs->data_ptr<int64_t>()
                                          : nullptr;
  a.grad_mc = reinterpret_cast<const void*>(grad_mc);
  a.shadow_mc = reinterpret_cast<void*>(shadow_mc);
  a.rank = (int)rank; a.world = (int)world;
  a.elem_offset = elem_offset; a.n = n;
  a.master = master.data_ptr<float>();
  a.m = m.has_value() ? m->data_ptr<float>() : nullptr;
  a.v = v.has_value() ? v->data_ptr<float>() : nullptr;
  a.state_base = state_base;
  a.opt_kind = (int)opt_kind; a.momentum = (float)momentum; a.nesterov = nesterov ? 1 : 0;
  const int nseg = seg_end.has_value() ? (int)seg_end->numel() : 0;
  a.seg_end = nseg ? seg_end->data_ptr<int64_t>() : nullptr;
  a.seg_wd = nseg ? seg_wd->data_ptr<float>() : nullptr;
  a.nseg = nseg;
  a.adam = lt::AdamArgs{(float)lr, (float)beta1, (float)beta2, (float)eps, (float)bc1, (float)bc2,
                        (float)grad_scale,
                        skip_flag.has_value() ? skip_flag->data_ptr<int>() : nullptr,
                        dyn.has_value() ? dyn->data_ptr<float>() : nullptr};
  a.epoch = (uint32_t)epoch; a.mode = (int)mode; a.max_blocks = (int)max_blocks;
  a.status = status.data_ptr<int>();
  check(lt::allreduce_adamw(a, cur_stream()), "allreduce_adamw");
}
void peer_broadcast(const Tensor& buf_ptrs, const Tensor& signal_ptrs, int64_t rank, int64_t world,
                    int64_t root, int64_t byte_offset, int64_t nbytes, int64_t epoch,
                    Tensor& status) {
  c10::cuda::CUDAGuard guard(status.device());
  check(lt::peer_broadcast((const uint64_t*)buf_ptrs.data_ptr<int64_t>(),
                           (const uint64_t*)signal_ptrs.data_ptr<int64_t>(), (int)rank, (int)world,
                           (int)root, byte_offset, nbytes, (uint32_t)epoch, status.data_ptr<int>(),
                           cur_stream()), "peer_broadcast");
}
void peer_allreduce(const Tensor& buf_ptrs, const Tensor& signal_ptrs, int64_t rank, int64_t world,
                    int64_t elem_offset, int64_t n, int64_t dtype_code, double scale, int64_t epoch,
                    Tensor& status) {
  c10::cuda::CUDAGuard guard(status.device());
  check(lt::peer_allreduce((const uint64_t*)buf_ptrs.data_ptr<int64_t>(),
                           (const uint64_t*)signal_ptrs.data_ptr<int64_t>(), (int)rank, (int)world,
                           elem_offset, n, (int)dtype_code, (float)scale, (uint32_t)epoch,
                           status.data_ptr<int>(), cur_stream()), "peer_allreduce");
}
void wait_flag_bounded(const Tensor& flag, int64_t expected, int64_t budget_cycles, Tensor& status) {
  c10::cuda::CUDAGuard guard(status.device());
  check(lt::wait_flag_bounded((const uint32_t*)flag.data_ptr<int>(), (uint32_t)expected,
                              budget_cycles, status.data_ptr<int>(), cur_stream()),
        "wait_flag_bounded");
}

std::vector<int64_t> launch_counts() {
  return {(int64_t)lt::gemm_launch_count(), (int64_t)lt::ops_launch_count(),
          (int64_t)lt::attention_launch_count(), (int64_t)lt::comm_launch_count()};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm);
  m.def("gemm_next_overlaps_prev", &gemm_next_overlaps_prev);
  m.def("gemm_gather", &gemm_gather);
  m.def("gemm_device_error", &gemm_device_error);
  m.def("binary", &binary);
  m.def("scalar", &scalar);
  m.def("unary", &unary);
  m.def("unary_backward", &unary_backward);
  m.def("add_broadcast", &add_broadcast);
  m.def("affine_cols", &affine_cols);
  m.def("column_sum", &column_sum);
  m.def("cast", &cast);
  m.def("cast_into", &cast_into);
  m.def("transpose2d", &transpose2d);
  m.def("fill_random", &fill_random);
  m.def("dropout", &dropout);
  m.def("dropout_dyn", &dropout_dyn);
  m.def("set_pdl", [](int64_t v) { lt::set_pdl_override((int)v); });
  m.def("split_bf16", &split_bf16);
  m.def("reduce", &reduce);
  m.def("dot", &dot);
  m.def("check_finite_scale", &check_finite_scale);
  m.def("softmax", &softmax);
  m.def("softmax_scores", &softmax_scores);
  m.def("softmax_scores_backward", &softmax_scores_backward);
  m.def("cross_entropy_forward", &cross_entropy_forward);
  m.def("cross_entropy_backward", &cross_entropy_backward);
  m.def("cross_entropy_fused", &cross_entropy_fused);
  m.def("pointwise_loss", &pointwise_loss);
  m.def("pointwise_loss_backward", &pointwise_loss_backward);
  m.def("layernorm_forward", &layernorm_forward);
  m.def("layernorm_backward", &layernorm_backward);
  m.def("layernorm_backward_dxsum", &layernorm_backward_dxsum);
  m.def("gelu_bias_forward", &gelu_bias_forward);
  m.def("gelu_bias_backward", &gelu_bias_backward);
  m.def("embedding_forward", &embedding_forward);
  m.def("embedding_backward", &embedding_backward);
  m.def("positional_backward", &positional_backward);
  m.def("im2col", &im2col);
  m.def("col2im", &col2im);
  m.def("relayout", &relayout);
  m.def("adamw_flat", &adamw_flat);
  m.def("sgd_flat", &sgd_flat);
  m.def("adamw_flat_dyn", &adamw_flat_dyn);
  m.def("sgd_flat_dyn", &sgd_flat_dyn);
  m.def("set_step_scalars", &set_step_scalars);
  m.def("flash_forward", &flash_forward);
  m.def("flash_backward", &flash_backward);
  m.def("attention_device_error", &attention_device_error);
  m.def("allreduce_adamw", &allreduce_adamw);
  m.def("peer_broadcast", &peer_broadcast);
  m.def("peer_allreduce", &peer_allreduce);
  m.def("wait_flag_bounded", &wait_flag_bounded);
  m.def("launch_counts", &launch_counts);
}
