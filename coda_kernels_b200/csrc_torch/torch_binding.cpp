// Compiled dispatch layer: the device operators of the four fused-linear functions registered with PyTorch from C++
// (TORCH_LIBRARY, namespace coda_b200n), each a thin call into the C ABI of libcoda_b200.so.  It does what the ctypes
// table in _lib.py does, without the per-launch Python work: tensors in, pointers / strides / extents / the current
// CUDA stream out.  The `*_out` ops allocate nothing: they mutate the outputs the Python wrapper passes in and return
// nothing, the convention of the reference's `_kernel_op` (coda/core/gemm/gemm_interface.py:78-100).  Below them sit
// whole-operator entry points (`swiglu_fwd`, `swiglu_bwd`, ...): one dispatcher call per direction of an autograd node,
// which allocates the outputs with the caching allocator and issues that direction's launches back to back, so a short
// step (a head-sharded rank, a small batch) is not bound by the interpreter between launches.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <tuple>

#include "../../include/coda_b200.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<Tensor>;

inline void check(int rc, const char* what) {
  TORCH_CHECK(rc == 0, what, " failed (code ", rc, "): ", coda_b200_last_error());
}
inline void* stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }
inline int* status_ptr(const Tensor& status) { return status.data_ptr<int>(); }
inline const void* ptr_or_null(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }

void gemm_out(const Tensor& A, const Tensor& B, Tensor& out, const OptTensor& alpha, const OptTensor& C, const Tensor& status) {
  const c10::cuda::CUDAGuard guard(A.device());
  const int M = static_cast<int>(A.size(0)), N = static_cast<int>(B.size(1)), K = static_cast<int>(A.size(1));
  const float* alpha_ptr = alpha.has_value() ? alpha->data_ptr<float>() : nullptr;
  if (!C.has_value()) {
    // A plain product may be balanced by stream-K; its fp32 workspace (the one allocation of this layer's `*_out` ops)
    // comes from the caching allocator and is only asked for when the library would use it.
    const int64_t ws_bytes = coda_b200_gemm_workspace_bytes(M, N, K);
    Tensor ws;
    if (ws_bytes > 0) ws = at::empty({ws_bytes / 4}, A.options().dtype(at::kFloat));
    check(coda_b200_gemm_ws(A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), out.data_ptr(), out.stride(0),
                            out.scalar_type() == at::kFloat, M, N, K, alpha_ptr, ws_bytes > 0 ? ws.data_ptr() : nullptr, ws_bytes,
                            status_ptr(status), stream_of(A)),
          "gemm");
    return;
  }
  check(coda_b200_gemm_add(A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), C->data_ptr(), C->stride(0),
                           C->scalar_type() == at::kFloat, out.data_ptr(), out.stride(0), out.scalar_type() == at::kFloat, M, N, K,
                           alpha_ptr, status_ptr(status), stream_of(A)),
        "gemm");
}

void gemm_sigmoid_out(const Tensor& A, const Tensor& B, Tensor& out, const Tensor& status) {
  const c10::cuda::CUDAGuard guard(A.device());
  check(coda_b200_gemm_sigmoid(A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), out.data_ptr(),
                               out.stride(0), out.scalar_type() == at::kFloat, static_cast<int>(A.size(0)), static_cast<int>(B.size(1)),
                               static_cast<int>(A.size(1)), status_ptr(status), stream_of(A)),
        "gemm_sigmoid");
}

void gemm_swiglu_out(const Tensor& A, const Tensor& B, Tensor& preact, Tensor& postact, const Tensor& status) {
  const c10::cuda::CUDAGuard guard(A.device());
  check(coda_b200_gemm_swiglu(A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), preact.data_ptr(),
                              preact.stride(0), postact.data_ptr(), postact.stride(0), static_cast<int>(A.size(0)),
                              static_cast<int>(B.size(1)), static_cast<int>(A.size(1)), status_ptr(status), stream_of(A)),
        "gemm_swiglu");
}

void gemm_lse_out(const Tensor& A, const Tensor& B, const OptTensor& probs, Tensor& part_max, Tensor& part_sum, const Tensor& target,
                  Tensor& target_logit, const Tensor& status) {
  const c10::cuda::CUDAGuard guard(A.device());
  check(coda_b200_gemm_lse(A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1),
                           probs.has_value() ? probs->data_ptr() : nullptr, probs.has_value() ? probs->stride(0) : 0,
                           part_max.data_ptr<float>(), part_sum.data_ptr<float>(), target.data_ptr<int32_t>(),
                           target_logit.data_ptr<float>(), static_cast<int>(A.size(0)), static_cast<int>(B.size(1)),
                           static_cast<int>(A.size(1)), status_ptr(status), stream_of(A)),
        "gemm_lse");
}

void lse_finalize_out(const Tensor& part_max, const Tensor& part_sum, const Tensor& target, const Tensor& target_logit,
                      int64_t ignore_index, Tensor& lse, Tensor& losses) {
  const c10::cuda::CUDAGuard guard(part_max.device());
  check(coda_b200_lse_finalize(part_max.data_ptr<float>(), part_sum.data_ptr<float>(), static_cast<int>(part_max.size(1)),
                               target.data_ptr<int32_t>(), target_logit.data_ptr<float>(), static_cast<int>(ignore_index),
                               lse.data_ptr<float>(), losses.data_ptr<float>(), static_cast<int>(part_max.size(0)), stream_of(part_max)),
        "lse_finalize");
}

void ce_grad_fixup_(Tensor& probs, const Tensor& part_max, const Tensor& lse, const Tensor& target, int64_t ignore_index) {
  const c10::cuda::CUDAGuard guard(probs.device());
  check(coda_b200_ce_grad_fixup(probs.data_ptr(), probs.stride(0), part_max.data_ptr<float>(), static_cast<int>(part_max.size(1)),
                                lse.data_ptr<float>(), target.data_ptr<int32_t>(), static_cast<int>(ignore_index),
                                static_cast<int>(probs.size(0)), static_cast<int>(probs.size(1)), stream_of(probs)),
        "ce_grad_fixup");
}

void gemm_qknorm_rope_out(const Tensor& A, const Tensor& B, Tensor& qk, Tensor& preact, const OptTensor& v, Tensor& mean_sq,
                          const Tensor& gamma, const Tensor& positions, const Tensor& frequencies, int64_t head_dim, int64_t hq,
                          int64_t hk, double eps, const Tensor& status) {
  const c10::cuda::CUDAGuard guard(A.device());
  check(coda_b200_gemm_qknorm_rope(A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), qk.data_ptr(),
                                   qk.stride(0), preact.data_ptr(), preact.stride(0), v.has_value() ? v->data_ptr() : nullptr,
                                   v.has_value() ? v->stride(0) : 0, mean_sq.data_ptr<float>(), gamma.data_ptr(), positions.data_ptr(),
                                   positions.scalar_type() == at::kFloat, frequencies.data_ptr<float>(), static_cast<int>(head_dim),
                                   static_cast<int>(hq), static_cast<int>(hk), static_cast<float>(eps), static_cast<int>(A.size(0)),
                                   static_cast<int>(B.size(1)), static_cast<int>(A.size(1)), status_ptr(status), stream_of(A)),
        "gemm_qknorm_rope");
}

void dswiglu_out(const Tensor& preact, const Tensor& dout, Tensor& grad_pre) {
  const c10::cuda::CUDAGuard guard(dout.device());
  check(coda_b200_dswiglu(preact.data_ptr(), preact.stride(0), dout.data_ptr(), dout.stride(0), grad_pre.data_ptr(), grad_pre.stride(0),
                          static_cast<int>(dout.size(0)), static_cast<int>(dout.size(1)), stream_of(dout)),
        "dswiglu");
}

void dsigmoid_out(const Tensor& out, const Tensor& dout, Tensor& grad_pre) {
  const c10::cuda::CUDAGuard guard(dout.device());
  check(coda_b200_dsigmoid(out.data_ptr(), out.stride(0), out.scalar_type() == at::kFloat, dout.data_ptr(), dout.stride(0),
                           grad_pre.data_ptr(), grad_pre.stride(0), static_cast<int>(dout.size(0)), static_cast<int>(dout.size(1)),
                           stream_of(dout)),
        "dsigmoid");
}

void qknorm_rope_bwd_out(const Tensor& dq, const Tensor& dk, const OptTensor& dv, const Tensor& preact, const Tensor& mean_sq,
                         const Tensor& gamma, const Tensor& positions, const Tensor& frequencies, int64_t head_dim, int64_t hq, int64_t hk,
                         double eps, Tensor& grad, Tensor& dgamma, Tensor& scratch) {
  const c10::cuda::CUDAGuard guard(preact.device());
  check(coda_b200_qknorm_rope_bwd(dq.data_ptr(), dq.stride(0), dk.data_ptr(), dk.stride(0), dv.has_value() ? dv->data_ptr() : nullptr,
                                  dv.has_value() ? dv->stride(0) : 0, dv.has_value() ? static_cast<int>(dv->size(1)) : 0, preact.data_ptr(),
                                  preact.stride(0), mean_sq.data_ptr<float>(), gamma.data_ptr(), positions.data_ptr(),
                                  positions.scalar_type() == at::kFloat, frequencies.data_ptr<float>(), static_cast<int>(head_dim),
                                  static_cast<int>(hq), static_cast<int>(hk), static_cast<float>(eps), grad.data_ptr(), grad.stride(0),
                                  dgamma.data_ptr<float>(), scratch.data_ptr(), static_cast<int64_t>(scratch.numel() * scratch.element_size()),
                                  static_cast<int>(preact.size(0)), stream_of(preact)),
        "qknorm_rope_bwd");
}

// ---------------------------------------------------------------------------------------- whole-operator entry points

using OptPair = std::tuple<OptTensor, OptTensor>;

inline void require_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2, name, " must be a 2-D bfloat16 CUDA tensor");
}
inline Tensor new_matrix(const Tensor& like, int64_t rows, int64_t cols, at::ScalarType dtype) {
  return at::empty({rows, cols}, like.options().dtype(dtype));
}
// Contiguous and 16-byte aligned: gamma and the rotary frequencies are read 16 bytes at a time.
inline Tensor aligned16(const Tensor& t) {
  Tensor c = t.contiguous();
  return (reinterpret_cast<uintptr_t>(c.data_ptr()) & 15u) == 0 ? c : c.clone();
}

// dx = alpha * grad_pre @ weight, dweight = alpha * grad_pre^T @ x (either may be skipped).  The [N, K] weight and
// both operands of the weight gradient are consumed as MN-major views: no transposed copy.
OptPair linear_backward(const Tensor& grad_pre, const Tensor& x, const Tensor& weight, bool need_dx, bool need_dw, const OptTensor& alpha,
                        const Tensor& status) {
  require_bf16(grad_pre, "grad_pre");
  require_bf16(x, "x");
  require_bf16(weight, "weight");
  OptTensor dx, dw;
  if (need_dx) {
    Tensor out = new_matrix(x, grad_pre.size(0), weight.size(1), at::kBFloat16);
    gemm_out(grad_pre, weight, out, alpha, c10::nullopt, status);
    dx = out;
  }
  if (need_dw) {
    Tensor out = new_matrix(x, grad_pre.size(1), x.size(1), at::kBFloat16);
    gemm_out(grad_pre.t(), x, out, alpha, c10::nullopt, status);
    dw = out;
  }
  return {dx, dw};
}

std::tuple<Tensor, Tensor> swiglu_fwd(const Tensor& x, const Tensor& weight, const Tensor& status) {
  require_bf16(x, "x");
  require_bf16(weight, "weight");
  TORCH_CHECK(weight.size(0) % 2 == 0, "gemm_swiglu: N must be even");
  Tensor preact = new_matrix(x, x.size(0), weight.size(0), at::kBFloat16);
  Tensor postact = new_matrix(x, x.size(0), weight.size(0) / 2, at::kBFloat16);
  gemm_swiglu_out(x, weight.t(), preact, postact, status);
  return {preact, postact};
}

OptPair swiglu_bwd(const Tensor& preact, const Tensor& dout, const Tensor& x, const Tensor& weight, bool need_dx, bool need_dw,
                   const Tensor& status) {
  require_bf16(preact, "preact");
  require_bf16(dout, "dout");
  TORCH_CHECK(preact.stride(1) == 1 && dout.stride(1) == 1 && preact.size(1) == 2 * dout.size(1) && preact.size(0) == dout.size(0),
              "dswiglu: bad shapes");
  Tensor grad_pre = at::empty_like(preact);
  dswiglu_out(preact, dout, grad_pre);
  return linear_backward(grad_pre, x, weight, need_dx, need_dw, c10::nullopt, status);
}

Tensor sigmoid_fwd(const Tensor& x, const Tensor& weight, bool out_fp32, const Tensor& status) {
  require_bf16(x, "x");
  require_bf16(weight, "weight");
  Tensor out = new_matrix(x, x.size(0), weight.size(0), out_fp32 ? at::kFloat : at::kBFloat16);
  gemm_sigmoid_out(x, weight.t(), out, status);
  return out;
}

OptPair sigmoid_bwd(const Tensor& out, const Tensor& dout, const Tensor& x, const Tensor& weight, bool need_dx, bool need_dw,
                    const Tensor& status) {
  require_bf16(dout, "dout");
  TORCH_CHECK(out.sizes() == dout.sizes() && (out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat), "dsigmoid: bad out");
  Tensor grad_pre = at::empty_like(dout);
  dsigmoid_out(out, dout, grad_pre);
  return linear_backward(grad_pre, x, weight, need_dx, need_dw, c10::nullopt, status);
}

// (loss, 1 / count or nothing, gradient of the summed row losses w.r.t. the logits or nothing).  With `store_grad` the
// [M, V] buffer first receives unnormalised probabilities from the GEMM epilogue and is then rewritten in place to
// softmax - onehot; without it nothing of that size exists.
std::tuple<Tensor, OptTensor, OptTensor> cross_entropy_fwd(const Tensor& x, const Tensor& weight, const Tensor& target, int64_t ignore_index,
                                                           bool mean, bool store_grad, const Tensor& status) {
  require_bf16(x, "x");
  require_bf16(weight, "weight");
  TORCH_CHECK(target.is_cuda() && target.scalar_type() == at::kInt && target.is_contiguous() && target.numel() == x.size(0),
              "target must be a contiguous int32 CUDA tensor with one label per row");
  const int64_t M = x.size(0), V = weight.size(0);
  const int64_t tiles = coda_b200_lse_tiles(static_cast<int>(V));
  const auto f32 = x.options().dtype(at::kFloat);
  OptTensor probs;
  if (store_grad) probs = new_matrix(x, M, V, at::kBFloat16);
  Tensor part_max = at::empty({M, tiles}, f32), part_sum = at::empty({M, tiles}, f32);
  Tensor target_logit = at::zeros({M}, f32), lse = at::empty({M}, f32), losses = at::empty({M}, f32);
  gemm_lse_out(x, weight.t(), probs, part_max, part_sum, target, target_logit, status);
  lse_finalize_out(part_max, part_sum, target, target_logit, ignore_index, lse, losses);
  if (store_grad) ce_grad_fixup_(*probs, part_max, lse, target, ignore_index);
  Tensor loss = losses.sum();
  OptTensor inv_count;
  if (mean) {  // ignored rows already carry an exact zero; the divisor stays on the device
    inv_count = target.ne(ignore_index).sum().to(at::kFloat).reciprocal();
    loss = loss * *inv_count;
  }
  return {loss, inv_count, probs};
}

OptPair cross_entropy_bwd(const Tensor& dloss, const OptTensor& inv_count, const Tensor& dlogits, const Tensor& x, const Tensor& weight,
                          bool need_dx, bool need_dw, const Tensor& status) {
  const Tensor alpha = (inv_count.has_value() ? dloss * *inv_count : dloss).reshape({1}).to(at::kFloat);
  return linear_backward(dlogits, x, weight, need_dx, need_dw, alpha, status);
}

std::tuple<Tensor, Tensor, Tensor, Tensor> qknorm_rope_fwd(const Tensor& x, const Tensor& weight, const Tensor& gamma, const Tensor& positions,
                                                          const Tensor& frequencies, int64_t head_dim, int64_t hq, int64_t hk, double eps,
                                                          const Tensor& status) {
  require_bf16(x, "x");
  require_bf16(weight, "weight");
  TORCH_CHECK(gamma.is_cuda() && gamma.scalar_type() == at::kBFloat16 && gamma.numel() == 2 * head_dim, "gamma must hold [gamma_q | gamma_k]");
  TORCH_CHECK(positions.scalar_type() == at::kInt || positions.scalar_type() == at::kFloat, "positions must be int32 or float32");
  TORCH_CHECK(frequencies.scalar_type() == at::kFloat, "frequencies must be float32");
  const int64_t M = x.size(0), N = weight.size(0), heads = hq + hk, size_qk = heads * head_dim;
  TORCH_CHECK(frequencies.numel() == size_qk, "frequencies must have (hq + hk) * head_dim entries");
  TORCH_CHECK(positions.numel() == M, "positions must have one entry per row");
  TORCH_CHECK(N >= size_qk, "weight has fewer rows than the q and k heads need");
  Tensor qk = new_matrix(x, M, size_qk, at::kBFloat16), preact = new_matrix(x, M, size_qk, at::kBFloat16);
  Tensor mean_sq = new_matrix(x, M, heads, at::kFloat), v = new_matrix(x, M, N - size_qk, at::kBFloat16);
  OptTensor v_arg;
  if (N > size_qk) v_arg = v;
  gemm_qknorm_rope_out(x, weight.t(), qk, preact, v_arg, mean_sq, aligned16(gamma), positions.contiguous(), aligned16(frequencies), head_dim,
                       hq, hk, eps, status);
  return {qk, preact, mean_sq, v};
}

// (dx, dweight, dgamma in gamma's dtype).  [grad_pre | dv] is one buffer, so each GEMM of the backward runs once over
// the whole [q | k | v] weight.
std::tuple<OptTensor, OptTensor, Tensor> qknorm_rope_bwd(const Tensor& dq, const Tensor& dk, const Tensor& dv, const Tensor& x,
                                                         const Tensor& weight, const Tensor& preact, const Tensor& mean_sq, const Tensor& gamma,
                                                         const Tensor& positions, const Tensor& frequencies, int64_t head_dim, int64_t hq,
                                                         int64_t hk, double eps, bool need_dx, bool need_dw, const Tensor& status) {
  require_bf16(dq, "dq");
  require_bf16(dk, "dk");
  require_bf16(preact, "preact");
  const int64_t M = preact.size(0), size_qk = preact.size(1), nv = dv.size(1);
  Tensor grad = new_matrix(x, M, size_qk + nv, at::kBFloat16);
  const auto f32 = x.options().dtype(at::kFloat);
  Tensor dgamma = at::empty({2 * head_dim}, f32);
  const int64_t scratch_bytes = coda_b200_qknorm_rope_bwd_scratch_bytes(static_cast<int>(M), static_cast<int>(head_dim));
  Tensor scratch = at::empty({(scratch_bytes + 3) / 4}, f32);
  OptTensor dv_arg;
  if (nv > 0) {
    require_bf16(dv, "dv");
    dv_arg = dv;
  }
  qknorm_rope_bwd_out(dq, dk, dv_arg, preact, mean_sq, aligned16(gamma), positions.contiguous(), aligned16(frequencies), head_dim, hq, hk,
                      eps, grad, dgamma, scratch);
  auto [dx, dw] = linear_backward(grad, x, weight, need_dx, need_dw, c10::nullopt, status);
  return {dx, dw, dgamma.to(gamma.scalar_type())};
}

}  // namespace

TORCH_LIBRARY(coda_b200n, m) {
  m.def("gemm_out(Tensor A, Tensor B, Tensor(a!) out, Tensor? alpha, Tensor? C, Tensor status) -> ()");
  m.def("gemm_sigmoid_out(Tensor A, Tensor B, Tensor(a!) out, Tensor status) -> ()");
  m.def("gemm_swiglu_out(Tensor A, Tensor B, Tensor(a!) preact, Tensor(b!) postact, Tensor status) -> ()");
  m.def("gemm_lse_out(Tensor A, Tensor B, Tensor(a!)? probs, Tensor(b!) part_max, Tensor(c!) part_sum, Tensor target, "
        "Tensor(d!) target_logit, Tensor status) -> ()");
  m.def("lse_finalize_out(Tensor part_max, Tensor part_sum, Tensor target, Tensor target_logit, int ignore_index, "
        "Tensor(a!) lse, Tensor(b!) losses) -> ()");
  m.def("ce_grad_fixup_(Tensor(a!) probs, Tensor part_max, Tensor lse, Tensor target, int ignore_index) -> ()");
  m.def("gemm_qknorm_rope_out(Tensor A, Tensor B, Tensor(a!) qk, Tensor(b!) preact, Tensor(c!)? v, Tensor(d!) mean_sq, Tensor gamma, "
        "Tensor positions, Tensor frequencies, int head_dim, int num_heads_q, int num_heads_k, float eps, Tensor status) -> ()");
  m.def("dswiglu_out(Tensor preact, Tensor dout, Tensor(a!) grad_pre) -> ()");
  m.def("dsigmoid_out(Tensor out, Tensor dout, Tensor(a!) grad_pre) -> ()");
  m.def("qknorm_rope_bwd_out(Tensor dq, Tensor dk, Tensor? dv, Tensor preact, Tensor mean_sq, Tensor gamma, Tensor positions, "
        "Tensor frequencies, int head_dim, int num_heads_q, int num_heads_k, float eps, Tensor(a!) grad, Tensor(b!) dgamma, "
        "Tensor(c!) scratch) -> ()");

  m.def("linear_backward(Tensor grad_pre, Tensor x, Tensor weight, bool need_dx, bool need_dw, Tensor? alpha, Tensor status) -> "
        "(Tensor?, Tensor?)");
  m.def("swiglu_fwd(Tensor x, Tensor weight, Tensor status) -> (Tensor, Tensor)");
  m.def("swiglu_bwd(Tensor preact, Tensor dout, Tensor x, Tensor weight, bool need_dx, bool need_dw, Tensor status) -> (Tensor?, Tensor?)");
  m.def("sigmoid_fwd(Tensor x, Tensor weight, bool out_fp32, Tensor status) -> Tensor");
  m.def("sigmoid_bwd(Tensor out, Tensor dout, Tensor x, Tensor weight, bool need_dx, bool need_dw, Tensor status) -> (Tensor?, Tensor?)");
  m.def("cross_entropy_fwd(Tensor x, Tensor weight, Tensor target, int ignore_index, bool mean, bool store_grad, Tensor status) -> "
        "(Tensor, Tensor?, Tensor?)");
  m.def("cross_entropy_bwd(Tensor dloss, Tensor? inv_count, Tensor dlogits, Tensor x, Tensor weight, bool need_dx, bool need_dw, "
        "Tensor status) -> (Tensor?, Tensor?)");
  m.def("qknorm_rope_fwd(Tensor x, Tensor weight, Tensor gamma, Tensor positions, Tensor frequencies, int head_dim, int num_heads_q, "
        "int num_heads_k, float eps, Tensor status) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("qknorm_rope_bwd(Tensor dq, Tensor dk, Tensor dv, Tensor x, Tensor weight, Tensor preact, Tensor mean_sq, Tensor gamma, "
        "Tensor positions, Tensor frequencies, int head_dim, int num_heads_q, int num_heads_k, float eps, bool need_dx, bool need_dw, "
        "Tensor status) -> (Tensor?, Tensor?, Tensor)");
}

TORCH_LIBRARY_IMPL(coda_b200n, CUDA, m) {
  m.impl("gemm_out", gemm_out);
  m.impl("gemm_sigmoid_out", gemm_sigmoid_out);
  m.impl("gemm_swiglu_out", gemm_swiglu_out);
  m.impl("gemm_lse_out", gemm_lse_out);
  m.impl("lse_finalize_out", lse_finalize_out);
  m.impl("ce_grad_fixup_", ce_grad_fixup_);
  m.impl("gemm_qknorm_rope_out", gemm_qknorm_rope_out);
  m.impl("dswiglu_out", dswiglu_out);
  m.impl("dsigmoid_out", dsigmoid_out);
  m.impl("qknorm_rope_bwd_out", qknorm_rope_bwd_out);
  m.impl("linear_backward", linear_backward);
  m.impl("swiglu_fwd", swiglu_fwd);
  m.impl("swiglu_bwd", swiglu_bwd);
  m.impl("sigmoid_fwd", sigmoid_fwd);
  m.impl("sigmoid_bwd", sigmoid_bwd);
  m.impl("cross_entropy_fwd", cross_entropy_fwd);
  m.impl("cross_entropy_bwd", cross_entropy_bwd);
  m.impl("qknorm_rope_fwd", qknorm_rope_fwd);
  m.impl("qknorm_rope_bwd", qknorm_rope_bwd);
}
