// Compiled dispatch layer: the device operators of the four fused-linear functions registered with PyTorch from C++
// (TORCH_LIBRARY, namespace coda_b200n), each a thin call into the C ABI of libcoda_b200.so.  It does what the ctypes
// table in _lib.py does, without the per-launch Python work: tensors in, pointers / strides / extents / the current
// CUDA stream out.  Nothing is allocated here; every op mutates the outputs the Python wrapper passes in and returns
// nothing, the convention of the reference's `_kernel_op` (coda/core/gemm/gemm_interface.py:78-100).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

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
  check(coda_b200_gemm_add(A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), ptr_or_null(C),
                           C.has_value() ? C->stride(0) : 0, C.has_value() && C->scalar_type() == at::kFloat, out.data_ptr(),
                           out.stride(0), out.scalar_type() == at::kFloat, static_cast<int>(A.size(0)), static_cast<int>(B.size(1)),
                           static_cast<int>(A.size(1)), alpha.has_value() ? alpha->data_ptr<float>() : nullptr, status_ptr(status),
                           stream_of(A)),
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
}
