// Python bindings of the elementwise training kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>
#include <tuple>

#include "comm.h"
#include "optim.h"

namespace py = pybind11;
using namespace pccl;

namespace {

void check_flat(const at::Tensor& t, const char* name, at::ScalarType dt) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
  TORCH_CHECK(t.scalar_type() == dt, name, " has the wrong dtype");
}

void sq_norm(const at::Tensor& x, at::Tensor& out) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "x must be a contiguous CUDA tensor");
  TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16, "x must be float32 or bfloat16");
  check_flat(out, "out", at::kFloat);
  TORCH_CHECK(out.numel() == 1, "out must hold one float");
  c10::cuda::CUDAGuard guard(x.device());
  PCCL_CUDA(launch_sq_norm(x.data_ptr(), x.scalar_type() == at::kBFloat16, (uint64_t)x.numel(), out.data_ptr<float>(),
                           at::cuda::getCurrentCUDAStream().stream()));
}

void adamw(at::Tensor& master, at::Tensor& m, at::Tensor& v, const at::Tensor& grad, at::Tensor& param, double lr,
           double beta1, double beta2, double eps, double weight_decay, int64_t step, double grad_scale,
           double max_grad_norm, std::optional<at::Tensor> total_sq_norm) {
  check_flat(master, "master", at::kFloat);
  check_flat(m, "exp_avg", at::kFloat);
  check_flat(v, "exp_avg_sq", at::kFloat);
  check_flat(param, "param", at::kBFloat16);
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous(), "grad must be a contiguous CUDA tensor");
  TORCH_CHECK(grad.scalar_type() == at::kFloat || grad.scalar_type() == at::kBFloat16, "grad must be float32 or bfloat16");
  const int64_t n = master.numel();
  TORCH_CHECK(m.numel() == n && v.numel() == n && grad.numel() == n && param.numel() == n, "size mismatch");
  TORCH_CHECK(step >= 1, "step counts from 1");
  AdamWArgs a;
  a.lr = (float)lr;
  a.beta1 = (float)beta1;
  a.beta2 = (float)beta2;
  a.eps = (float)eps;
  a.weight_decay = (float)weight_decay;
  a.bias1 = (float)(1.0 / (1.0 - std::pow(beta1, (double)step)));
  a.bias2 = (float)(1.0 / (1.0 - std::pow(beta2, (double)step)));
  a.grad_scale = (float)grad_scale;
  a.max_grad_norm = (float)max_grad_norm;
  const float* norm = nullptr;
  if (total_sq_norm.has_value()) {
    check_flat(*total_sq_norm, "total_sq_norm", at::kFloat);
    norm = total_sq_norm->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(master.device());
  PCCL_CUDA(launch_adamw(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr(),
                         grad.scalar_type() == at::kBFloat16, param.data_ptr(), (uint64_t)n, a, norm,
                         at::cuda::getCurrentCUDAStream().stream()));
}

void ce_fwd_bwd(at::Tensor& logits, const at::Tensor& targets, at::Tensor& loss_sum, double grad_scale,
                int64_t ignore_index, std::optional<at::Tensor> bad_targets) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kBFloat16,
              "logits must be a 2-D bfloat16 CUDA tensor");
  TORCH_CHECK(logits.stride(1) == 1 && logits.stride(0) % 8 == 0, "logits rows must be contiguous and 16-byte aligned");
  TORCH_CHECK(((uintptr_t)logits.data_ptr()) % 16 == 0, "logits must be 16-byte aligned");
  check_flat(targets, "targets", at::kLong);
  check_flat(loss_sum, "loss_sum", at::kFloat);
  TORCH_CHECK(targets.numel() == logits.size(0), "one target per row");
  int* bad = nullptr;
  if (bad_targets.has_value()) {
    check_flat(*bad_targets, "bad_targets", at::kInt);
    TORCH_CHECK(bad_targets->numel() >= 1, "bad_targets must hold one int32");
    bad = bad_targets->data_ptr<int>();
  }
  c10::cuda::CUDAGuard guard(logits.device());
  PCCL_CUDA(launch_ce_fwd_bwd(logits.data_ptr(), targets.data_ptr<int64_t>(), loss_sum.data_ptr<float>(), logits.size(0),
                              (int)logits.size(1), logits.stride(0), (float)grad_scale, ignore_index, bad,
                              at::cuda::getCurrentCUDAStream().stream()));
}

// Scratch that lives as long as the process: one buffer per device, grown on demand.  The
// column-sum family uses the front of it and the layer-norm backward the rest, so launches of
// the same family must be ordered with each other on the device (the engine issues them on
// one stream); two of them running at once on different streams would share partial sums.
at::Tensor& scratch(int device, int64_t floats) {
  static at::Tensor bufs[64];
  at::Tensor& b = bufs[device & 63];
  if (!b.defined() || b.numel() < floats)
    b = at::zeros({std::max<int64_t>(floats, 1 << 20)}, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, device));
  return b;
}
at::Tensor& counters(int device, int64_t ints) {
  static at::Tensor bufs[64];
  at::Tensor& b = bufs[device & 63];
  if (!b.defined() || b.numel() < ints)
    b = at::zeros({std::max<int64_t>(ints, 4096)}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  return b;
}

void col_sum(const at::Tensor& x, at::Tensor& out) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.is_contiguous(),
              "x must be a contiguous 2-D bfloat16 CUDA tensor");
  check_flat(out, "out", at::kBFloat16);
  const int64_t T = x.size(0);
  const int N = (int)x.size(1);
  TORCH_CHECK(out.numel() == N && N % 8 == 0 && ((uintptr_t)x.data_ptr()) % 16 == 0, "out must hold N elements, N % 8 == 0");
  c10::cuda::CUDAGuard guard(x.device());
  const int dev = x.get_device();
  const int R = col_sum_row_splits(T, N);
  TORCH_CHECK((int64_t)R * N <= (int64_t)64 * 8192, "too many columns for the column-sum scratch");
  at::Tensor& part = scratch(dev, (int64_t)R * N);
  at::Tensor& cnt = counters(dev, (N + 63) / 64);
  PCCL_CUDA(launch_col_sum(x.data_ptr(), T, N, out.data_ptr(), part.data_ptr<float>(), cnt.data_ptr<int>(), R,
                           at::cuda::getCurrentCUDAStream().stream()));
}

bool ln_bwd_supported(int64_t d) { return d == 1024 || d == 2048 || d == 4096; }

// du = dg * gelu'(u), and bias_grad[c] = sum_r du[r, c], in one pass.
at::Tensor gelu_bwd_col_sum(const at::Tensor& dg, const at::Tensor& u, at::Tensor& bias_grad) {
  TORCH_CHECK(dg.is_cuda() && dg.dim() == 2 && dg.scalar_type() == at::kBFloat16 && dg.is_contiguous(),
              "dg must be a contiguous 2-D bfloat16 CUDA tensor");
  TORCH_CHECK(u.sizes() == dg.sizes() && u.scalar_type() == at::kBFloat16 && u.is_contiguous() && u.device() == dg.device(),
              "u must match dg");
  check_flat(bias_grad, "bias_grad", at::kBFloat16);
  const int64_t T = dg.size(0);
  const int N = (int)dg.size(1);
  TORCH_CHECK(bias_grad.numel() == N && N % 8 == 0 && ((uintptr_t)dg.data_ptr()) % 16 == 0 && ((uintptr_t)u.data_ptr()) % 16 == 0,
              "bias_grad must hold N elements, N % 8 == 0, 16-byte aligned inputs");
  c10::cuda::CUDAGuard guard(dg.device());
  const int dev = dg.get_device();
  at::Tensor du = at::empty_like(dg);
  const int R = col_sum_row_splits(T, N);
  TORCH_CHECK((int64_t)R * N <= (int64_t)64 * 8192, "too many columns for the column-sum scratch");
  at::Tensor& part = scratch(dev, (int64_t)R * N);
  at::Tensor& cnt = counters(dev, (N + 63) / 64);
  PCCL_CUDA(launch_gelu_bwd_col_sum(dg.data_ptr(), u.data_ptr(), du.data_ptr(), T, N, bias_grad.data_ptr(),
                                    part.data_ptr<float>(), cnt.data_ptr<int>(), R, at::cuda::getCurrentCUDAStream().stream()));
  return du;
}

// [a | b | c] and its column sums in one pass (the packed q/k/v gradient and the QKV bias gradient).
at::Tensor cat3_col_sum(const at::Tensor& a, const at::Tensor& b, const at::Tensor& c, at::Tensor& bias_grad) {
  for (const at::Tensor* t : {&a, &b, &c})
    TORCH_CHECK(t->is_cuda() && t->dim() == 2 && t->scalar_type() == at::kBFloat16 && t->is_contiguous() &&
                    t->sizes() == a.sizes() && t->device() == a.device() && ((uintptr_t)t->data_ptr()) % 16 == 0,
                "a, b, c must be contiguous 2-D bfloat16 CUDA tensors of one shape, 16-byte aligned");
  const int64_t T = a.size(0);
  const int N = 3 * (int)a.size(1);
  check_flat(bias_grad, "bias_grad", at::kBFloat16);
  TORCH_CHECK(a.size(1) % 8 == 0 && bias_grad.numel() == N, "columns must be a multiple of 8; bias_grad holds 3x columns");
  c10::cuda::CUDAGuard guard(a.device());
  const int dev = a.get_device();
  at::Tensor cat = at::empty({T, N}, a.options());
  const int R = col_sum_row_splits(T, N);
  TORCH_CHECK((int64_t)R * N <= (int64_t)64 * 8192, "too many columns for the column-sum scratch");
  at::Tensor& part = scratch(dev, (int64_t)R * N);
  at::Tensor& cnt = counters(dev, (N + 63) / 64);
  PCCL_CUDA(launch_cat3_col_sum(a.data_ptr(), b.data_ptr(), c.data_ptr(), cat.data_ptr(), T, N, bias_grad.data_ptr(),
                                part.data_ptr<float>(), cnt.data_ptr<int>(), R, at::cuda::getCurrentCUDAStream().stream()));
  return cat;
}

at::Tensor gelu(const at::Tensor& u) {
  TORCH_CHECK(u.is_cuda() && u.scalar_type() == at::kBFloat16 && u.is_contiguous(), "u must be a contiguous bfloat16 CUDA tensor");
  TORCH_CHECK(u.numel() % 8 == 0 && ((uintptr_t)u.data_ptr()) % 16 == 0, "numel % 8 == 0 and 16-byte alignment required");
  c10::cuda::CUDAGuard guard(u.device());
  at::Tensor g = at::empty_like(u);
  PCCL_CUDA(launch_gelu_fwd(u.data_ptr(), g.data_ptr(), u.numel(), at::cuda::getCurrentCUDAStream().stream()));
  return g;
}

// y = layer_norm(x + branch) with the sum written back over branch; branch may be None.
std::tuple<at::Tensor, at::Tensor, at::Tensor> ln_fwd(const at::Tensor& x, std::optional<at::Tensor> branch,
                                                      const at::Tensor& gamma, const at::Tensor& beta, double eps) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.is_contiguous(), "x: contiguous 2-D bf16");
  const int64_t T = x.size(0), d = x.size(1);
  TORCH_CHECK(d == 1024 || d == 2048 || d == 4096, "layer-norm kernel takes d in {1024, 2048, 4096}");
  check_flat(gamma, "gamma", at::kBFloat16);
  check_flat(beta, "beta", at::kBFloat16);
  TORCH_CHECK(gamma.numel() == d && beta.numel() == d, "gamma and beta must hold d elements");
  TORCH_CHECK(((uintptr_t)x.data_ptr() | (uintptr_t)gamma.data_ptr() | (uintptr_t)beta.data_ptr()) % 16 == 0, "16-byte alignment");
  void* bptr = nullptr;
  if (branch.has_value()) {
    TORCH_CHECK(branch->sizes() == x.sizes() && branch->scalar_type() == at::kBFloat16 && branch->is_contiguous() &&
                    branch->device() == x.device() && ((uintptr_t)branch->data_ptr()) % 16 == 0,
                "branch must match x");
    bptr = branch->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty_like(x);
  at::Tensor mean = at::empty({T}, x.options().dtype(at::kFloat));
  at::Tensor rstd = at::empty({T}, x.options().dtype(at::kFloat));
  PCCL_CUDA(launch_ln_fwd(x.data_ptr(), bptr, gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), mean.data_ptr<float>(),
                          rstd.data_ptr<float>(), T, (int)d, (float)eps, at::cuda::getCurrentCUDAStream().stream()));
  return {y, mean, rstd};
}

at::Tensor ln_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& mean, const at::Tensor& rstd,
                  const at::Tensor& gamma, at::Tensor& dgamma, at::Tensor& dbeta, std::optional<at::Tensor> resid,
                  std::optional<at::Tensor> dx_col_sum) {
  TORCH_CHECK(dy.is_cuda() && dy.dim() == 2 && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous(), "dy: 2-D bf16");
  TORCH_CHECK(x.sizes() == dy.sizes() && x.scalar_type() == at::kBFloat16 && x.is_contiguous(), "x must match dy");
  const int64_t T = dy.size(0), d = dy.size(1);
  TORCH_CHECK(ln_bwd_supported(d), "layer-norm backward kernel takes d in {1024, 2048, 4096}");
  check_flat(mean, "mean", at::kFloat);
  check_flat(rstd, "rstd", at::kFloat);
  check_flat(gamma, "gamma", at::kBFloat16);
  check_flat(dgamma, "dgamma", at::kBFloat16);
  check_flat(dbeta, "dbeta", at::kBFloat16);
  TORCH_CHECK(mean.numel() == T && rstd.numel() == T && gamma.numel() == d && dgamma.numel() == d && dbeta.numel() == d,
              "size mismatch");
  const void* rptr = nullptr;
  if (resid.has_value()) {
    TORCH_CHECK(resid->sizes() == dy.sizes() && resid->scalar_type() == at::kBFloat16 && resid->is_contiguous() &&
                    resid->device() == dy.device() && ((uintptr_t)resid->data_ptr()) % 16 == 0,
                "resid must match dy");
    rptr = resid->data_ptr();
  }
  void* sptr = nullptr;
  if (dx_col_sum.has_value()) {
    check_flat(*dx_col_sum, "dx_col_sum", at::kBFloat16);
    TORCH_CHECK(dx_col_sum->numel() == d && dx_col_sum->device() == dy.device(), "dx_col_sum must hold d elements");
    sptr = dx_col_sum->data_ptr();
  }
  c10::cuda::CUDAGuard guard(dy.device());
  const int dev = dy.get_device();
  at::Tensor dx = at::empty_like(dy);
  const int64_t part = (int64_t)ln_bwd_blocks() * d;
  at::Tensor& sc = scratch(dev, 3 * part + (int64_t)64 * 8192);
  float* pg = sc.data_ptr<float>() + (int64_t)64 * 8192;     // the front of the buffer belongs to col_sum
  PCCL_CUDA(launch_ln_bwd(dy.data_ptr(), x.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), gamma.data_ptr(),
                          dx.data_ptr(), rptr, dgamma.data_ptr(), dbeta.data_ptr(), sptr, pg, T, (int)d,
                          at::cuda::getCurrentCUDAStream().stream()));
  return dx;
}

}  // namespace

void bind_optim(py::module_& m) {
  m.def("col_sum", &col_sum, "out[c] = sum_r x[r, c] (bf16 in/out, fp32 accumulation)");
  m.def("ln_bwd", &ln_bwd, py::arg("dy"), py::arg("x"), py::arg("mean"), py::arg("rstd"), py::arg("gamma"), py::arg("dgamma"),
        py::arg("dbeta"), py::arg("resid") = py::none(), py::arg("dx_col_sum") = py::none(),
        "layer-norm backward: returns dx (+ resid), writes dgamma, dbeta and optionally the column sums of dx");
  m.def("ln_fwd", &ln_fwd, py::arg("x"), py::arg("branch"), py::arg("gamma"), py::arg("beta"), py::arg("eps"),
        "layer norm of x (+ branch, summed in place into branch): returns (y, mean, rstd)");
  m.def("gelu", &gelu, "tanh-form GELU, bf16");
  m.def("cat3_col_sum", &cat3_col_sum, "returns [a | b | c]; bias_grad = its column sums");
  m.def("gelu_bwd_col_sum", &gelu_bwd_col_sum, "du = dg * gelu'(u); bias_grad = column sums of du");
  m.def("ln_bwd_supported", &ln_bwd_supported);
  m.def("sq_norm", &sq_norm, "out += sum(x*x)");
  m.def("adamw", &adamw, py::arg("master"), py::arg("exp_avg"), py::arg("exp_avg_sq"), py::arg("grad"), py::arg("param"),
        py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"), py::arg("step"),
        py::arg("grad_scale") = 1.0, py::arg("max_grad_norm") = 0.0, py::arg("total_sq_norm") = py::none());
  m.def("ce_fwd_bwd", &ce_fwd_bwd, py::arg("logits"), py::arg("targets"), py::arg("loss_sum"), py::arg("grad_scale"),
        py::arg("ignore_index") = -100, py::arg("bad_targets") = py::none());
}
