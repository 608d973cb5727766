// Python bindings of the elementwise training kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

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
                int64_t ignore_index) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kBFloat16,
              "logits must be a 2-D bfloat16 CUDA tensor");
  TORCH_CHECK(logits.stride(1) == 1 && logits.stride(0) % 8 == 0, "logits rows must be contiguous and 16-byte aligned");
  TORCH_CHECK(((uintptr_t)logits.data_ptr()) % 16 == 0, "logits must be 16-byte aligned");
  check_flat(targets, "targets", at::kLong);
  check_flat(loss_sum, "loss_sum", at::kFloat);
  TORCH_CHECK(targets.numel() == logits.size(0), "one target per row");
  c10::cuda::CUDAGuard guard(logits.device());
  PCCL_CUDA(launch_ce_fwd_bwd(logits.data_ptr(), targets.data_ptr<int64_t>(), loss_sum.data_ptr<float>(), logits.size(0),
                              (int)logits.size(1), logits.stride(0), (float)grad_scale, ignore_index,
                              at::cuda::getCurrentCUDAStream().stream()));
}

}  // namespace

void bind_optim(py::module_& m) {
  m.def("sq_norm", &sq_norm, "out += sum(x*x)");
  m.def("adamw", &adamw, py::arg("master"), py::arg("exp_avg"), py::arg("exp_avg_sq"), py::arg("grad"), py::arg("param"),
        py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"), py::arg("step"),
        py::arg("grad_scale") = 1.0, py::arg("max_grad_norm") = 0.0, py::arg("total_sq_norm") = py::none());
  m.def("ce_fwd_bwd", &ce_fwd_bwd, py::arg("logits"), py::arg("targets"), py::arg("loss_sum"), py::arg("grad_scale"),
        py::arg("ignore_index") = -100);
}
