// Python bindings of the tcgen05 GEMM and the fused all-gather+GEMM.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <optional>

#include "comm.h"
#include "gemm.h"

namespace py = pybind11;
using namespace pccl;

namespace {

int sm_count(int device) {
  static int cached[64] = {0};
  if (device >= 0 && device < 64 && cached[device] > 0) return cached[device];
  int n = 0;
  PCCL_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
  if (device >= 0 && device < 64) cached[device] = n;
  return n;
}

void check_bf16_2d(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2 && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), name,
              " must be a contiguous 2-D bfloat16 CUDA tensor");
}

void fill_common(GemmArgs& a, const at::Tensor& A, const at::Tensor& C, const std::optional<at::Tensor>& bias, int N, int K,
                 at::Tensor& err) {
  std::memset(&a, 0, sizeof(a));
  a.M = (int)A.size(0);
  a.N = N;
  a.K = K;
  a.A = A.data_ptr();
  a.C = C.data_ptr();
  a.error = err.data_ptr<int>();
  if (bias.has_value()) {
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kBFloat16 && bias->numel() == N && bias->is_contiguous(),
                "bias must be a contiguous bfloat16 vector of N elements");
    a.bias = bias->data_ptr();
  }
}

// C = A @ W^T (+ bias).  Returns (C, error flag tensor): error stays 0 unless a bounded wait ran out.
std::tuple<at::Tensor, at::Tensor> gemm(const at::Tensor& A, const at::Tensor& W, std::optional<at::Tensor> bias,
                                        std::optional<at::Tensor> out, bool two_cta) {
  check_bf16_2d(A, "A");
  check_bf16_2d(W, "W");
  TORCH_CHECK(A.size(1) == W.size(1), "A is [M,K], W is [N,K]: K differs");
  const int N = (int)W.size(0), K = (int)W.size(1);
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0, "K and N must be multiples of 8");
  c10::cuda::CUDAGuard guard(A.device());
  at::Tensor C = out.has_value() ? *out : at::empty({A.size(0), N}, A.options());
  check_bf16_2d(C, "out");
  TORCH_CHECK(C.size(0) == A.size(0) && C.size(1) == N, "out has the wrong shape");
  at::Tensor err = at::zeros({1}, A.options().dtype(at::kInt));
  GemmArgs a;
  fill_common(a, A, C, bias, N, K, err);
  a.W = W.data_ptr();
  a.two_cta = two_cta ? 1 : 0;
  PCCL_CUDA(launch_gemm_sm100(a, sm_count(A.get_device()), at::cuda::getCurrentCUDAStream().stream()));
  return {C, err};
}

// U = A @ W^T + bias and G = gelu(U) from one kernel: the first linear layer of a transformer MLP
// with its activation in the epilogue.  Returns (U, G, error flag); the backward pass needs both.
std::tuple<at::Tensor, at::Tensor, at::Tensor> gemm_gelu(const at::Tensor& A, const at::Tensor& W,
                                                         std::optional<at::Tensor> bias, bool two_cta) {
  check_bf16_2d(A, "A");
  check_bf16_2d(W, "W");
  TORCH_CHECK(A.size(1) == W.size(1), "A is [M,K], W is [N,K]: K differs");
  const int N = (int)W.size(0), K = (int)W.size(1);
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0, "K and N must be multiples of 8");
  c10::cuda::CUDAGuard guard(A.device());
  at::Tensor U = at::empty({A.size(0), N}, A.options());
  at::Tensor G = at::empty({A.size(0), N}, A.options());
  at::Tensor err = at::zeros({1}, A.options().dtype(at::kInt));
  GemmArgs a;
  fill_common(a, A, U, bias, N, K, err);
  a.W = W.data_ptr();
  a.act_out = G.data_ptr();
  a.two_cta = two_cta ? 1 : 0;
  PCCL_CUDA(launch_gemm_sm100(a, sm_count(A.get_device()), at::cuda::getCurrentCUDAStream().stream()));
  return {U, G, err};
}

// Fused all-gather + GEMM on a communicator group.  w_shard: this rank's [N/P, K] rows, in
// the symmetric heap; w_full: local [N, K] buffer that receives the gathered weight.
std::tuple<at::Tensor, at::Tensor> ag_gemm(Comm& c, int gid, const at::Tensor& A, const at::Tensor& w_shard,
                                           at::Tensor& w_full, std::optional<at::Tensor> bias,
                                           std::optional<at::Tensor> out, int gather_ctas, bool two_cta) {
  check_bf16_2d(A, "A");
  check_bf16_2d(w_shard, "w_shard");
  check_bf16_2d(w_full, "w_full");
  TORCH_CHECK(c.nlocal() == 1, "the fused kernel runs one rank per process");
  const int P = c.group_size(gid);
  const int N = (int)w_full.size(0), K = (int)w_full.size(1);
  TORCH_CHECK(A.size(1) == K && w_shard.size(1) == K && w_shard.size(0) * P == N, "shape mismatch between A, shard and full weight");
  TORCH_CHECK(N % (P * kGemmBN) == 0, "every rank must own a multiple of 256 rows");
  TORCH_CHECK(K % 8 == 0, "K must be a multiple of 8");
  const int64_t off = c.offset_of((uint64_t)w_shard.data_ptr(), (uint64_t)w_shard.nbytes(), c.rank());
  TORCH_CHECK(off >= 0 && off % 16 == 0, "w_shard must live in the symmetric heap (pccl.empty_symmetric)");
  const int dev = c.device();
  c10::cuda::CUDAGuard guard(dev);
  at::Tensor C = out.has_value() ? *out : at::empty({A.size(0), N}, A.options());
  check_bf16_2d(C, "out");
  at::Tensor err = at::zeros({1}, A.options().dtype(at::kInt));
  at::Tensor flags = at::zeros({N / kGemmBN}, A.options().dtype(at::kInt));
  GemmArgs a;
  fill_common(a, A, C, bias, N, K, err);
  a.W = w_full.data_ptr();
  a.gather_ctas = P > 1 ? std::max(two_cta ? 2 : 1, two_cta ? (gather_ctas + 1) / 2 * 2 : gather_ctas) : 0;
  a.two_cta = two_cta ? 1 : 0;
  a.shard_off = (uint64_t)off;
  a.panel_flags = reinterpret_cast<uint32_t*>(flags.data_ptr<int>());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
  if (P > 1) {
    c.begin_call(gid, &a.g, stream);
  } else {
    // one rank: the shard is the whole weight; multiply straight out of it
    a.W = w_shard.data_ptr();
    PCCL_CUDA(cudaMemcpyAsync(w_full.data_ptr(), w_shard.data_ptr(), w_shard.nbytes(), cudaMemcpyDeviceToDevice, stream));
  }
  PCCL_CUDA(launch_gemm_sm100(a, sm_count(dev), stream));
  return {C, err};
}

// Same kernel with peers that are plain local buffers and no handshake: for tests on one GPU.
std::tuple<at::Tensor, at::Tensor> ag_gemm_local(const at::Tensor& A, std::vector<at::Tensor> shards, int me,
                                                 at::Tensor& w_full, std::optional<at::Tensor> bias, int gather_ctas,
                                                 bool two_cta) {
  check_bf16_2d(A, "A");
  check_bf16_2d(w_full, "w_full");
  const int P = (int)shards.size();
  TORCH_CHECK(P >= 2 && P <= kMaxRanks && me >= 0 && me < P, "need 2..8 shards and a valid index");
  const int N = (int)w_full.size(0), K = (int)w_full.size(1);
  TORCH_CHECK(N % (P * kGemmBN) == 0 && K % 8 == 0 && A.size(1) == K, "shape mismatch");
  c10::cuda::CUDAGuard guard(A.device());
  at::Tensor C = at::empty({A.size(0), N}, A.options());
  at::Tensor err = at::zeros({1}, A.options().dtype(at::kInt));
  at::Tensor flags = at::zeros({N / kGemmBN}, A.options().dtype(at::kInt));
  GemmArgs a;
  fill_common(a, A, C, bias, N, K, err);
  a.W = w_full.data_ptr();
  a.gather_ctas = std::max(two_cta ? 2 : 1, two_cta ? (gather_ctas + 1) / 2 * 2 : gather_ctas);
  a.two_cta = two_cta ? 1 : 0;
  a.shard_off = 0;
  a.panel_flags = reinterpret_cast<uint32_t*>(flags.data_ptr<int>());
  a.g.size = P;
  a.g.nlocal = 1;
  a.g.first_local = me;
  a.g.timeout_ns = 2ull * 1000 * 1000 * 1000;
  for (int p = 0; p < P; ++p) {
    check_bf16_2d(shards[p], "shard");
    TORCH_CHECK(shards[p].size(0) * P == N && shards[p].size(1) == K, "shard has the wrong shape");
    a.g.heap[p] = (char*)shards[p].data_ptr();
  }
  PCCL_CUDA(launch_gemm_sm100(a, sm_count(A.get_device()), at::cuda::getCurrentCUDAStream().stream()));
  return {C, err};
}

}  // namespace

void bind_gemm(py::module_& m) {
  m.def("gemm", &gemm, py::arg("A"), py::arg("W"), py::arg("bias") = py::none(), py::arg("out") = py::none(),
        py::arg("two_cta") = true,
        "C = A @ W^T (+bias) on the tcgen05 tensor cores; returns (C, error_flag)");
  m.def("gemm_gelu", &gemm_gelu, py::arg("A"), py::arg("W"), py::arg("bias") = py::none(), py::arg("two_cta") = true,
        "(U, gelu(U), error_flag) with U = A @ W^T (+bias): activation fused into the GEMM epilogue");
  m.def("ag_gemm_local", &ag_gemm_local, py::arg("A"), py::arg("shards"), py::arg("me"), py::arg("w_full"),
        py::arg("bias") = py::none(), py::arg("gather_ctas") = 8, py::arg("two_cta") = true);
  m.def("ag_gemm",
        [](std::shared_ptr<Comm> c, int gid, const at::Tensor& A, const at::Tensor& w_shard, at::Tensor& w_full,
           std::optional<at::Tensor> bias, std::optional<at::Tensor> out, int gather_ctas, bool two_cta) {
          return ag_gemm(*c, gid, A, w_shard, w_full, bias, out, gather_ctas, two_cta);
        },
        py::arg("comm"), py::arg("gid"), py::arg("A"), py::arg("w_shard"), py::arg("w_full"), py::arg("bias") = py::none(),
        py::arg("out") = py::none(), py::arg("gather_ctas") = 16, py::arg("two_cta") = true);
}
