// Python bindings of the tcgen05 GEMM and the fused all-gather+GEMM.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <cuda.h>

#include <map>
#include <mutex>
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

// One error word per device for every GEMM launch of this process: it stays 0 until a bounded
// wait of some launch runs out, and is never cleared by a launch (clear it with gemm_reset_error).
// Sharing it saves a memset per call; the training step issues hundreds of GEMMs.
at::Tensor& error_word(int device) {
  static at::Tensor words[64];
  at::Tensor& w = words[device & 63];
  if (!w.defined()) w = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  return w;
}

// Scratch for tiles that are split along K (see GemmArgs::sk_tiles): one buffer per device and
// stream, allocated on first use and kept, with a launch counter that makes every launch's flags
// distinct.  Launches that share a stream run one after the other, so they can share the scratch.
struct SkWorkspace {
  at::Tensor scratch, flags;
  uint32_t epoch = 0;
  at::Tensor counter;          // tiles handed out at run time: the draw counter of this stream
  uint32_t next_base = 0;
};
bool g_split_last_wave = true;
bool g_split_single_round = false;        // also split shapes with fewer tiles than CTA pairs (slower back to back: measured)
bool g_dynamic_tiles = false;  // hand tiles out at run time instead of dealing them out in advance
int g_max_pairs = 0, g_group_m = 0;      // tuning knobs, 0: the kernel's defaults
int g_wide = -1;                         // units of two row-tiles that share their W half: 1 always, 0 never, -1 where measured faster

SkWorkspace& sk_workspace(int device, cudaStream_t stream, int pairs) {
  static std::map<std::pair<int, cudaStream_t>, SkWorkspace> all;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  SkWorkspace& w = all[{device, stream}];
  const int64_t floats = (int64_t)pairs * (int64_t)(kGemmSkScratchBytesPerPair / sizeof(float));
  if (!w.scratch.defined() || w.scratch.numel() < floats) {
    w.scratch = at::empty({floats}, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, device));
    w.flags = at::zeros({(int64_t)pairs * (int64_t)kGemmSkFlagsPerPair}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
    w.epoch = 0;
    w.counter = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
    w.next_base = 0;
  }
  return w;
}

// Decide whether this plain CTA-pair launch splits its last round along K, and wire the scratch in.
void maybe_split_last_wave(GemmArgs& a, int device, cudaStream_t stream) {
  a.max_pairs = g_max_pairs;
  a.group_m = g_group_m;
  if (g_wide != 0 && g_max_pairs == 0 && a.two_cta && a.panel_flags == nullptr && a.M > 256) {
    // Units of two row-tiles (never split along K).  Measured on the training shapes: 6-28 % faster than
    // single tiles for contractions of 4096 and more when the units fill their rounds, slower for short
    // contractions, where the epilogue of a unit (both accumulators) is no longer hidden.
    const long long units = (long long)((a.M + 511) / 512) * ((a.N + 255) / 256);
    const long long pairs = sm_count(device) / 2;
    const long long rounds = (units + pairs - 1) / pairs;
    const bool fills = units * 5 >= rounds * pairs * 4;                  // at least 0.8 of the slots of its rounds
    if (g_wide > 0 || (a.K >= 4096 && fills)) a.wide = 1;
  }
  if (g_max_pairs > 0) return;           // a reduced grid is for measurements of the plain walk
  if (g_dynamic_tiles && a.two_cta) {
    // every pair draws its next tile (or unit) from a counter; the counter runs on from launch to launch
    const int sms = sm_count(device);
    int pairs = (sms - a.gather_ctas) / 2;
    const int tiles = (a.wide ? (a.M + 511) / 512 : (a.M + 255) / 256) * ((a.N + 255) / 256);
    if (a.panel_flags == nullptr && tiles < pairs) pairs = tiles;
    SkWorkspace& w = sk_workspace(device, stream, sms / 2);
    a.sched_counter = reinterpret_cast<uint32_t*>(w.counter.data_ptr<int>());
    a.sched_base = w.next_base;
    w.next_base += (uint32_t)tiles + (uint32_t)pairs;
    return;
  }
  if (a.wide) return;
  if (!g_split_last_wave || !a.two_cta || a.panel_flags != nullptr) return;
  const int sms = sm_count(device);
  const int n = gemm_sk_tiles(a.M, a.N, a.K, sms);
  if (n <= 0) return;
  // fewer tiles than CTA pairs: splitting every tile wins a single cold launch, but back to back under the power
  // cap the unsplit launch is faster (2048 x 2048 x 8192: 65 against 74 us), so it is opt-in
  if ((long long)((a.M + 255) / 256) * ((a.N + 255) / 256) < sms / 2 && !g_split_single_round) return;
  SkWorkspace& w = sk_workspace(device, stream, sms / 2);
  a.sk_tiles = n;
  a.sk_scratch = w.scratch.data_ptr<float>();
  a.sk_flags = reinterpret_cast<uint32_t*>(w.flags.data_ptr<int>());
  a.sk_epoch = ++w.epoch;
  if (a.sk_epoch == 0) a.sk_epoch = ++w.epoch;      // 0 is what fresh flags hold
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
  at::Tensor err = error_word(A.get_device());
  GemmArgs a;
  fill_common(a, A, C, bias, N, K, err);
  a.W = W.data_ptr();
  a.two_cta = two_cta ? 1 : 0;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
  maybe_split_last_wave(a, A.get_device(), stream);
  PCCL_CUDA(launch_gemm_sm100(a, sm_count(A.get_device()), stream));
  return {C, err};
}

// General layouts on the CTA-pair kernel.  C[M,N] = opA * opB with
//   a_mn false: A is [M,K]            a_mn true: A is [K,M]  (the product uses A^T)
//   b_mn false: B is [N,K] (B^T used) b_mn true: B is [K,N]
// so (false,false) is a linear layer's forward, (false,true) its data gradient dy * W and
// (true,true) its weight gradient dy^T * x.  bias (length N) is optional.
at::Tensor gemm_ex(const at::Tensor& A, const at::Tensor& B, bool a_mn, bool b_mn, std::optional<at::Tensor> bias,
                   std::optional<at::Tensor> out, std::optional<at::Tensor> gelu_grad_of) {
  check_bf16_2d(A, "A");
  check_bf16_2d(B, "B");
  const int M = (int)(a_mn ? A.size(1) : A.size(0)), K = (int)(a_mn ? A.size(0) : A.size(1));
  const int N = (int)(b_mn ? B.size(1) : B.size(0)), Kb = (int)(b_mn ? B.size(0) : B.size(1));
  TORCH_CHECK(K == Kb, "contraction lengths differ: ", K, " vs ", Kb);
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0, "K and N must be multiples of 8");
  TORCH_CHECK(!a_mn || M % 64 == 0, "a transposed A needs M % 64 == 0");
  TORCH_CHECK(!b_mn || N % 64 == 0, "a transposed B needs N % 64 == 0");
  c10::cuda::CUDAGuard guard(A.device());
  at::Tensor C = out.has_value() ? *out : at::empty({M, N}, A.options());
  check_bf16_2d(C, "out");
  TORCH_CHECK(C.size(0) == M && C.size(1) == N, "out has the wrong shape");
  at::Tensor err = error_word(A.get_device());
  GemmArgs a;
  fill_common(a, A, C, bias, N, K, err);
  a.M = M;
  a.W = B.data_ptr();
  a.two_cta = 1;
  a.a_mn = a_mn ? 1 : 0;
  a.b_mn = b_mn ? 1 : 0;
  if (gelu_grad_of.has_value()) {
    check_bf16_2d(*gelu_grad_of, "gelu_grad_of");
    TORCH_CHECK(gelu_grad_of->size(0) == M && gelu_grad_of->size(1) == N && !bias.has_value(),
                "gelu_grad_of must have the shape of the result, and excludes a bias");
    a.gelu_grad_of = gelu_grad_of->data_ptr();
  }
  cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
  maybe_split_last_wave(a, A.get_device(), stream);
  PCCL_CUDA(launch_gemm_sm100(a, sm_count(A.get_device()), stream));
  return C;
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
  at::Tensor err = error_word(A.get_device());
  GemmArgs a;
  fill_common(a, A, U, bias, N, K, err);
  a.W = W.data_ptr();
  a.act_out = G.data_ptr();
  a.two_cta = two_cta ? 1 : 0;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
  maybe_split_last_wave(a, A.get_device(), stream);
  PCCL_CUDA(launch_gemm_sm100(a, sm_count(A.get_device()), stream));
  return {U, G, err};
}

// ---------------------------------------------------------------- gather by the copy engines
// The second way to feed the fused kernel: instead of gatherer CTAs, the GPU's copy engines pull
// the peers' shards into the local buffer (one cudaMemcpyAsync per run of panels on a copy
// stream), and a stream-ordered 32-bit write raises each panel's flag when its bytes have
// landed.  All SMs multiply; a tile whose panel has not arrived waits on the flag exactly as
// it does for gatherer CTAs.  The copies need no SM, so they make progress while the persistent
// GEMM kernel occupies every SM (a flag-setting kernel could not: it would wait for the GEMM
// that waits for its flag).  The peers' shards must not change while they are read: this path
// has no handshake with the peers' kernels, the caller orders it against the writers (ZeRO-3
// parameters only change in the optimizer step, behind a barrier).
struct CopyLane {
  cudaStream_t stream = nullptr;
  cudaEvent_t ready = nullptr, done = nullptr;
};

CopyLane& copy_lane(int device) {
  static CopyLane lanes[64];
  CopyLane& l = lanes[device & 63];
  if (l.stream == nullptr) {
    PCCL_CUDA(cudaStreamCreateWithFlags(&l.stream, cudaStreamNonBlocking));
    PCCL_CUDA(cudaEventCreateWithFlags(&l.ready, cudaEventDisableTiming));
    PCCL_CUDA(cudaEventCreateWithFlags(&l.done, cudaEventDisableTiming));
  }
  return l;
}

using WriteValue32Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
using BatchMemOpFn = CUresult (*)(CUstream, unsigned int, CUstreamBatchMemOpParams*, unsigned int);

template <typename Fn>
Fn driver_entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return reinterpret_cast<Fn>(p);
}

// Write `value` into `count` consecutive 32-bit words at `first`, in stream order: one batched
// stream memory operation where the driver offers it, else one write per word.
void stream_write_words(cudaStream_t stream, uint32_t* first, int count, uint32_t value) {
  static BatchMemOpFn batch = driver_entry<BatchMemOpFn>("cuStreamBatchMemOp");
  static WriteValue32Fn single = driver_entry<WriteValue32Fn>("cuStreamWriteValue32");
  if (count <= 0) return;
  if (batch != nullptr && count > 1) {
    CUstreamBatchMemOpParams ops[64];
    for (int done = 0; done < count;) {
      const int n = std::min(64, count - done);
      std::memset(ops, 0, sizeof(CUstreamBatchMemOpParams) * n);
      for (int i = 0; i < n; ++i) {
        ops[i].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_32;
        ops[i].writeValue.address = reinterpret_cast<CUdeviceptr>(first + done + i);
        ops[i].writeValue.value = value;
        ops[i].writeValue.flags = CU_STREAM_WRITE_VALUE_DEFAULT;
      }
      const CUresult r = batch(reinterpret_cast<CUstream>(stream), (unsigned)n, ops, 0u);
      if (r != CUDA_SUCCESS) throw Error("cuStreamBatchMemOp failed with code " + std::to_string((int)r));
      done += n;
    }
    return;
  }
  if (single == nullptr) throw Error("this driver offers no stream memory operations (cuStreamWriteValue32)");
  for (int i = 0; i < count; ++i) {
    const CUresult r = single(reinterpret_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(first + i), value, 0u);
    if (r != CUDA_SUCCESS) throw Error("cuStreamWriteValue32 failed with code " + std::to_string((int)r));
  }
}

// Panel flags of the copy-engine feed: one buffer per device that is never cleared.  Every call
// takes the next number; its flag writes store that number and its kernel waits for a flag to
// reach it, so neither a memset nor a fresh allocation sits in front of a launch.
struct CeFlags {
  at::Tensor words;
  uint32_t epoch = 0;
};
CeFlags& ce_flags(int device, int panels) {
  static CeFlags all[64];
  CeFlags& f = all[device & 63];
  if (!f.words.defined() || f.words.numel() < panels) {
    f.words = at::zeros({std::max<int64_t>(panels, 1024)}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
    f.epoch = 0;
  }
  return f;
}

// One fused call fed by the copy engines.  Order of enqueueing: the event that holds the copies
// back until everything queued so far on `compute` is done (earlier readers of w_full), then the
// GEMM kernel, which starts on the own panels at once, then the copies and flag writes on the
// copy stream while the kernel already runs; the copies need no SM, so they progress beside the
// persistent kernel.  `panels_per_copy` <= 0: one copy per peer shard.
cudaError_t launch_fed_by_copy_engines(GemmArgs& a, char* w_full, int panels_per_copy, cudaStream_t compute, int device) {
  const int P = a.g.size, me = a.g.first_local;
  const int tpr = (a.N / P) / kGemmBN;
  const uint64_t panel_bytes = (uint64_t)kGemmBN * a.K * 2;
  const int ppc = panels_per_copy > 0 ? std::min(panels_per_copy, tpr) : tpr;
  CopyLane& l = copy_lane(device);
  CeFlags& f = ce_flags(device, a.N / kGemmBN);
  a.gather_ctas = 0;
  a.panel_flags = reinterpret_cast<uint32_t*>(f.words.data_ptr<int>());
  a.flag_target = ++f.epoch;
  if (a.flag_target == 0) a.flag_target = ++f.epoch;     // 0 is what a fresh buffer holds
  PCCL_CUDA(cudaEventRecord(l.ready, compute));
  const cudaError_t e = launch_gemm_sm100(a, sm_count(device), compute);
  if (e != cudaSuccess) return e;
  PCCL_CUDA(cudaStreamWaitEvent(l.stream, l.ready, 0));
  for (int k = 1; k < P; ++k) {
    const int p = (me + k) % P;
    for (int j0 = 0; j0 < tpr; j0 += ppc) {
      const int n = std::min(ppc, tpr - j0);
      const uint64_t dst_off = ((uint64_t)p * tpr + j0) * panel_bytes;
      PCCL_CUDA(cudaMemcpyAsync(w_full + dst_off, a.g.heap[p] + a.shard_off + (uint64_t)j0 * panel_bytes,
                                (uint64_t)n * panel_bytes, cudaMemcpyDeviceToDevice, l.stream));
      stream_write_words(l.stream, a.panel_flags + p * tpr + j0, n, a.flag_target);
    }
  }
  // the own rows last: the kernel multiplies them straight out of the shard, the copy only
  // completes the gathered weight for whoever uses it afterwards
  const uint64_t own_bytes = (uint64_t)tpr * panel_bytes;
  PCCL_CUDA(cudaMemcpyAsync(w_full + (uint64_t)me * own_bytes, a.g.heap[me] + a.shard_off, own_bytes, cudaMemcpyDeviceToDevice,
                            l.stream));
  PCCL_CUDA(cudaEventRecord(l.done, l.stream));
  PCCL_CUDA(cudaStreamWaitEvent(compute, l.done, 0));   // later work on `compute` sees the whole gathered weight
  return cudaSuccess;
}

int even_gatherers(int gather_ctas, bool two_cta) {
  return std::max(two_cta ? 2 : 1, two_cta ? (gather_ctas + 1) / 2 * 2 : gather_ctas);
}

// Fused all-gather + GEMM on a communicator group.  w_shard: this rank's [N/P, K] rows, in
// the symmetric heap; w_full: local [N, K] buffer that receives the gathered weight.
// copy_engine: gather with the copy engines (see above) instead of gatherer CTAs.
std::tuple<at::Tensor, at::Tensor> ag_gemm(Comm& c, int gid, const at::Tensor& A, const at::Tensor& w_shard,
                                           at::Tensor& w_full, std::optional<at::Tensor> bias,
                                           std::optional<at::Tensor> out, int gather_ctas, bool two_cta, bool copy_engine,
                                           int panels_per_copy) {
  check_bf16_2d(A, "A");
  check_bf16_2d(w_shard, "w_shard");
  check_bf16_2d(w_full, "w_full");
  TORCH_CHECK(c.nlocal() == 1, "the fused kernel runs one rank per process");
  const int P = c.group_size(gid);
  const int N = (int)w_full.size(0), K = (int)w_full.size(1);
  TORCH_CHECK(A.size(1) == K && w_shard.size(1) == K && w_shard.size(0) * P == N, "shape mismatch between A, shard and full weight");
  TORCH_CHECK(N % (P * kGemmBN) == 0, "every rank must own a multiple of 256 rows");
  TORCH_CHECK(K % 8 == 0, "K must be a multiple of 8");
  TORCH_CHECK(!copy_engine || two_cta, "the copy-engine gather feeds the CTA-pair kernel only");
  const int64_t off = c.offset_of((uint64_t)w_shard.data_ptr(), (uint64_t)w_shard.nbytes(), c.rank());
  TORCH_CHECK(off >= 0 && off % 16 == 0, "w_shard must live in the symmetric heap (pccl.empty_symmetric)");
  const int dev = c.device();
  c10::cuda::CUDAGuard guard(dev);
  at::Tensor C = out.has_value() ? *out : at::empty({A.size(0), N}, A.options());
  check_bf16_2d(C, "out");
  at::Tensor err = error_word(dev);
  GemmArgs a;
  fill_common(a, A, C, bias, N, K, err);
  a.W = w_full.data_ptr();
  a.two_cta = two_cta ? 1 : 0;
  a.shard_off = (uint64_t)off;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
  if (P == 1) {
    // one rank: the shard is the whole weight; multiply straight out of it
    a.W = w_shard.data_ptr();
    PCCL_CUDA(cudaMemcpyAsync(w_full.data_ptr(), w_shard.data_ptr(), w_shard.nbytes(), cudaMemcpyDeviceToDevice, stream));
    PCCL_CUDA(launch_gemm_sm100(a, sm_count(dev), stream));
    return {C, err};
  }
  c.begin_call(gid, &a.g, stream);
  if (copy_engine) {
    PCCL_CUDA(launch_fed_by_copy_engines(a, (char*)w_full.data_ptr(), panels_per_copy, stream, dev));
  } else {
    at::Tensor flags = at::zeros({N / kGemmBN}, A.options().dtype(at::kInt));    // counters: one add per gatherer CTA
    a.panel_flags = reinterpret_cast<uint32_t*>(flags.data_ptr<int>());
    a.gather_ctas = even_gatherers(gather_ctas, two_cta);
    PCCL_CUDA(launch_gemm_sm100(a, sm_count(dev), stream));
  }
  return {C, err};
}

// Same kernel with peers that are plain local buffers and no handshake: for tests on one GPU.
std::tuple<at::Tensor, at::Tensor> ag_gemm_local(const at::Tensor& A, std::vector<at::Tensor> shards, int me,
                                                 at::Tensor& w_full, std::optional<at::Tensor> bias, int gather_ctas,
                                                 bool two_cta, bool copy_engine, int panels_per_copy) {
  check_bf16_2d(A, "A");
  check_bf16_2d(w_full, "w_full");
  const int P = (int)shards.size();
  TORCH_CHECK(P >= 2 && P <= kMaxRanks && me >= 0 && me < P, "need 2..8 shards and a valid index");
  const int N = (int)w_full.size(0), K = (int)w_full.size(1);
  TORCH_CHECK(N % (P * kGemmBN) == 0 && K % 8 == 0 && A.size(1) == K, "shape mismatch");
  TORCH_CHECK(!copy_engine || two_cta, "the copy-engine gather feeds the CTA-pair kernel only");
  const int dev = A.get_device();
  c10::cuda::CUDAGuard guard(A.device());
  at::Tensor C = at::empty({A.size(0), N}, A.options());
  at::Tensor err = error_word(dev);
  at::Tensor flags = at::zeros({N / kGemmBN}, A.options().dtype(at::kInt));
  GemmArgs a;
  fill_common(a, A, C, bias, N, K, err);
  a.W = w_full.data_ptr();
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
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
  if (copy_engine) {
    PCCL_CUDA(launch_fed_by_copy_engines(a, (char*)w_full.data_ptr(), panels_per_copy, stream, dev));
  } else {
    a.gather_ctas = even_gatherers(gather_ctas, two_cta);
    PCCL_CUDA(launch_gemm_sm100(a, sm_count(dev), stream));
  }
  return {C, err};
}

}  // namespace

void bind_gemm(py::module_& m) {
  m.def("gemm", &gemm, py::arg("A"), py::arg("W"), py::arg("bias") = py::none(), py::arg("out") = py::none(),
        py::arg("two_cta") = true,
        "C = A @ W^T (+bias) on the tcgen05 tensor cores; returns (C, error_flag)");
  m.def("gemm_ex", &gemm_ex, py::arg("A"), py::arg("B"), py::arg("a_mn") = false, py::arg("b_mn") = false,
        py::arg("bias") = py::none(), py::arg("out") = py::none(), py::arg("gelu_grad_of") = py::none(),
        "C = opA * opB on the CTA-pair tcgen05 kernel; a_mn: A stored [K,M]; b_mn: B stored [K,N] (else [N,K]); "
        "gelu_grad_of: C is multiplied elementwise by gelu'(u) of this [M,N] tensor in the epilogue");
  m.def("gemm_set_dynamic_tiles", [](bool on) { g_dynamic_tiles = on; }, py::arg("on"),
        "CTA pairs draw their tiles from a counter at run time (robust beside kernels that hold some SMs) instead of a "
        "fixed round-robin share; excludes the split of the last round");
  m.def("gemm_set_split_last_wave", [](bool on, bool single_round) { g_split_last_wave = on; g_split_single_round = single_round; },
        py::arg("on"), py::arg("single_round") = false,
        "split the tiles of a partly filled last round along K over all CTA pairs (default on); single_round: also "
        "when the shape has fewer tiles than CTA pairs (default off)");
  m.def("gemm_set_wide", [](int mode) { g_wide = mode; }, py::arg("mode"),
        "Plain CTA-pair products in units of two vertically adjacent 256 x 256 tiles that share their W half (fewer "
        "operand bytes from L2 and HBM per FLOP; dealt out in advance, no split along K): 1 always, 0 never, "
        "-1 (default) for contractions of 4096 and more whose units fill their rounds");
  m.def("gemm_set_tuning", [](int max_pairs, int group_m) { g_max_pairs = max_pairs; g_group_m = group_m; },
        py::arg("max_pairs") = 0, py::arg("group_m") = 0,
        "measurement knobs of the CTA-pair kernel: cap on the CTA pairs used, row-tiles per band of the tile walk (0: defaults)");
  m.def("gemm_sk_tiles", &gemm_sk_tiles, py::arg("M"), py::arg("N"), py::arg("K"), py::arg("sm_count"),
        "how many leading tiles a plain launch of this shape splits along K (0: none)");
  m.def("gemm_error_word", [](int device) { return error_word(device); }, py::arg("device"),
        "the device's shared GEMM error word (0 unless a bounded wait of some launch ran out)");
  m.def("gemm_reset_error", [](int device) { error_word(device).zero_(); }, py::arg("device"));
  m.def("gemm_gelu", &gemm_gelu, py::arg("A"), py::arg("W"), py::arg("bias") = py::none(), py::arg("two_cta") = true,
        "(U, gelu(U), error_flag) with U = A @ W^T (+bias): activation fused into the GEMM epilogue");
  m.def("ag_gemm_local", &ag_gemm_local, py::arg("A"), py::arg("shards"), py::arg("me"), py::arg("w_full"),
        py::arg("bias") = py::none(), py::arg("gather_ctas") = 8, py::arg("two_cta") = true, py::arg("copy_engine") = false,
        py::arg("panels_per_copy") = 0);
  m.def("ag_gemm",
        [](std::shared_ptr<Comm> c, int gid, const at::Tensor& A, const at::Tensor& w_shard, at::Tensor& w_full,
           std::optional<at::Tensor> bias, std::optional<at::Tensor> out, int gather_ctas, bool two_cta, bool copy_engine,
           int panels_per_copy) {
          return ag_gemm(*c, gid, A, w_shard, w_full, bias, out, gather_ctas, two_cta, copy_engine, panels_per_copy);
        },
        py::arg("comm"), py::arg("gid"), py::arg("A"), py::arg("w_shard"), py::arg("w_full"), py::arg("bias") = py::none(),
        py::arg("out") = py::none(), py::arg("gather_ctas") = 16, py::arg("two_cta") = true, py::arg("copy_engine") = false,
        py::arg("panels_per_copy") = 0);
}
