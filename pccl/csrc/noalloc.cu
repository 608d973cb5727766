// Implementation of the allocation-free reduce-scatter entry point (see noalloc.h for who
// needs it and for the rules).  The kernel is the library's ordinary reduce-scatter
// kernel; the only difference is where its scratch memory comes from.
#include "noalloc.h"

#include <cstdio>
#include <cstring>
#include <mutex>

#include "launch.h"

namespace {

using namespace pccl;

// Per emulated rank: staging for world-1 partial-sum blocks in the widest wire type (fp32),
// one signal region, one status word and one poison word.
constexpr uint64_t kStageBytes = (uint64_t)(PCCL_NOALLOC_MAX_RANKS - 1) * PCCL_NOALLOC_MAX_BLOCK_ELEMS * 4;   // 917,504
constexpr uint64_t kStageStride = (kStageBytes + 255) / 256 * 256;
constexpr uint64_t kSigStride = (kRegionBytes + 255) / 256 * 256;
constexpr uint64_t kStatusStride = 256;
constexpr uint64_t kRankStride = kStageStride + kSigStride + kStatusStride;
constexpr uint64_t kNoAllocScratchBytes = kRankStride * PCCL_NOALLOC_MAX_RANKS;                                  // ~8.6 MiB

// In host code this name is only a stand-in; the device address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
struct PerDevice {
  unsigned char* base = nullptr;   // device address of g_noalloc_scratch on this device
  uint32_t epoch = 0;              // call number carried by the flags
};
PerDevice g_dev[kMaxDevices];
std::mutex g_mu;

int fail(char* err, size_t err_len, int code, const char* fmt, long long a = 0, long long b = 0) {
  if (err != nullptr && err_len > 0) std::snprintf(err, err_len, fmt, a, b);
  return code;
}

}  // namespace

extern "C" int pccl_reduce_scatter_noalloc(const void* const* inputs, void* const* outputs, int world,
                                           uint64_t block_elems, int in_dtype, int out_dtype, int algo, float scale,
                                           cudaStream_t stream, char* err, size_t err_len) {
  if (inputs == nullptr || outputs == nullptr) return fail(err, err_len, -1, "inputs and outputs must not be null");
  if (world < 1 || world > PCCL_NOALLOC_MAX_RANKS)
    return fail(err, err_len, -2, "world size %lld is outside 1..%lld", world, PCCL_NOALLOC_MAX_RANKS);
  if (block_elems > PCCL_NOALLOC_MAX_BLOCK_ELEMS)
    return fail(err, err_len, -3,
                "block of %lld elements exceeds the built-in scratch (at most %lld elements per rank); "
                "use a communicator with its own staging area for larger reductions",
                (long long)block_elems, PCCL_NOALLOC_MAX_BLOCK_ELEMS);
  if (in_dtype < 0 || in_dtype > 2 || out_dtype < 0 || out_dtype > 2 || !(out_dtype == in_dtype || out_dtype == kF32))
    return fail(err, err_len, -4, "unsupported dtype pair (in %lld, out %lld)", in_dtype, out_dtype);
  if (algo != kDirect && algo != kRing && algo != kRecursive) return fail(err, err_len, -5, "unknown algorithm %lld", algo);
  if (algo == kRecursive && !is_pow2(world))
    return fail(err, err_len, -6, "recursive halving needs a power-of-two world size, got %lld", world);
  for (int r = 0; r < world; ++r)
    if (inputs[r] == nullptr || outputs[r] == nullptr) return fail(err, err_len, -1, "rank %lld has a null buffer", r);
  if (block_elems == 0) return 0;

  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices)
    return fail(err, err_len, -7, "cannot determine the current device (cuda error %lld)", (long long)e);

  std::lock_guard<std::mutex> lk(g_mu);
  PerDevice& pd = g_dev[device];
  if (pd.base == nullptr) {
    // First call on this device: resolve the device address of the static array.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(err, err_len, -8, "cudaGetSymbolAddress failed (cuda error %lld)", (long long)e);
    pd.base = static_cast<unsigned char*>(p);
  }

  ReduceScatterArgs a;
  std::memset(&a, 0, sizeof(a));
  GroupDev& g = a.g;
  g.size = world;
  g.nlocal = world;
  g.first_local = 0;
  g.epoch = ++pd.epoch;
  g.timeout_ns = 2ull * 1000 * 1000 * 1000;
  for (int r = 0; r < world; ++r) {
    unsigned char* rank_base = pd.base + (uint64_t)r * kRankStride;
    g.heap[r] = reinterpret_cast<char*>(rank_base);                                   // staging at offset 0
    g.sig[r] = reinterpret_cast<uint32_t*>(rank_base + kStageStride);
    g.status[r] = reinterpret_cast<Status*>(rank_base + kStageStride + kSigStride);
    g.poison[r] = reinterpret_cast<uint32_t*>(rank_base + kStageStride + kSigStride + 128);
    a.in[r] = static_cast<const char*>(inputs[r]);
    a.out[r] = static_cast<char*>(outputs[r]);
    // status and poison words must start at zero; the flags need no clearing (epoch-valued)
    e = cudaMemsetAsync(rank_base + kStageStride + kSigStride, 0, kStatusStride, stream);
    if (e != cudaSuccess) return fail(err, err_len, -9, "cudaMemsetAsync failed (cuda error %lld)", (long long)e);
  }
  a.algo = algo;
  a.in_dtype = in_dtype;
  a.wire_dtype = in_dtype;
  a.out_dtype = out_dtype;
  a.stage_off = 0;
  a.dst_stride = block_elems * (uint64_t)dtype_size(in_dtype);
  a.sub_stride = 0;
  a.sub_elems = block_elems;
  a.out_sub_stride = block_elems * (uint64_t)dtype_size(out_dtype);
  a.nsub = 1;
  a.scale = scale;
  const int lanes = (int)((block_elems + 4095) / 4096);   // at most 8 lanes x 8 ranks: always co-resident
  e = launch_reduce_scatter(a, lanes < 1 ? 1 : lanes, stream);
  if (e != cudaSuccess) return fail(err, err_len, -10, "kernel launch failed (cuda error %lld)", (long long)e);
  return 0;
}

extern "C" int pccl_reduce_scatter_noalloc_status(cudaStream_t stream, int world, uint32_t* codes, char* err, size_t err_len) {
  if (codes == nullptr) return fail(err, err_len, -1, "codes must not be null");
  if (world < 1 || world > PCCL_NOALLOC_MAX_RANKS)
    return fail(err, err_len, -2, "world size %lld is outside 1..%lld", world, PCCL_NOALLOC_MAX_RANKS);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices)
    return fail(err, err_len, -7, "cannot determine the current device (cuda error %lld)", (long long)e);
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    base = g_dev[device].base;
  }
  if (base == nullptr) return fail(err, err_len, -11, "no call has been made on device %lld yet", device);
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(err, err_len, -12, "cudaStreamSynchronize failed (cuda error %lld)", (long long)e);
  int bad = 0;
  for (int r = 0; r < world; ++r) {
    Status s;
    e = cudaMemcpy(&s, base + (uint64_t)r * kRankStride + kStageStride + kSigStride, sizeof(Status), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(err, err_len, -13, "cudaMemcpy of the status word failed (cuda error %lld)", (long long)e);
    codes[r] = s.code;
    if (s.code != kStatusOk) bad = 1;
  }
  return bad;
}
