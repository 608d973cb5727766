// Host-side communicator: the table of peer-mapped heaps and signal pads, the symmetric
// allocator, the groups with their call counters, the status words that the kernels
// report into, and the launch of each collective.
//
// It replaces what the reference obtains from mpi4py: there an MPI_Comm is pulled out of
// the Python object (pccl/src/pccl.cpp:26,106) and workspaces come from the torch caching
// allocator on every call (pccl/src/pccl.cpp:54-59,67-73,127-131).  Peer-mapped memory
// cannot be allocated per call, so this object owns one heap for its whole life.
//
// Nothing here depends on torch; tensors are resolved to addresses by the binding layer.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "device_types.h"

namespace pccl {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

void throw_cuda(cudaError_t e, const char* expr, const char* file, int line);
#define PCCL_CUDA(expr)                                                   \
  do {                                                                    \
    cudaError_t pccl_e_ = (expr);                                         \
    if (pccl_e_ != cudaSuccess) ::pccl::throw_cuda(pccl_e_, #expr, __FILE__, __LINE__); \
  } while (0)

// First-fit allocator over byte offsets [0, size).  Every rank performs the same sequence
// of calls, so equal offsets name the same object on every rank (a symmetric heap).
class OffsetAllocator {
 public:
  explicit OffsetAllocator(uint64_t size = 0);
  int64_t alloc(uint64_t bytes, uint64_t align);  // -1 when it does not fit
  void free(int64_t off);
  uint64_t used() const { return used_; }
  uint64_t size() const { return size_; }
  uint64_t largest_free() const;

 private:
  uint64_t size_, used_ = 0;
  std::map<uint64_t, uint64_t> free_;   // offset -> length
  std::map<uint64_t, uint64_t> live_;   // offset -> length
};

struct GroupState {
  std::vector<int> ranks;     // world ranks, in group order
  int my_index = -1;          // index of this process in the group; -1: not a member (real mode)
  uint32_t epoch = 0;
  uint32_t region = 0;        // which slice of the signal pads belongs to this group
  cudaEvent_t tail = nullptr; // orders calls issued from different streams
  cudaStream_t last_stream = nullptr;
  bool used = false;
};

class Comm {
 public:
  // heaps/sigs: one address per WORLD rank as mapped into this process.  nlocal == world
  // means every rank lives on this GPU and one launch drives all of them (test emulation).
  Comm(int world, int rank, int nlocal, int device, std::vector<uint64_t> heaps, std::vector<uint64_t> sigs,
       uint64_t mc_heap, uint64_t heap_bytes, uint64_t sig_bytes, uint64_t staging_bytes);
  ~Comm();
  Comm(const Comm&) = delete;
  Comm& operator=(const Comm&) = delete;

  int world() const { return world_; }
  int rank() const { return rank_; }
  int nlocal() const { return nlocal_; }
  int device() const { return device_; }
  bool emulated() const { return nlocal_ > 1 || (world_ == 1 && false); }
  bool has_multimem() const { return mc_heap_ != 0; }
  uint64_t heap_bytes() const { return heap_bytes_; }
  uint64_t heap_base(int world_rank) const { return heaps_.at(world_rank); }
  uint64_t staging_off() const { return staging_off_; }
  uint64_t staging_bytes() const { return staging_bytes_; }
  int max_lanes() const { return max_lanes_; }
  // Eager area: two halves inside the heap, used alternately by the eager calls of the WORLD group
  // (group 0).  eager_capacity() is the size of one half (0: no area); next_eager_half() returns the
  // offset of the half the next eager call writes into and advances the alternation.  Every rank
  // issues the same sequence of eager calls, so the ranks agree on the half.
  uint64_t eager_capacity() const { return eager_half_bytes_; }
  uint64_t next_eager_half() { return eager_off_ + (uint64_t)((eager_calls_++) & 1u) * eager_half_bytes_; }

  int64_t alloc(uint64_t bytes, uint64_t align = 256);
  void free(int64_t off);
  uint64_t heap_used() const { return allocator_.used(); }
  // Offset of an address inside the heap of world rank `owner`, or -1.
  int64_t offset_of(uint64_t addr, uint64_t bytes, int owner) const;

  int new_group(const std::vector<int>& world_ranks);
  const GroupState& group(int gid) const { return groups_.at(gid); }
  int group_size(int gid) const { return (int)groups_.at(gid).ranks.size(); }
  int group_rank(int gid) const { return groups_.at(gid).my_index; }

  void set_timeout_ms(double ms) { timeout_ns_ = (uint64_t)(ms * 1e6); }
  double timeout_ms() const { return timeout_ns_ / 1e6; }

  // Status of local rank slot `li` (0 in real mode).  Reading does not synchronise.
  Status status(int li) const;
  bool poisoned() const;
  // Forget a failure: zero status words, poison flags, every signal region of this
  // process and all call counters.  Every rank must do this between the same two calls,
  // with no kernel of the communicator in flight (the caller synchronises the ranks).
  void reset_after_failure();

  // ---- collectives: fill the group part of the argument block, launch, bump the epoch
  void all_gather(int gid, AllGatherArgs a, int nlanes, cudaStream_t stream);
  void reduce_scatter(int gid, ReduceScatterArgs a, int nlanes, cudaStream_t stream);
  void all_reduce(int gid, AllReduceArgs a, int nlanes, cudaStream_t stream);
  // reduce-scatter + all-gather of the same schedule family (ring / recursive) in one launch
  void all_reduce_rsag(int gid, AllReduceRsAgArgs a, int nlanes, cudaStream_t stream);
  void broadcast(int gid, BroadcastArgs a, int nlanes, cudaStream_t stream);
  void barrier(int gid, cudaStream_t stream);

  // ---- debugging aids, both off by default
  // Stress mode: every lane sleeps a pseudo-random time below `jitter_ns` (at most 10 ms) before
  // each wait and signal.  Trace: keep up to `trace_events` records of passed synchronisation
  // points in device memory (0 frees the buffer).  Call with no kernel of the communicator in flight.
  void set_debug(uint64_t jitter_ns, uint64_t trace_events);
  // Synchronises the device, copies the trace out and empties it.  Also returns how many
  // records did not fit.
  std::vector<TraceEvent> read_trace(uint64_t* dropped);

  // Fill `g` for a launch on `stream` (also used by fused kernels living in other files).
  // `uses_staging`: the launch reads or writes the communicator's staging area.  Every group
  // shares that area, so such launches are ordered with one another across groups and streams.
  void begin_call(int gid, GroupDev* g, cudaStream_t stream, bool uses_staging = false);
  uint64_t kernels_launched() const { return launches_; }

 private:
  int clamp_lanes(int nlanes, const GroupState& gs) const;
  void check_extent(uint64_t off, uint64_t bytes, const char* what) const;
  bool in_staging(uint64_t off) const { return staging_bytes_ > 0 && off >= staging_off_ && off < staging_off_ + staging_bytes_; }

  int world_, rank_, nlocal_, device_;
  std::vector<uint64_t> heaps_, sigs_;
  uint64_t mc_heap_, heap_bytes_, sig_bytes_;
  uint64_t staging_off_ = 0, staging_bytes_ = 0;
  uint64_t eager_off_ = 0, eager_half_bytes_ = 0;
  uint64_t eager_calls_ = 0;
  cudaEvent_t staging_tail_ = nullptr;        // last launch that touched the staging area, on any group
  cudaStream_t staging_stream_ = nullptr;
  bool staging_used_ = false;
  OffsetAllocator allocator_;
  std::vector<GroupState> groups_;
  Status* status_ = nullptr;      // pinned, mapped: nlocal entries
  uint32_t* poison_ = nullptr;    // device: nlocal words
  uint64_t timeout_ns_ = 20ull * 1000 * 1000 * 1000;
  int max_lanes_ = 0;
  uint64_t launches_ = 0;
  TraceBuf* trace_ = nullptr;     // device
  uint32_t trace_capacity_ = 0;
  uint32_t jitter_ns_ = 0;
  mutable std::mutex mu_;
};

}  // namespace pccl
