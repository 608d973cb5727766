#include "comm.h"

#include <algorithm>
#include <cstring>
#include <sstream>

#include "launch.h"

namespace pccl {

void throw_cuda(cudaError_t e, const char* expr, const char* file, int line) {
  std::ostringstream os;
  os << "CUDA error " << (int)e << " (" << cudaGetErrorName(e) << ": " << cudaGetErrorString(e) << ") in `" << expr
     << "` at " << file << ":" << line;
  throw Error(os.str());
}

// ------------------------------------------------------------------ OffsetAllocator
OffsetAllocator::OffsetAllocator(uint64_t size) : size_(size) {
  if (size > 0) free_[0] = size;
}

int64_t OffsetAllocator::alloc(uint64_t bytes, uint64_t align) {
  if (bytes == 0) bytes = 1;
  if (align == 0) align = 1;
  for (auto it = free_.begin(); it != free_.end(); ++it) {
    const uint64_t start = it->first, len = it->second;
    const uint64_t aligned = (start + align - 1) / align * align;
    if (aligned + bytes > start + len) continue;
    const uint64_t tail_start = aligned + bytes, tail_len = start + len - tail_start;
    free_.erase(it);
    if (aligned > start) free_[start] = aligned - start;
    if (tail_len > 0) free_[tail_start] = tail_len;
    live_[aligned] = bytes;
    used_ += bytes;
    return (int64_t)aligned;
  }
  return -1;
}

void OffsetAllocator::free(int64_t off) {
  auto it = live_.find((uint64_t)off);
  if (it == live_.end()) throw Error("OffsetAllocator::free: offset was not allocated");
  uint64_t start = it->first, len = it->second;
  used_ -= len;
  live_.erase(it);
  // The alignment gap in front of a block stays a separate free range; merge neighbours.
  auto next = free_.lower_bound(start);
  if (next != free_.end() && start + len == next->first) {
    len += next->second;
    next = free_.erase(next);
  }
  if (next != free_.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == start) {
      start = prev->first;
      len += prev->second;
      free_.erase(prev);
    }
  }
  free_[start] = len;
}

uint64_t OffsetAllocator::largest_free() const {
  uint64_t m = 0;
  for (auto& kv : free_) m = std::max(m, kv.second);
  return m;
}

// ------------------------------------------------------------------ Comm
Comm::Comm(int world, int rank, int nlocal, int device, std::vector<uint64_t> heaps, std::vector<uint64_t> sigs,
           uint64_t mc_heap, uint64_t heap_bytes, uint64_t sig_bytes, uint64_t staging_bytes)
    : world_(world), rank_(rank), nlocal_(nlocal), device_(device), heaps_(std::move(heaps)), sigs_(std::move(sigs)),
      mc_heap_(mc_heap), heap_bytes_(heap_bytes), sig_bytes_(sig_bytes), allocator_(heap_bytes) {
  if (world < 1 || world > kMaxRanks) throw Error("world size must be between 1 and 8 (one NVSwitch domain)");
  if (nlocal != 1 && nlocal != world) throw Error("nlocal must be 1 (one rank per process) or world (emulation)");
  if (rank < 0 || rank >= world) throw Error("rank out of range");
  if ((int)heaps_.size() != world || (int)sigs_.size() != world) throw Error("need one heap and one signal pad per rank");
  if (sig_bytes < kRegionBytes) throw Error("signal pad smaller than one group region");
  PCCL_CUDA(cudaSetDevice(device));
  PCCL_CUDA(cudaHostAlloc((void**)&status_, sizeof(Status) * nlocal, cudaHostAllocMapped | cudaHostAllocPortable));
  std::memset(status_, 0, sizeof(Status) * nlocal);
  PCCL_CUDA(cudaMalloc((void**)&poison_, sizeof(uint32_t) * nlocal));
  PCCL_CUDA(cudaMemset(poison_, 0, sizeof(uint32_t) * nlocal));
  PCCL_CUDA(cudaEventCreateWithFlags(&staging_tail_, cudaEventDisableTiming));
  max_lanes_ = max_resident_lanes(device);
  if (max_lanes_ <= 0) throw Error("could not determine how many lanes fit on the device");
  if (staging_bytes > 0) {
    const int64_t off = allocator_.alloc(staging_bytes, 4096);
    if (off < 0) throw Error("staging area does not fit into the symmetric heap");
    staging_off_ = (uint64_t)off;
    staging_bytes_ = staging_bytes;
  }
  // the eager area: at most 2 x 8 MiB, at most an eighth of the heap; none in very small heaps
  uint64_t half = std::min<uint64_t>(8ull << 20, heap_bytes / 16) / 4096 * 4096;
  if (world > 1 && half >= (64u << 10)) {
    const int64_t off = allocator_.alloc(2 * half, 4096);
    if (off >= 0) {
      eager_off_ = (uint64_t)off;
      eager_half_bytes_ = half;
    }
  }
}

Comm::~Comm() {
  for (auto& g : groups_)
    if (g.tail) cudaEventDestroy(g.tail);
  if (staging_tail_) cudaEventDestroy(staging_tail_);
  if (status_) cudaFreeHost(status_);
  if (poison_) cudaFree(poison_);
  if (trace_) cudaFree(trace_);
}

void Comm::set_debug(uint64_t jitter_ns, uint64_t trace_events) {
  if (jitter_ns > 10ull * 1000 * 1000) throw Error("jitter above 10 ms per synchronisation point is refused");
  if (trace_events > (1ull << 24)) throw Error("trace capacity above 16 Mi records is refused");
  jitter_ns_ = (uint32_t)jitter_ns;
  if (trace_ != nullptr && trace_events != trace_capacity_) {
    PCCL_CUDA(cudaDeviceSynchronize());
    PCCL_CUDA(cudaFree(trace_));
    trace_ = nullptr;
    trace_capacity_ = 0;
  }
  if (trace_events > 0 && trace_ == nullptr) {
    const size_t bytes = sizeof(TraceBuf) + (size_t)trace_events * sizeof(TraceEvent);
    PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&trace_), bytes));
    PCCL_CUDA(cudaMemset(trace_, 0, bytes));
    const uint32_t cap = (uint32_t)trace_events;
    PCCL_CUDA(cudaMemcpy(&trace_->capacity, &cap, sizeof(cap), cudaMemcpyHostToDevice));
    trace_capacity_ = cap;
  }
}

std::vector<TraceEvent> Comm::read_trace(uint64_t* dropped) {
  std::vector<TraceEvent> out;
  if (dropped) *dropped = 0;
  if (trace_ == nullptr) return out;
  PCCL_CUDA(cudaDeviceSynchronize());
  unsigned long long count = 0;
  PCCL_CUDA(cudaMemcpy(&count, &trace_->count, sizeof(count), cudaMemcpyDeviceToHost));
  const uint64_t kept = count < trace_capacity_ ? count : trace_capacity_;
  out.resize(kept);
  if (kept > 0) PCCL_CUDA(cudaMemcpy(out.data(), trace_->ev, kept * sizeof(TraceEvent), cudaMemcpyDeviceToHost));
  if (dropped) *dropped = count - kept;
  PCCL_CUDA(cudaMemset(&trace_->count, 0, sizeof(count)));
  return out;
}

int64_t Comm::alloc(uint64_t bytes, uint64_t align) {
  std::lock_guard<std::mutex> lk(mu_);
  return allocator_.alloc(bytes, align);
}

void Comm::free(int64_t off) {
  std::lock_guard<std::mutex> lk(mu_);
  allocator_.free(off);
}

int64_t Comm::offset_of(uint64_t addr, uint64_t bytes, int owner) const {
  const uint64_t base = heaps_.at(owner);
  if (addr < base || addr + bytes > base + heap_bytes_) return -1;
  return (int64_t)(addr - base);
}

int Comm::new_group(const std::vector<int>& world_ranks) {
  std::lock_guard<std::mutex> lk(mu_);
  if (world_ranks.empty() || (int)world_ranks.size() > kMaxRanks) throw Error("bad group size");
  std::vector<int> seen(world_, 0);
  for (int r : world_ranks) {
    if (r < 0 || r >= world_) throw Error("group rank outside the communicator");
    if (seen[r]++) throw Error("duplicate rank in group");
  }
  const uint32_t region = (uint32_t)groups_.size();
  if ((uint64_t)(region + 1) * kRegionBytes > sig_bytes_) throw Error("signal pad exhausted: too many groups");
  GroupState g;
  g.ranks = world_ranks;
  g.region = region;
  if (nlocal_ == 1) {
    auto it = std::find(world_ranks.begin(), world_ranks.end(), rank_);
    g.my_index = it == world_ranks.end() ? -1 : (int)(it - world_ranks.begin());
  } else {
    g.my_index = 0;
  }
  PCCL_CUDA(cudaEventCreateWithFlags(&g.tail, cudaEventDisableTiming));
  groups_.push_back(g);
  return (int)groups_.size() - 1;
}

Status Comm::status(int li) const {
  if (li < 0 || li >= nlocal_) throw Error("local rank slot out of range");
  Status s;
  std::memcpy(&s, (const void*)&status_[li], sizeof(Status));
  return s;
}

bool Comm::poisoned() const {
  for (int i = 0; i < nlocal_; ++i)
    if (((volatile Status*)status_)[i].code != kStatusOk) return true;
  return false;
}

void Comm::reset_after_failure() {
  std::lock_guard<std::mutex> lk(mu_);
  PCCL_CUDA(cudaDeviceSynchronize());
  std::memset(status_, 0, sizeof(Status) * nlocal_);
  PCCL_CUDA(cudaMemset(poison_, 0, sizeof(uint32_t) * nlocal_));
  if (nlocal_ == 1) {
    PCCL_CUDA(cudaMemset((void*)sigs_[rank_], 0, sig_bytes_));
  } else {
    for (int r = 0; r < world_; ++r) PCCL_CUDA(cudaMemset((void*)sigs_[r], 0, sig_bytes_));
  }
  for (auto& g : groups_) {
    g.epoch = 0;
    g.used = false;
  }
  eager_calls_ = 0;
  PCCL_CUDA(cudaDeviceSynchronize());
}

void Comm::begin_call(int gid, GroupDev* g, cudaStream_t stream, bool uses_staging) {
  GroupState& gs = groups_.at(gid);
  if (gs.my_index < 0) throw Error("this rank is not a member of the group");
  // The staging area belongs to the communicator, not to a group: two launches that use it must
  // not overlap on this rank even when they belong to different groups (whose flags are
  // separate) and sit on different streams.  A peer writes into this rank's staging only after
  // this rank's kernel of the same call has signalled its entry, so local ordering is enough.
  if (uses_staging) {
    if (staging_used_ && staging_stream_ != stream) {
      PCCL_CUDA(cudaEventRecord(staging_tail_, staging_stream_));
      PCCL_CUDA(cudaStreamWaitEvent(stream, staging_tail_, 0));
    }
    staging_used_ = true;
    staging_stream_ = stream;
  }
  // Calls on one group share its flags, so they must execute in issue order even when the
  // caller switches streams.
  if (gs.used && gs.last_stream != stream) {
    PCCL_CUDA(cudaEventRecord(gs.tail, gs.last_stream));
    PCCL_CUDA(cudaStreamWaitEvent(stream, gs.tail, 0));
  }
  gs.used = true;
  gs.last_stream = stream;
  gs.epoch += 1;
  std::memset(g, 0, sizeof(GroupDev));
  const int P = (int)gs.ranks.size();
  g->size = P;
  g->epoch = gs.epoch;
  g->timeout_ns = timeout_ns_;
  g->trace = trace_;
  g->jitter_ns = jitter_ns_;
  g->mc_heap = (char*)mc_heap_;
  for (int i = 0; i < P; ++i) {
    g->heap[i] = (char*)heaps_[gs.ranks[i]];
    g->sig[i] = (uint32_t*)(sigs_[gs.ranks[i]] + (uint64_t)gs.region * kRegionBytes);
  }
  if (nlocal_ > 1) {
    g->nlocal = P;
    g->first_local = 0;
    for (int i = 0; i < P; ++i) {
      g->status[i] = status_ + gs.ranks[i];
      g->poison[i] = poison_ + gs.ranks[i];
    }
  } else {
    g->nlocal = 1;
    g->first_local = gs.my_index;
    g->status[0] = status_;
    g->poison[0] = poison_;
  }
  launches_ += 1;
}

int Comm::clamp_lanes(int nlanes, const GroupState& gs) const {
  int cap = max_lanes_;
  if (nlocal_ > 1) cap = std::max(1, max_lanes_ / (int)gs.ranks.size());  // all emulated ranks must be resident
  return std::max(1, std::min(nlanes, cap));
}

// Every address a kernel forms inside a peer's heap is "offset given by the host + something the
// kernel derives from the sizes"; the largest such address is checked here, on the host, before
// anything is launched, so a wrong offset or stride becomes an exception instead of a stray
// store into a neighbour's buffer (the memory checker of the toolkit cannot be used on the pool).
void Comm::check_extent(uint64_t off, uint64_t bytes, const char* what) const {
  if (off > heap_bytes_ || bytes > heap_bytes_ - off)
    throw Error(std::string(what) + ": the range [" + std::to_string(off) + ", +" + std::to_string(bytes) +
                ") leaves the symmetric heap of " + std::to_string(heap_bytes_) + " bytes");
}

void Comm::all_gather(int gid, AllGatherArgs a, int nlanes, cudaStream_t stream) {
  if (a.algo == kMultimem && mc_heap_ == 0) throw Error("multimem all-gather requested but no multicast mapping exists");
  {
    const uint64_t P = (uint64_t)group_size(gid), ns = (uint64_t)(a.nsub > 0 ? a.nsub - 1 : 0);
    if (a.algo == kPull) {
      check_extent(a.in_off, ns * a.in_sub_stride + a.sub_bytes, "all-gather (pull) input slot");
    } else if (P > 1) {
      check_extent(a.recv_off, (P - 1) * a.src_stride + ns * a.sub_stride + a.sub_bytes, "all-gather landing zone");
    }
  }
  if (a.algo == kRecursive && !is_pow2(group_size(gid))) throw Error("recursive doubling needs a power-of-two group");
  // user tensors never lie inside the staging area (the allocator has reserved it), so an offset
  // there means staging; pull leaves recv_off unused and stages only a private input
  const bool staged = a.algo == kPull ? (a.in[0] != nullptr || in_staging(a.in_off)) : in_staging(a.recv_off);
  begin_call(gid, &a.g, stream, staged);
  PCCL_CUDA(launch_all_gather(a, clamp_lanes(nlanes, groups_[gid]), stream));
}

void Comm::reduce_scatter(int gid, ReduceScatterArgs a, int nlanes, cudaStream_t stream) {
  if (a.algo == kMultimem && mc_heap_ == 0) throw Error("multimem reduce-scatter requested but no multicast mapping exists");
  if (a.algo == kRecursive && !is_pow2(group_size(gid))) throw Error("recursive halving needs a power-of-two group");
  {
    const uint64_t P = (uint64_t)group_size(gid), ns = (uint64_t)(a.nsub > 0 ? a.nsub : 1);
    if (a.algo == kPull || a.algo == kMultimem) {
      check_extent(a.in_off, (P - 1) * a.dst_stride + (ns - 1) * a.sub_stride + a.sub_elems * (uint64_t)dtype_size(a.in_dtype),
                   "reduce-scatter symmetric input");
    } else if (P > 1) {
      check_extent(a.stage_off, (P - 1) * ns * a.sub_elems * (uint64_t)dtype_size(a.wire_dtype), "reduce-scatter staging");
    }
  }
  const bool staged = a.algo != kPull && a.algo != kMultimem && in_staging(a.stage_off);
  begin_call(gid, &a.g, stream, staged);
  PCCL_CUDA(launch_reduce_scatter(a, clamp_lanes(nlanes, groups_[gid]), stream));
}

void Comm::all_reduce(int gid, AllReduceArgs a, int nlanes, cudaStream_t stream) {
  if (a.algo == kMultimem && mc_heap_ == 0) throw Error("multimem all-reduce requested but no multicast mapping exists");
  if (group_size(gid) > 1) check_extent(a.buf_off, a.elems * (uint64_t)dtype_size(a.dtype), "all-reduce working buffer");
  begin_call(gid, &a.g, stream, in_staging(a.buf_off));
  PCCL_CUDA(launch_all_reduce(a, clamp_lanes(nlanes, groups_[gid]), stream));
}

void Comm::all_reduce_rsag(int gid, AllReduceRsAgArgs a, int nlanes, cudaStream_t stream) {
  if (a.rs.algo != a.ag.algo || (a.rs.algo != kRing && a.rs.algo != kRecursive))
    throw Error("the two-phase all-reduce runs the ring or the recursive schedules");
  if (a.rs.algo == kRecursive && !is_pow2(group_size(gid))) throw Error("recursive halving/doubling needs a power-of-two group");
  {
    const uint64_t P = (uint64_t)group_size(gid);
    check_extent(a.rs.stage_off, (P - 1) * a.rs.sub_elems * (uint64_t)dtype_size(a.rs.wire_dtype), "all-reduce staging of partial sums");
    check_extent(a.ag.recv_off, (P - 1) * a.ag.src_stride + a.ag.sub_bytes, "all-reduce gather landing zone");
  }
  const bool staged = in_staging(a.rs.stage_off) || in_staging(a.ag.recv_off);
  begin_call(gid, &a.rs.g, stream, staged);     // two call numbers: one per phase
  begin_call(gid, &a.ag.g, stream, staged);
  PCCL_CUDA(launch_all_reduce_rsag(a, clamp_lanes(nlanes, groups_[gid]), stream));
}

void Comm::broadcast(int gid, BroadcastArgs a, int nlanes, cudaStream_t stream) {
  if (a.use_multimem && mc_heap_ == 0) throw Error("multimem broadcast requested but no multicast mapping exists");
  if (a.root < 0 || a.root >= group_size(gid)) throw Error("broadcast root outside the group");
  if (group_size(gid) > 1) check_extent(a.buf_off, a.bytes, "broadcast buffer");
  begin_call(gid, &a.g, stream, in_staging(a.buf_off));
  PCCL_CUDA(launch_broadcast(a, clamp_lanes(nlanes, groups_[gid]), stream));
}

void Comm::barrier(int gid, cudaStream_t stream) {
  BarrierArgs a;
  begin_call(gid, &a.g, stream);
  PCCL_CUDA(launch_barrier(a, stream));
}

}  // namespace pccl
