// Plain-old-data structures shared by host code and device kernels.
//
// A collective call is ONE kernel launch.  Its argument block carries, for every rank of
// the group, the base address of that rank's symmetric heap and of its signal pad as seen
// from the launching process (peer-mapped over NVLink, or plain local pointers when
// several ranks are emulated on one GPU), so the kernel itself performs every step of the
// algorithm: no host loop, no per-step synchronisation with the CPU as in
// pccl/src/all_gather.cpp:41-66 or pccl/src/reduce_scatter.cpp:50-89 of the reference.
#pragma once
#include <stdint.h>

#include "schedule.h"

namespace pccl {

// ------------------------------------------------------------------ signal pad layout
// One region per group.  slot(lane, kind, src) is written by group member `src`
// (lane `lane` of its kernel) and only ever read by the owner of the pad.
constexpr int kMaxLanes = 160;              // >= 148 SMs: at most one lane per SM
constexpr int kSlotEntry = 0;               // "my lane has entered call #epoch"
constexpr int kSlotExit = 1;                // "my lane no longer reads your memory"
constexpr int kSlotStep0 = 2;               // arrival of step t: kSlotStep0 + t
constexpr int kSlotKinds = 2 + kMaxSteps + 2;   // 12, two spare kinds for fused kernels
constexpr int kSlotPanel = 2 + kMaxSteps;       // fused all-gather+GEMM: panel arrival
constexpr uint32_t kRegionWords = kMaxLanes * kSlotKinds * kMaxRanks;
constexpr uint64_t kRegionBytes = uint64_t(kRegionWords) * 4;

PCCL_HD uint32_t slot_index(int lane, int kind, int src) {
  return (uint32_t(lane) * kSlotKinds + uint32_t(kind)) * kMaxRanks + uint32_t(src);
}

// ------------------------------------------------------------------ status word
// Lives in pinned, host-mapped memory; written by the first lane that gives up.
enum StatusCode : uint32_t {
  kStatusOk = 0,
  kStatusTimeout = 1,      // a bounded wait ran out
  kStatusPoisoned = 2,     // gave up because another lane had already failed
  kStatusBadArgs = 3,
};

struct Status {
  uint32_t code;       // StatusCode, claimed with atomicCAS
  uint32_t epoch;      // call number within the group
  int32_t rank;        // group index of the waiting rank
  int32_t peer;        // group index it was waiting for
  int32_t lane;
  int32_t slot_kind;   // kSlotEntry / kSlotExit / kSlotStep0+t
  uint32_t seen;       // flag value last read
  uint32_t collective; // CollectiveId
};

enum CollectiveId : uint32_t {
  kCollAllGather = 1,
  kCollReduceScatter = 2,
  kCollAllReduce = 3,
  kCollBroadcast = 4,
  kCollBarrier = 5,
  kCollAgGemm = 6,
  kCollWaitProbe = 7,
};

// ------------------------------------------------------------------ optional device-side trace
// One record per synchronisation point a lane passed (a completed wait or a published flag), in
// the order the records were claimed.  The buffer is plain device memory read back on request.
struct TraceEvent {
  uint64_t t_ns;       // %globaltimer
  uint32_t epoch;      // call number within the group
  uint16_t lane;
  uint8_t rank;        // group index of the lane's rank
  uint8_t what;        // bits 0-5: slot kind; bit 6: signal (else wait); bit 7: reserved
  uint32_t collective; // CollectiveId
  uint32_t pad;
};
struct TraceBuf {
  unsigned long long count;   // records claimed so far (may exceed capacity: the rest was dropped)
  uint32_t capacity;
  uint32_t pad;
  TraceEvent ev[1];           // capacity records follow
};

// ------------------------------------------------------------------ group as the kernel sees it
struct GroupDev {
  int size;                          // P
  int nlocal;                        // ranks driven by this launch: 1, or P when emulated on one GPU
  int first_local;                   // group index of blockIdx.y == 0
  uint32_t epoch;                    // call number; flags carry this value
  char* heap[kMaxRanks];             // symmetric heap base of group member i
  uint32_t* sig[kMaxRanks];          // signal region of this group inside member i's pad
  char* mc_heap;                     // multicast alias of the heaps (NVLS) or nullptr
  Status* status[kMaxRanks];         // per local rank (index by blockIdx.y); device-visible pinned memory
  uint32_t* poison[kMaxRanks];       // per local rank device word: non-zero once any lane failed
  uint64_t timeout_ns;               // time limit of every single wait
  TraceBuf* trace;                   // nullptr unless tracing is switched on
  uint32_t jitter_ns;                // stress mode: every lane sleeps a pseudo-random time below this before each wait and signal
};

enum DType : int { kBF16 = 0, kF16 = 1, kF32 = 2 };
PCCL_HD int dtype_size(int dt) { return dt == kF32 ? 4 : 2; }

// ------------------------------------------------------------------ all-gather
// Member s contributes nsub sub-blocks of sub_bytes each; sub-block j of member s lives at
//   recv_off + s*src_stride + j*sub_stride      (byte offsets inside every member's heap)
// which is how the 2-D un-permute of pccl/all_gather.py:158-159 becomes address arithmetic.
struct AllGatherArgs {
  GroupDev g;
  int algo;
  const char* in[kMaxRanks];    // per local rank: nsub*sub_bytes contiguous, or nullptr = already in place
  char* out[kMaxRanks];         // per local rank: private output to copy the result into, or nullptr
  uint64_t recv_off;            // landing zone inside the heaps (user tensor or staging)
  uint64_t out_src_stride;      // layout of the private output (same meaning as below)
  uint64_t out_sub_stride;
  uint64_t src_stride;
  uint64_t sub_stride;
  uint64_t sub_bytes;           // bytes of one sub-block handled by this launch
  uint64_t in_sub_stride;       // distance between consecutive sub-blocks of `in` (and of the kPull staging)
  int nsub;
  uint64_t in_off;              // kPull: offset of the contribution inside the owner's heap
  int eager;                    // direct schedule without the entry handshake: recv_off is the half of the eager
                                // area that this call may overwrite (see Comm::eager_half)
};

// ------------------------------------------------------------------ reduce-scatter
// Input sub-block j destined for member d lives at in + d*dst_stride + j*sub_stride (bytes).
// The result is nsub*sub_elems contiguous elements: out = cast(scale * sum over members).
struct ReduceScatterArgs {
  GroupDev g;
  int algo;
  int in_dtype, wire_dtype, out_dtype;
  const char* in[kMaxRanks];    // per local rank
  char* out[kMaxRanks];         // per local rank
  uint64_t in_off;              // kPull/kMultimem: offset of the input inside the heaps
  uint64_t stage_off;           // staging for partial sums inside the heaps (push variants)
  uint64_t dst_stride;
  uint64_t sub_stride;
  uint64_t sub_elems;           // elements of one sub-block handled by this launch
  uint64_t out_sub_stride;      // bytes between consecutive sub-blocks of `out`
  int nsub;
  float scale;
  int eager;                    // direct schedule without the entry handshake: stage_off is this call's half of the eager area
};

// ------------------------------------------------------------------ all-reduce (in place, two-shot)
struct AllReduceArgs {
  GroupDev g;
  int algo;                     // kDirect (pull-reduce + push) or kMultimem
  int dtype;
  char* data[kMaxRanks];        // per local rank: private tensor, or nullptr when it already sits at buf_off
  uint64_t buf_off;             // working buffer inside the heaps
  uint64_t elems;               // total element count (any value; slices are ceil-divided)
  float scale;
};

// All-reduce as reduce-scatter followed by all-gather in one launch (ring or recursive
// halving/doubling): the two phases with their own group blocks, i.e. their own call numbers.
struct AllReduceRsAgArgs {
  ReduceScatterArgs rs;
  AllGatherArgs ag;
};

struct BroadcastArgs {
  GroupDev g;
  int root;
  char* data[kMaxRanks];        // per local rank: private tensor or nullptr when symmetric
  uint64_t buf_off;
  uint64_t bytes;
  int use_multimem;
};

struct BarrierArgs {
  GroupDev g;
};

}  // namespace pccl
