// Collective schedules: which rank talks to which, about which blocks, at which step.
//
// Every function is __host__ __device__ so that the device kernels, the host-side
// validation code and the unit tests (which simulate all P ranks in one process) use
// the very same index arithmetic.
//
// Parity: the recursive-doubling all-gather follows pccl/src/all_gather.cpp:40-66 of the
// reference (partner r^s, nearest partner first), recursive halving follows
// pccl/src/reduce_scatter.cpp:50-96 (farthest partner first, naturally ordered result),
// ring reduce-scatter follows pccl/src/reduce_scatter.cpp:127-152.  The ring all-gather
// and the direct (all-to-all over the switch) variants do not exist in the reference.
//
// All schedules are expressed as PUSH schedules: at step t a rank writes into one
// destination's memory and expects one source to write into its own.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define PCCL_HD __host__ __device__ __forceinline__
#else
#define PCCL_HD inline
#endif

namespace pccl {

constexpr int kMaxRanks = 8;        // one NVSwitch domain
constexpr int kMaxSteps = 8;        // >= kMaxRanks - 1

enum Algo : int {
  kDirect = 0,     // every rank exchanges with all P-1 peers (bandwidth-optimal on a switch)
  kRing = 1,       // P-1 neighbour steps
  kRecursive = 2,  // log2(P) steps: doubling for all-gather, halving for reduce-scatter
  kPull = 3,       // direct, but the consumer loads from the peers' symmetric input
  kMultimem = 4,   // NVLS: multimem.st / multimem.ld_reduce through the switch
  kEager = 5,      // small messages: the direct schedule into a double-buffered landing area of the
                   // communicator, without the entry handshake (one flag trip instead of three)
};

struct Step {
  int dst;         // group index this rank writes to
  int src;         // group index that writes to this rank
  int send_first;  // first block of the contiguous block range that is sent
  int recv_first;  // first block of the contiguous block range that is received
  int nblocks;     // number of blocks in either range
};

PCCL_HD bool is_pow2(int p) { return p > 0 && (p & (p - 1)) == 0; }

PCCL_HD int ilog2(int p) {
  int l = 0;
  while ((1 << (l + 1)) <= p) ++l;
  return l;
}

PCCL_HD int pmod(int a, int p) {
  int m = a % p;
  return m < 0 ? m + p : m;
}

// Number of push steps of an algorithm on P ranks (0 for P == 1).
PCCL_HD int num_steps(int algo, int P) {
  if (P <= 1) return 0;
  return algo == kRecursive ? ilog2(P) : P - 1;
}

// ---------------------------------------------------------------- all-gather
// Block b is rank b's contribution.  After all steps every rank holds every block.
PCCL_HD Step ag_step(int algo, int P, int r, int t) {
  Step s;
  if (algo == kRing) {
    s.dst = pmod(r + 1, P);
    s.src = pmod(r - 1, P);
    s.send_first = pmod(r - t, P);
    s.recv_first = pmod(r - t - 1, P);
    s.nblocks = 1;
  } else if (algo == kRecursive) {
    const int seg = 1 << t;
    const int partner = r ^ seg;
    s.dst = s.src = partner;
    s.send_first = (r / seg) * seg;        // the seg-aligned run of blocks gathered so far
    s.recv_first = (partner / seg) * seg;
    s.nblocks = seg;
  } else {  // direct: step t goes to the t-th next neighbour so that no two ranks hit one peer at once
    s.dst = pmod(r + 1 + t, P);
    s.src = pmod(r - 1 - t, P);
    s.send_first = r;
    s.recv_first = s.src;
    s.nblocks = 1;
  }
  return s;
}

// Does step t forward data that arrived in an earlier step (so it has to wait for it)?
PCCL_HD bool ag_step_depends_on_recv(int algo, int t) {
  return algo != kDirect && t > 0;
}

// ------------------------------------------------------------ reduce-scatter
// Block b of every rank's input is destined for rank b.  A step sends PARTIAL SUMS of the
// blocks [send_first, send_first+nblocks) and receives partial sums of
// [recv_first, recv_first+nblocks) into staging slot rs_stage_offset(t).
PCCL_HD Step rs_step(int algo, int P, int r, int t) {
  Step s;
  if (algo == kRing) {
    s.dst = pmod(r + 1, P);
    s.src = pmod(r - 1, P);
    s.send_first = pmod(r - t - 1, P);
    s.recv_first = pmod(r - t - 2, P);
    s.nblocks = 1;
  } else if (algo == kRecursive) {
    const int G = P >> t;       // size of the group still exchanging
    const int h = G >> 1;       // blocks exchanged this step
    const int base = (r / G) * G;  // first block of the active region of this rank
    if (r - base < h) {         // lower half keeps [base, base+h), sends [base+h, base+G)
      s.dst = s.src = r + h;
      s.send_first = base + h;
      s.recv_first = base;
    } else {                    // upper half keeps [base+h, base+G)
      s.dst = s.src = r - h;
      s.send_first = base;
      s.recv_first = base + h;
    }
    s.nblocks = h;
  } else {  // direct
    s.dst = pmod(r + 1 + t, P);
    s.src = pmod(r - 1 - t, P);
    s.send_first = s.dst;
    s.recv_first = r;
    s.nblocks = 1;
  }
  return s;
}

// Staging slot (in blocks) that receives the partials of step t.
PCCL_HD int rs_stage_offset(int algo, int P, int t) {
  if (algo != kRecursive) return t;
  int off = 0;
  for (int j = 0; j < t; ++j) off += P >> (j + 1);
  return off;
}

// Total staging blocks an algorithm needs on every rank: P-1 for all of them.
PCCL_HD int rs_stage_blocks(int /*algo*/, int P) { return P > 0 ? P - 1 : 0; }

// Bit j set: the partials received at step j are added into what is sent at step t
// (t == num_steps: into the final result).  Only steps whose received range covers the
// block in question contribute; the caller checks the range.
PCCL_HD unsigned rs_dep_mask(int algo, int P, int t) {
  const int n = num_steps(algo, P);
  if (algo == kRing) return t == 0 ? 0u : (1u << (t - 1));
  if (algo == kRecursive) return (1u << t) - 1u;
  return t == n ? ((1u << n) - 1u) : 0u;  // direct: raw inputs travel, summed once at the end
}

// ---------------------------------------------------------------- 2-D hierarchy
// World rank g of a grid with `intra` consecutive ranks per inner group:
// g = grid*intra*inter + outer*intra + inner   (pccl/process_groups.py:91-139 of the reference).
PCCL_HD int grid_inner_index(int g, int intra) { return g % intra; }
PCCL_HD int grid_outer_index(int g, int intra, int inter) { return (g / intra) % inter; }
PCCL_HD int grid_index(int g, int intra, int inter) { return g / (intra * inter); }
PCCL_HD int grid_world_rank(int grid, int outer, int inner, int intra, int inter) {
  return (grid * inter + outer) * intra + inner;
}

}  // namespace pccl
