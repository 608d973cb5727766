// The collective kernels.  One launch runs a whole collective: every step of the ring,
// recursive doubling/halving or direct schedule happens inside the kernel, with data
// moving over peer-mapped memory (NVLink 5 through NVSwitch) and with system-scope flags
// in place of the per-step host synchronisation + MPI_Sendrecv of the reference
// (pccl/src/all_gather.cpp:41-66, pccl/src/reduce_scatter.cpp:50-89 and :127-146).
//
// Work is split into LANES: lane c (= blockIdx.x) of every rank handles the same byte or
// element range of every block, and only ever synchronises with lane c of its peers.
// Lanes never synchronise with one another, so a grid needs no grid-wide barrier and the
// kernels are persistent with at most one CTA per SM.
//
// Bulk data moves through the SM's copy engine (cp.async.bulk through a ring of shared
// memory stages, bulk.cuh): few lanes keep NVLink busy and the other SMs stay free for the
// GEMMs of the training step.  Ranges that are not 16-byte aligned use the load/store
// loops of primitives.cuh.
//
// The reference's fp32 vectorAdd launch per step (pccl/src/common.cu:5-19) does not exist
// here: partial sums are formed in fp32 registers while the data is on its way.
#include <cuda_runtime.h>

#include "bulk.cuh"
#include "launch.h"
#include "primitives.cuh"

namespace pccl {

namespace {

__device__ __forceinline__ int step_kind(int algo, int t) { return kSlotStep0 + (algo == kDirect ? 0 : t); }

// Below this many bytes per lane the copy-engine pipeline costs more (barrier set-up, first
// load latency) than it saves; the thread loops take over.
constexpr uint64_t kBulkMinBytes = 192 * 1024;

// Copy one range to ndst destinations: copy engine when aligned, thread loops otherwise.
template <bool REMOTE_SRC>
__device__ __forceinline__ bool lane_copy(BulkPipe& pipe, char* const* dsts, int ndst, const char* src, uint64_t len) {
  if (len == 0 || ndst == 0) return true;
  bool aligned = (reinterpret_cast<uintptr_t>(src) & 15u) == 0 && len >= kBulkMinBytes;
  for (int d = 0; d < ndst; ++d) aligned = aligned && (reinterpret_cast<uintptr_t>(dsts[d]) & 15u) == 0;
  uint64_t done = 0;
  if (aligned) {
    done = len & ~(uint64_t)15;
    if (!cta_bulk_copy(pipe, dsts, ndst, src, done)) return false;
  }
  if (done < len) {
    char* rest[kMaxRanks + 1];
    int nr = 0;
    for (int d = 0; d < ndst; ++d)
      if (dsts[d] != src) rest[nr++] = dsts[d] + done;
    cta_copy_multi<REMOTE_SRC>(rest, nr, src + done, len - done);
  }
  return true;
}
template <bool REMOTE_SRC>
__device__ __forceinline__ bool lane_copy1(BulkPipe& pipe, char* dst, const char* src, uint64_t len) {
  if (dst == src) return true;
  char* d[1] = {dst};
  return lane_copy<REMOTE_SRC>(pipe, d, 1, src, len);
}

// Publish a flag after data: first make sure the copy engine's stores have been performed.
__device__ __forceinline__ void publish_mask(const GroupDev& g, const LaneCtx& c, int kind, unsigned mask) {
  cta_bulk_flush();
  cta_signal_mask(g, c, kind, mask);
}
__device__ __forceinline__ void publish(const GroupDev& g, const LaneCtx& c, int kind, int dst) {
  publish_mask(g, c, kind, 1u << dst);
}

// ============================================================================ all-gather
// The whole all-gather as a device function, so that a kernel can run it after another phase
// (the two-phase all-reduce below).  `gran`: bytes a lane's range is a multiple of; `coll`: the
// collective the status word names when a wait gives up.
__device__ __forceinline__ void all_gather_body(const AllGatherArgs& a, BulkPipe& pipe, uint64_t gran, uint32_t coll) {
  const GroupDev& g = a.g;
  const int P = g.size;
  const LaneCtx c{(int)blockIdx.y, g.first_local + (int)blockIdx.y, (int)blockIdx.x, coll};
  const int me = c.me;
  uint64_t lo, hi;
  lane_range(a.sub_bytes, gran, c.lane, gridDim.x, &lo, &hi);
  const uint64_t len = hi - lo;
  if (len == 0) return;  // the same lane is empty on every rank
  const int algo = a.algo;
  char* mine = g.heap[me] + a.recv_off;
  const char* in = a.in[c.li];
  char* out = a.out[c.li];
  const unsigned others = others_mask(P, me);

  auto pos = [&](int s, int j) -> uint64_t { return (uint64_t)s * a.src_stride + (uint64_t)j * a.sub_stride + lo; };
  auto opos = [&](int s, int j) -> uint64_t {
    return (uint64_t)s * a.out_src_stride + (uint64_t)j * a.out_sub_stride + lo;
  };
  // This rank's own contribution: the private input, else (kPull) its slot at in_off, else
  // its block of the landing zone (in-place call).
  auto own = [&](int j) -> const char* {
    if (in != nullptr) return in + (uint64_t)j * a.in_sub_stride + lo;
    if (algo == kPull) return g.heap[me] + a.in_off + (uint64_t)j * a.in_sub_stride + lo;
    return mine + pos(me, j);
  };

  if (P == 1) {
    for (int j = 0; j < a.nsub; ++j) {
      char* d = out != nullptr ? out + opos(0, j) : mine + pos(0, j);
      if (!lane_copy1<false>(pipe, d, own(j), len)) return;
    }
    cta_bulk_flush();
    return;
  }

  if (algo == kPull) {
    // Contributions sit at in_off of every heap; consumers load them.
    char* stage = g.heap[me] + a.in_off;
    if (in != nullptr) {
      for (int j = 0; j < a.nsub; ++j)
        if (!lane_copy1<false>(pipe, stage + (uint64_t)j * a.in_sub_stride + lo, own(j), len)) return;
    }
    publish_mask(g, c, kSlotEntry, others);
    for (int j = 0; j < a.nsub; ++j) {
      char* d = out != nullptr ? out + opos(me, j) : mine + pos(me, j);
      if (!lane_copy1<false>(pipe, d, own(j), len)) return;
    }
    for (int k = 1; k < P; ++k) {
      const int p = pmod(me + k, P);
      if (!cta_wait(g, c, kSlotEntry, p)) return;
      const char* theirs = g.heap[p] + a.in_off;
      for (int j = 0; j < a.nsub; ++j) {
        char* d = out != nullptr ? out + opos(p, j) : mine + pos(p, j);
        if (!lane_copy1<true>(pipe, d, theirs + (uint64_t)j * a.in_sub_stride + lo, len)) return;
      }
    }
    publish_mask(g, c, kSlotExit, others);     // flush: our loads of their memory are complete
    cta_wait_mask(g, c, kSlotExit, others);
    return;
  }

  if (algo == kMultimem) {
    // One multimem.st per 16 bytes lands in every member's landing zone (own included).
    cta_signal_mask(g, c, kSlotEntry, others);
    if (!cta_wait_mask(g, c, kSlotEntry, others)) return;
    for (int j = 0; j < a.nsub; ++j) {
      const char* s = own(j);
      char* d = g.mc_heap + a.recv_off + pos(me, j);
      const uint64_t nvec = len >> 4;
      constexpr int U = 8;
      const uint64_t nt = blockDim.x;
      uint64_t i = threadIdx.x;
      for (; i + (U - 1) * nt < nvec; i += U * nt) {
        uint4 v[U];
#pragma unroll
        for (int k = 0; k < U; ++k) v[k] = ld_v4(s + ((i + k * nt) << 4));
#pragma unroll
        for (int k = 0; k < U; ++k) multimem_st_v4(d + ((i + k * nt) << 4), v[k]);
      }
      for (; i < nvec; i += nt) multimem_st_v4(d + (i << 4), ld_v4(s + (i << 4)));
    }
    cta_signal_mask(g, c, kSlotStep0, others);
    if (!cta_wait_mask(g, c, kSlotStep0, others)) return;
  } else if (algo == kDirect) {
    // One pass over the own block feeds every peer (and the local copies) from one staging read.
    // Eager calls land in the half of the eager area that no peer can still be reading (it was last
    // used two eager calls ago, and every peer has since been seen in the call in between), so they
    // need no handshake before the first store.
    if (!a.eager) {
      cta_signal_mask(g, c, kSlotEntry, others);
      if (!cta_wait_mask(g, c, kSlotEntry, others)) return;
    }
    for (int j = 0; j < a.nsub; ++j) {
      char* dsts[kMaxRanks + 1];
      int nd = 0;
      for (int k = 1; k < P; ++k) dsts[nd++] = g.heap[pmod(me + k, P)] + a.recv_off + pos(me, j);
      if (in != nullptr) dsts[nd++] = mine + pos(me, j);
      if (out != nullptr) dsts[nd++] = out + opos(me, j);
      if (!lane_copy<false>(pipe, dsts, nd, own(j), len)) return;
    }
    publish_mask(g, c, kSlotStep0, others);
    if (!cta_wait_mask(g, c, kSlotStep0, others)) return;
  } else {
    // Ring and recursive doubling: forward what has arrived.
    if (in != nullptr)
      for (int j = 0; j < a.nsub; ++j)
        if (!lane_copy1<false>(pipe, mine + pos(me, j), own(j), len)) return;
    publish_mask(g, c, kSlotEntry, others);      // flush: later steps read the landing zone
    unsigned entered = 0, arrived = 0;
    const int n = num_steps(algo, P);
    for (int t = 0; t < n; ++t) {
      const Step s = ag_step(algo, P, me, t);
      if (ag_step_depends_on_recv(algo, t) && !((arrived >> (t - 1)) & 1u)) {
        if (!cta_wait(g, c, step_kind(algo, t - 1), ag_step(algo, P, me, t - 1).src)) return;
        arrived |= 1u << (t - 1);
      }
      if (!((entered >> s.dst) & 1u)) {
        if (!cta_wait(g, c, kSlotEntry, s.dst)) return;
        entered |= 1u << s.dst;
      }
      char* theirs = g.heap[s.dst] + a.recv_off;
      for (int b = s.send_first; b < s.send_first + s.nblocks; ++b)
        for (int j = 0; j < a.nsub; ++j) {
          if (b == me) {
            if (!lane_copy1<false>(pipe, theirs + pos(b, j), own(j), len)) return;
          } else {
            if (!lane_copy1<true>(pipe, theirs + pos(b, j), mine + pos(b, j), len)) return;
          }
        }
      publish(g, c, step_kind(algo, t), s.dst);
    }
    for (int t = 0; t < n; ++t)
      if (!((arrived >> t) & 1u))
        if (!cta_wait(g, c, step_kind(algo, t), ag_step(algo, P, me, t).src)) return;
  }

  if (out != nullptr) {
    for (int s = 0; s < P; ++s)
      for (int j = 0; j < a.nsub; ++j) {
        if (s == me) {
          if (algo != kDirect && !lane_copy1<false>(pipe, out + opos(s, j), own(j), len)) return;
        } else {
          if (!lane_copy1<true>(pipe, out + opos(s, j), mine + pos(s, j), len)) return;
        }
      }
  }
  cta_bulk_flush();
}

__global__ void __launch_bounds__(kCollThreads, 1) all_gather_kernel(const __grid_constant__ AllGatherArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  BulkPipe pipe;
  bulk_pipe_init(pipe, smem, a.g.timeout_ns);
  all_gather_body(a, pipe, 16, kCollAllGather);
}

// ============================================================================ reduce-scatter
// Sum nsrc sources (first one of type TA, the rest TW) into one destination.
template <int TA, int TW, int TOUT, bool REMOTE_W>
__device__ __forceinline__ bool lane_reduce(BulkPipe& pipe, char* out, const char* a_src, const char* const* w, int nw,
                                            uint64_t cnt, float scale) {
  constexpr uint64_t SA = Elem<TA>::size, SO = Elem<TOUT>::size;
  uint64_t done = 0;
  if constexpr (TA == TW) {
    bool aligned = cnt * SA >= kBulkMinBytes && (reinterpret_cast<uintptr_t>(out) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(a_src) & 15u) == 0;
    for (int k = 0; k < nw; ++k) aligned = aligned && (reinterpret_cast<uintptr_t>(w[k]) & 15u) == 0;
    if (aligned) {
      const char* srcs[kMaxReduceSrc + 1];
      int ns = 0;
      srcs[ns++] = a_src;
      for (int k = 0; k < nw; ++k) srcs[ns++] = w[k];
      done = cnt & ~(uint64_t)7;
      char* o[1] = {out};
      if (!cta_bulk_reduce<TA, TOUT>(pipe, o, 1, srcs, ns, done, scale)) return false;
    }
  }
  if (done < cnt) {
    const char* wt[kMaxReduceSrc];
    for (int k = 0; k < nw; ++k) wt[k] = w[k] + done * Elem<TW>::size;
    char* o = out + done * SO;
    cta_reduce<TA, TW, TOUT, REMOTE_W>(&o, 1, a_src + done * SA, wt, nw, cnt - done, scale);
  }
  return true;
}

template <int TIN, int TW, int TOUT>
__device__ __forceinline__ void reduce_scatter_body(const ReduceScatterArgs& a, BulkPipe& pipe, uint32_t coll) {
  const GroupDev& g = a.g;
  const int P = g.size;
  const LaneCtx c{(int)blockIdx.y, g.first_local + (int)blockIdx.y, (int)blockIdx.x, coll};
  const int me = c.me;
  uint64_t lo, hi;
  lane_range(a.sub_elems, 8, c.lane, gridDim.x, &lo, &hi);
  const uint64_t cnt = hi - lo;
  if (cnt == 0) return;
  const int algo = a.algo;
  const char* in = a.in[c.li] != nullptr ? a.in[c.li] : g.heap[me] + a.in_off;
  char* out = a.out[c.li];
  const unsigned others = others_mask(P, me);
  constexpr uint64_t SI = Elem<TIN>::size, SW = Elem<TW>::size, SO = Elem<TOUT>::size;

  auto in_ptr = [&](const char* base, int d, int j) -> const char* {
    return base + (uint64_t)d * a.dst_stride + (uint64_t)j * a.sub_stride + lo * SI;
  };
  auto out_ptr = [&](int j) -> char* { return out + (uint64_t)j * a.out_sub_stride + lo * SO; };
  auto stage_ptr = [&](int rank, int slot, int j) -> char* {
    return g.heap[rank] + a.stage_off + (((uint64_t)slot * a.nsub + j) * a.sub_elems + lo) * SW;
  };

  if (P == 1) {
    for (int j = 0; j < a.nsub; ++j) {
      char* o = out_ptr(j);
      cta_reduce<TIN, TIN, TOUT, false>(&o, 1, in_ptr(in, 0, j), nullptr, 0, cnt, a.scale);
    }
    return;
  }

  if (algo == kPull) {
    // Every member's input sits at in_off of its heap; load block `me` from all of them.
    cta_signal_mask(g, c, kSlotEntry, others);
    if (!cta_wait_mask(g, c, kSlotEntry, others)) return;
    for (int j = 0; j < a.nsub; ++j) {
      const char* w[kMaxReduceSrc];
      int nw = 0;
      for (int k = 1; k < P; ++k) w[nw++] = in_ptr(g.heap[pmod(me + k, P)] + a.in_off, me, j);
      if (!lane_reduce<TIN, TIN, TOUT, true>(pipe, out_ptr(j), in_ptr(in, me, j), w, nw, cnt, a.scale)) return;
    }
    cta_signal_mask(g, c, kSlotExit, others);
    cta_wait_mask(g, c, kSlotExit, others);
    return;
  }

  if (algo == kMultimem) {
    // The switch adds the P copies (fp32 accumulation) and returns one vector.
    cta_signal_mask(g, c, kSlotEntry, others);
    if (!cta_wait_mask(g, c, kSlotEntry, others)) return;
    constexpr int EPV = 16 / (int)SI;  // elements per 16-byte vector
    for (int j = 0; j < a.nsub; ++j) {
      const char* src = in_ptr(g.mc_heap + a.in_off, me, j);
      char* o = out_ptr(j);
      const uint64_t nvec = cnt / EPV;
      auto emit = [&](uint64_t i, const uint4& v) {
        float f[8];
        if constexpr (TIN == kF32) {
          f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
        } else {
          Elem<TIN>::unpack(v, f);
        }
#pragma unroll
        for (int e = 0; e < EPV; ++e) f[e] *= a.scale;
        char* dst = o + i * EPV * SO;
        if constexpr (TOUT == kF32) {
          st_v4(dst, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
          if constexpr (EPV == 8)
            st_v4(dst + 16, make_uint4(__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])));
        } else if constexpr (EPV == 8) {
          st_v4(dst, Elem<TOUT>::pack(f));
        } else {
#pragma unroll
          for (int e = 0; e < EPV; ++e) Elem<TOUT>::store1(dst + e * SO, f[e]);
        }
      };
      constexpr int U = 8;     // switch-side reductions in flight per thread
      const uint64_t nt = blockDim.x;
      uint64_t i = threadIdx.x;
      for (; i + (U - 1) * nt < nvec; i += U * nt) {
        uint4 v[U];
#pragma unroll
        for (int k = 0; k < U; ++k) v[k] = multimem_ld_reduce_v4<TIN>(src + ((i + k * nt) << 4));
#pragma unroll
        for (int k = 0; k < U; ++k) emit(i + k * nt, v[k]);
      }
      for (; i < nvec; i += nt) emit(i, multimem_ld_reduce_v4<TIN>(src + (i << 4)));
    }
    cta_signal_mask(g, c, kSlotExit, others);
    cta_wait_mask(g, c, kSlotExit, others);
    return;
  }

  // Push schedules: partial sums travel in the wire dtype, fp32 in registers.  Eager calls (direct
  // schedule into this call's half of the eager area) skip the entry handshake.
  if (!a.eager) cta_signal_mask(g, c, kSlotEntry, others);
  unsigned entered = a.eager ? ~0u : 0u, arrived = 0;
  const int n = num_steps(algo, P);
  for (int t = 0; t <= n; ++t) {
    const unsigned deps = rs_dep_mask(algo, P, t);
    if (algo == kDirect && t == n) {
      if (!cta_wait_mask(g, c, kSlotStep0, others)) return;
      arrived = (1u << n) - 1u;
    } else {
      for (int jd = 0; jd < n; ++jd)
        if (((deps >> jd) & 1u) && !((arrived >> jd) & 1u)) {
          if (!cta_wait(g, c, step_kind(algo, jd), rs_step(algo, P, me, jd).src)) return;
          arrived |= 1u << jd;
        }
    }
    Step s;
    if (t < n) {
      s = rs_step(algo, P, me, t);
      if (!((entered >> s.dst) & 1u)) {
        if (!cta_wait(g, c, kSlotEntry, s.dst)) return;
        entered |= 1u << s.dst;
      }
    } else {
      s.dst = me; s.src = me; s.send_first = me; s.recv_first = me; s.nblocks = 1;
    }
    for (int b = s.send_first; b < s.send_first + s.nblocks; ++b)
      for (int j = 0; j < a.nsub; ++j) {
        const char* w[kMaxReduceSrc];
        int nw = 0;
        for (int jd = 0; jd < n; ++jd)
          if ((deps >> jd) & 1u) {
            const Step sj = rs_step(algo, P, me, jd);
            if (b >= sj.recv_first && b < sj.recv_first + sj.nblocks)
              w[nw++] = stage_ptr(me, rs_stage_offset(algo, P, jd) + (b - sj.recv_first), j);
          }
        if (t < n) {
          char* d = stage_ptr(s.dst, rs_stage_offset(algo, P, t) + (b - s.send_first), j);
          if (nw == 0 && TW == TIN) {
            if (!lane_copy1<false>(pipe, d, in_ptr(in, b, j), cnt * SI)) return;
          } else {
            cta_reduce<TIN, TW, TW, true>(&d, 1, in_ptr(in, b, j), w, nw, cnt, 1.0f);
          }
        } else {
          if (!lane_reduce<TIN, TW, TOUT, true>(pipe, out_ptr(j), in_ptr(in, b, j), w, nw, cnt, a.scale)) return;
        }
      }
    if (t < n) publish(g, c, step_kind(algo, t), s.dst);
  }
}

template <int TIN, int TW, int TOUT>
__global__ void __launch_bounds__(kCollThreads, 1) reduce_scatter_kernel(const __grid_constant__ ReduceScatterArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  BulkPipe pipe;
  bulk_pipe_init(pipe, smem, a.g.timeout_ns);
  reduce_scatter_body<TIN, TW, TOUT>(a, pipe, kCollReduceScatter);
}

// ============================================================================ all-reduce = reduce-scatter + all-gather
// The composition the reference's all-reduce uses (pccl/src/yacl.cpp:146-177: reduce-scatter into
// a temporary, all-gather back; recursive halving + recursive doubling, or ring + ring), as ONE
// launch: phase one leaves this rank's block of the sum in its slot of the tensor, phase two is
// the all-gather of those slots with the same schedule family.  The two phases are two calls as
// far as the flags go (consecutive call numbers), so a step flag of phase one can never be taken
// for one of phase two; a peer's block is pushed into this rank's tensor only after this rank has
// signalled its entry into phase two, that is after it has read all of its own input.
// Lanes keep the same element range in both phases (lane ranges are multiples of 8 elements).
template <int DT>
__global__ void __launch_bounds__(kCollThreads, 1) all_reduce_rsag_kernel(const __grid_constant__ AllReduceRsAgArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  BulkPipe pipe;
  bulk_pipe_init(pipe, smem, a.rs.g.timeout_ns);
  reduce_scatter_body<DT, DT, DT>(a.rs, pipe, kCollAllReduce);
  cta_bulk_flush();          // the block written by phase one is what phase two sends
  __syncthreads();
  all_gather_body(a.ag, pipe, 8 * Elem<DT>::size, kCollAllReduce);
}

// ============================================================================ all-reduce
// Two-shot in one kernel: member r reduces slice r (loading it from every heap) and writes
// the result back into slice r of every heap; nobody else touches slice r, so the
// operation is in place.  The composition reduce-scatter + all-gather is what
// pccl/src/yacl.cpp:146-177 of the reference does with two temporaries and two host loops.
template <int DT>
__global__ void __launch_bounds__(kCollThreads, 1) all_reduce_kernel(const __grid_constant__ AllReduceArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const GroupDev& g = a.g;
  const int P = g.size;
  const LaneCtx c{(int)blockIdx.y, g.first_local + (int)blockIdx.y, (int)blockIdx.x, kCollAllReduce};
  const int me = c.me;
  constexpr uint64_t S = Elem<DT>::size;
  const uint64_t per = (((a.elems + P - 1) / P) + 7) / 8 * 8;  // slice length, multiple of 8 elements
  char* data = a.data[c.li];
  char* buf = g.heap[me] + a.buf_off;
  const unsigned others = others_mask(P, me);
  BulkPipe pipe;
  bulk_pipe_init(pipe, smem, g.timeout_ns);

  auto slice = [&](int s, uint64_t* lo, uint64_t* cnt) {
    uint64_t b = (uint64_t)s * per, e = b + per;
    if (b > a.elems) b = a.elems;
    if (e > a.elems) e = a.elems;
    uint64_t l, h;
    lane_range(e - b, 8, c.lane, gridDim.x, &l, &h);
    *lo = b + l;
    *cnt = h - l;
  };

  if (P == 1) {
    uint64_t lo, cnt;
    slice(0, &lo, &cnt);
    char* p = (data != nullptr ? data : buf) + lo * S;
    if (a.scale != 1.0f) cta_reduce<DT, DT, DT, false>(&p, 1, p, nullptr, 0, cnt, a.scale);
    return;
  }

  if (data != nullptr)
    for (int s = 0; s < P; ++s) {
      uint64_t lo, cnt;
      slice(s, &lo, &cnt);
      if (!lane_copy1<false>(pipe, buf + lo * S, data + lo * S, cnt * S)) return;
    }
  publish_mask(g, c, kSlotEntry, others);
  if (!cta_wait_mask(g, c, kSlotEntry, others)) return;

  uint64_t lo, cnt;
  slice(me, &lo, &cnt);
  if (a.algo == kMultimem) {
    constexpr int EPV = 16 / (int)S;
    char* mc = g.mc_heap + a.buf_off + lo * S;
    const uint64_t nvec = cnt / EPV;
    for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
      uint4 v = multimem_ld_reduce_v4<DT>(mc + (i << 4));
      if (a.scale != 1.0f) {
        if constexpr (DT == kF32) {
          v.x = __float_as_uint(__uint_as_float(v.x) * a.scale); v.y = __float_as_uint(__uint_as_float(v.y) * a.scale);
          v.z = __float_as_uint(__uint_as_float(v.z) * a.scale); v.w = __float_as_uint(__uint_as_float(v.w) * a.scale);
        } else {
          float f[8];
          Elem<DT>::unpack(v, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] *= a.scale;
          v = Elem<DT>::pack(f);
        }
      }
      multimem_st_v4(mc + (i << 4), v);
    }
  } else {
    const char* w[kMaxReduceSrc];
    char* outs[kMaxRanks];
    int nw = 0, no = 0;
    outs[no++] = buf + lo * S;
    for (int k = 1; k < P; ++k) {
      const int p = pmod(me + k, P);
      w[nw++] = g.heap[p] + a.buf_off + lo * S;
      outs[no++] = g.heap[p] + a.buf_off + lo * S;
    }
    cta_reduce<DT, DT, DT, true>(outs, no, buf + lo * S, w, nw, cnt, a.scale);
  }
  cta_signal_mask(g, c, kSlotStep0, others);
  if (!cta_wait_mask(g, c, kSlotStep0, others)) return;

  if (data != nullptr)
    for (int s = 0; s < P; ++s) {
      uint64_t l2, c2;
      slice(s, &l2, &c2);
      if (!lane_copy1<true>(pipe, data + l2 * S, buf + l2 * S, c2 * S)) return;
    }
  cta_bulk_flush();
}

// ============================================================================ broadcast
__global__ void __launch_bounds__(kCollThreads, 1) broadcast_kernel(const __grid_constant__ BroadcastArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const GroupDev& g = a.g;
  const int P = g.size;
  const LaneCtx c{(int)blockIdx.y, g.first_local + (int)blockIdx.y, (int)blockIdx.x, kCollBroadcast};
  const int me = c.me;
  if (P == 1) return;
  uint64_t lo, hi;
  lane_range(a.bytes, 16, c.lane, gridDim.x, &lo, &hi);
  const uint64_t len = hi - lo;
  if (len == 0) return;
  BulkPipe pipe;
  bulk_pipe_init(pipe, smem, g.timeout_ns);
  char* data = a.data[c.li];
  char* buf = g.heap[me] + a.buf_off;
  const unsigned others = others_mask(P, me);
  if (me == a.root) {
    const char* src = data != nullptr ? data : buf;
    if (!cta_wait_mask(g, c, kSlotEntry, others)) return;
    if (a.use_multimem) {
      char* mc = g.mc_heap + a.buf_off + lo;
      for (uint64_t i = threadIdx.x; i < (len >> 4); i += blockDim.x) multimem_st_v4(mc + (i << 4), ld_v4(src + lo + (i << 4)));
    } else {
      char* dsts[kMaxRanks];
      int nd = 0;
      for (int k = 1; k < P; ++k) dsts[nd++] = g.heap[pmod(me + k, P)] + a.buf_off + lo;
      if (!lane_copy<false>(pipe, dsts, nd, src + lo, len)) return;
    }
    publish_mask(g, c, kSlotStep0, others);
  } else {
    cta_signal(g, c, kSlotEntry, a.root);
    if (!cta_wait(g, c, kSlotStep0, a.root)) return;
    if (data != nullptr && !lane_copy1<true>(pipe, data + lo, buf + lo, len)) return;
    cta_bulk_flush();
  }
}

// ============================================================================ barrier
__global__ void __launch_bounds__(64, 1) barrier_kernel(const __grid_constant__ BarrierArgs a) {
  const GroupDev& g = a.g;
  const LaneCtx c{(int)blockIdx.y, g.first_local + (int)blockIdx.y, 0, kCollBarrier};
  if (g.size == 1) return;
  const unsigned others = others_mask(g.size, c.me);
  cta_signal_mask(g, c, kSlotEntry, others);
  cta_wait_mask(g, c, kSlotEntry, others);
}

template <typename Args>
cudaError_t launch(void (*kernel)(const Args), const Args& args, int nlanes, int threads, size_t smem, cudaStream_t stream) {
  dim3 grid(nlanes, args.g.nlocal), block(threads);
  if (smem > 48 * 1024) {
    // once per kernel and device (the attribute belongs to the function in the current context)
    static thread_local const void* configured[64] = {nullptr};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || configured[dev] != reinterpret_cast<const void*>(kernel)) {
      cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) configured[dev] = reinterpret_cast<const void*>(kernel);
    }
  }
  if (args.g.nlocal > 1) {
    // Several ranks in one launch wait on one another: every CTA must be resident.
    void* params[] = {const_cast<Args*>(&args)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, params, smem, stream);
  }
  kernel<<<grid, block, smem, stream>>>(args);
  return cudaGetLastError();
}

// The two-phase kernel carries two argument blocks; its group geometry is that of the first.
cudaError_t launch_rsag(void (*kernel)(const AllReduceRsAgArgs), const AllReduceRsAgArgs& args, int nlanes, cudaStream_t stream) {
  dim3 grid(nlanes, args.rs.g.nlocal), block(kCollThreads);
  static thread_local const void* configured[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || configured[dev] != reinterpret_cast<const void*>(kernel)) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kBulkSmemBytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = reinterpret_cast<const void*>(kernel);
  }
  if (args.rs.g.nlocal > 1) {
    void* params[] = {const_cast<AllReduceRsAgArgs*>(&args)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, params, kBulkSmemBytes, stream);
  }
  kernel<<<grid, block, kBulkSmemBytes, stream>>>(args);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_all_gather(const AllGatherArgs& a, int nlanes, cudaStream_t stream) {
  return launch(all_gather_kernel, a, nlanes, kCollThreads, kBulkSmemBytes, stream);
}

#define PCCL_RS_CASE(TI, TW_, TO)                                                              \
  if (a.in_dtype == TI && a.wire_dtype == TW_ && a.out_dtype == TO)                            \
    return launch(reduce_scatter_kernel<TI, TW_, TO>, a, nlanes, kCollThreads, kBulkSmemBytes, stream);

cudaError_t launch_reduce_scatter(const ReduceScatterArgs& a, int nlanes, cudaStream_t stream) {
  PCCL_RS_CASE(kBF16, kBF16, kBF16)
  PCCL_RS_CASE(kBF16, kBF16, kF32)
  PCCL_RS_CASE(kBF16, kF32, kBF16)
  PCCL_RS_CASE(kBF16, kF32, kF32)
  PCCL_RS_CASE(kF16, kF16, kF16)
  PCCL_RS_CASE(kF16, kF16, kF32)
  PCCL_RS_CASE(kF16, kF32, kF16)
  PCCL_RS_CASE(kF16, kF32, kF32)
  PCCL_RS_CASE(kF32, kF32, kF32)
  PCCL_RS_CASE(kF32, kF32, kBF16)
  return cudaErrorInvalidValue;
}

cudaError_t launch_all_reduce(const AllReduceArgs& a, int nlanes, cudaStream_t stream) {
  if (a.dtype == kBF16) return launch(all_reduce_kernel<kBF16>, a, nlanes, kCollThreads, kBulkSmemBytes, stream);
  if (a.dtype == kF16) return launch(all_reduce_kernel<kF16>, a, nlanes, kCollThreads, kBulkSmemBytes, stream);
  if (a.dtype == kF32) return launch(all_reduce_kernel<kF32>, a, nlanes, kCollThreads, kBulkSmemBytes, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_all_reduce_rsag(const AllReduceRsAgArgs& a, int nlanes, cudaStream_t stream) {
  const int dt = a.rs.in_dtype;
  if (dt == kBF16) return launch_rsag(all_reduce_rsag_kernel<kBF16>, a, nlanes, stream);
  if (dt == kF16) return launch_rsag(all_reduce_rsag_kernel<kF16>, a, nlanes, stream);
  if (dt == kF32) return launch_rsag(all_reduce_rsag_kernel<kF32>, a, nlanes, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_broadcast(const BroadcastArgs& a, int nlanes, cudaStream_t stream) {
  return launch(broadcast_kernel, a, nlanes, kCollThreads, kBulkSmemBytes, stream);
}

cudaError_t launch_barrier(const BarrierArgs& a, cudaStream_t stream) {
  return launch(barrier_kernel, a, 1, 64, 0, stream);
}

int max_resident_lanes(int device) {
  int sms = 0, per_sm = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  if (cudaFuncSetAttribute(reinterpret_cast<const void*>(all_gather_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)kBulkSmemBytes) != cudaSuccess)
    return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, all_gather_kernel, kCollThreads, kBulkSmemBytes) != cudaSuccess)
    return 0;
  int m = sms * (per_sm > 0 ? 1 : 0);  // the kernels are written for one CTA per SM
  return m > kMaxLanes ? kMaxLanes : m;
}

}  // namespace pccl
