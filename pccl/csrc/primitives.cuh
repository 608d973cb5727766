// Device-side building blocks of the collective kernels: system-scope flags with bounded
// waits, CTA-wide copies to and from peer memory, fp32-accumulating reductions and the
// NVLS multimem wrappers.
//
// Memory-ordering contract used throughout:
//   producer:  data stores (weak)  ->  bar.sync  ->  fence.acq_rel.sys + st.release.sys flag
//   consumer:  ld.acquire.sys flag (one thread)  ->  bar.sync  ->  data loads
// Flags and peer data are never read through the non-coherent (.nc) path.
// Flags carry the call number (epoch) of the group, so they are never reset and a rank
// that runs ahead by one call cannot be mistaken for the current one.
//
// The reference gets ordering from a host-side cudaEventSynchronize before every
// MPI_Sendrecv (pccl/src/all_gather.cpp:57-63); here nothing leaves the device.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "device_types.h"

namespace pccl {

constexpr int kCollThreads = 512;

// ---------------------------------------------------------------- raw accessors
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// 16-byte load that bypasses L1: used for memory that another GPU may have written.
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_v4(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st_v4(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

// ---------------------------------------------------------------- status / failure
__device__ __forceinline__ void report_failure(const GroupDev& g, int li, uint32_t code, uint32_t coll,
                                               int me, int peer, int lane, int kind, uint32_t seen) {
  Status* st = g.status[li];
  if (st != nullptr && atomicCAS(&st->code, (uint32_t)kStatusOk, code) == kStatusOk) {
    st->epoch = g.epoch;
    st->rank = me;
    st->peer = peer;
    st->lane = lane;
    st->slot_kind = kind;
    st->seen = seen;
    st->collective = coll;
    __threadfence_system();
  }
  if (g.poison[li] != nullptr) atomicExch(g.poison[li], 1u);
}

// One thread spins until flag >= epoch (wrap-safe), the time limit runs out, or the
// communicator is poisoned.  Never traps, never spins without a limit.  (Polling with relaxed
// loads and one acquire fence at the end was tried and was not faster.)
__device__ __forceinline__ bool spin_until(const uint32_t* flag, uint32_t epoch, const GroupDev& g, int li,
                                           uint32_t* seen_out) {
  uint32_t v = ld_acquire_sys(flag);
  if ((int32_t)(v - epoch) >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  const uint32_t* poison = g.poison[li];
  uint32_t it = 0;
  for (;;) {
    v = ld_acquire_sys(flag);
    if ((int32_t)(v - epoch) >= 0) return true;
    if ((++it & 63u) == 0u) {
      if (poison != nullptr && *reinterpret_cast<const volatile uint32_t*>(poison) != 0u) break;
      if (global_timer_ns() - t0 > g.timeout_ns) break;
      __nanosleep(64);
    }
  }
  *seen_out = v;
  return false;
}

struct LaneCtx {
  int li;     // local rank slot (blockIdx.y)
  int me;     // my group index
  int lane;   // blockIdx.x
  uint32_t coll;
};

// Debug hooks of every synchronisation point; both are off (two predictable branches) unless the
// communicator switched them on.  Called by one thread.
//  * stress mode: sleep a pseudo-random, bounded time, so that lanes and ranks meet their waits
//    and signals in orders a quiet machine never produces; results must not change.
//  * trace: append (time, epoch, rank, lane, slot kind, wait|signal) to the trace buffer.
__device__ __forceinline__ void debug_jitter(const GroupDev& g, const LaneCtx& c, int kind) {
  if (g.jitter_ns == 0u) return;
  uint32_t h = g.epoch * 0x9E3779B1u ^ (uint32_t)c.lane * 0x85EBCA77u ^ (uint32_t)c.me * 0xC2B2AE3Du ^ (uint32_t)kind * 0x27D4EB2Fu ^
               (uint32_t)global_timer_ns();
  h ^= h >> 15;
  h *= 0x2C1B3C6Du;
  h ^= h >> 12;
  uint32_t ns = h % g.jitter_ns;
  while (ns > 0u) {                       // at most jitter_ns in total
    const uint32_t step = ns < 500000u ? ns : 500000u;
    __nanosleep(step);
    ns -= step;
  }
}
__device__ __forceinline__ void debug_trace(const GroupDev& g, const LaneCtx& c, int kind, bool is_signal) {
  TraceBuf* tb = g.trace;
  if (tb == nullptr) return;
  const unsigned long long i = atomicAdd(&tb->count, 1ull);
  if (i < tb->capacity) {
    TraceEvent e;
    e.t_ns = global_timer_ns();
    e.epoch = g.epoch;
    e.lane = (uint16_t)c.lane;
    e.rank = (uint8_t)c.me;
    e.what = (uint8_t)((kind & 63) | (is_signal ? 64 : 0));
    e.collective = c.coll;
    e.pad = 0;
    tb->ev[i] = e;
  }
}

// All threads of the CTA call this; thread 0 waits.  Returns false (to all threads) when
// the wait gave up; the status word then says where.
__device__ __forceinline__ bool cta_wait(const GroupDev& g, const LaneCtx& c, int kind, int src) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    debug_jitter(g, c, kind);
    uint32_t seen = 0;
    const uint32_t* flag = g.sig[c.me] + slot_index(c.lane, kind, src);
    bool ok = spin_until(flag, g.epoch, g, c.li, &seen);
    if (ok) debug_trace(g, c, kind, false);
    if (!ok) {
      const bool poisoned = g.poison[c.li] != nullptr &&
                            *reinterpret_cast<const volatile uint32_t*>(g.poison[c.li]) != 0u;
      report_failure(g, c.li, poisoned ? kStatusPoisoned : kStatusTimeout, c.coll, c.me, src, c.lane, kind, seen);
    }
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  const int ok = s_ok;
  __syncthreads();
  return ok != 0;
}

// Wait for the same slot kind from every member whose bit is set in `mask`.
__device__ __forceinline__ bool cta_wait_mask(const GroupDev& g, const LaneCtx& c, int kind, unsigned mask) {
  __shared__ int s_ok_all;
  if (threadIdx.x == 0) {
    s_ok_all = 1;
    debug_jitter(g, c, kind);
  }
  __syncthreads();
  if (threadIdx.x < (unsigned)g.size && ((mask >> threadIdx.x) & 1u)) {
    uint32_t seen = 0;
    const int src = threadIdx.x;
    const uint32_t* flag = g.sig[c.me] + slot_index(c.lane, kind, src);
    if (!spin_until(flag, g.epoch, g, c.li, &seen)) {
      const bool poisoned = g.poison[c.li] != nullptr &&
                            *reinterpret_cast<const volatile uint32_t*>(g.poison[c.li]) != 0u;
      report_failure(g, c.li, poisoned ? kStatusPoisoned : kStatusTimeout, c.coll, c.me, src, c.lane, kind, seen);
      atomicExch(&s_ok_all, 0);
    }
  }
  __syncthreads();
  const int ok = s_ok_all;
  if (ok != 0 && threadIdx.x == 0) debug_trace(g, c, kind, false);
  __syncthreads();
  return ok != 0;
}

// Publish slot(lane, kind, me) = epoch in the pad of every member in `mask`.
// The leading bar.sync orders every thread's earlier stores before the release.
__device__ __forceinline__ void cta_signal_mask(const GroupDev& g, const LaneCtx& c, int kind, unsigned mask) {
  if (threadIdx.x == 0) {
    debug_jitter(g, c, kind);          // the whole CTA waits at the barrier below: the flags go out late
    debug_trace(g, c, kind, true);
  }
  __syncthreads();
  if (threadIdx.x < (unsigned)g.size && ((mask >> threadIdx.x) & 1u)) {
    __threadfence_system();
    st_release_sys(g.sig[threadIdx.x] + slot_index(c.lane, kind, c.me), g.epoch);
  }
}
__device__ __forceinline__ void cta_signal(const GroupDev& g, const LaneCtx& c, int kind, int dst) {
  cta_signal_mask(g, c, kind, 1u << dst);
}

__device__ __forceinline__ unsigned others_mask(int P, int me) { return ((1u << P) - 1u) & ~(1u << me); }

// ---------------------------------------------------------------- lane partition
// Split `total` bytes/elements into gridDim.x contiguous pieces on `gran` boundaries.
__device__ __forceinline__ void lane_range(uint64_t total, uint64_t gran, int lane, int nlanes, uint64_t* lo,
                                           uint64_t* hi) {
  const uint64_t units = (total + gran - 1) / gran;
  const uint64_t per = (units + nlanes - 1) / nlanes;
  uint64_t a = per * lane, b = a + per;
  if (a > units) a = units;
  if (b > units) b = units;
  a *= gran;
  b *= gran;
  if (a > total) a = total;
  if (b > total) b = total;
  *lo = a;
  *hi = b;
}

// ---------------------------------------------------------------- CTA-wide copy
// REMOTE_SRC: the source may have been written by another GPU during this kernel.
template <bool REMOTE_SRC>
__device__ __forceinline__ void cta_copy(char* __restrict__ dst, const char* __restrict__ src, uint64_t n) {
  if (n == 0 || dst == src) return;
  const uint64_t tid = threadIdx.x, nt = blockDim.x;
  const uintptr_t ds = reinterpret_cast<uintptr_t>(dst), ss = reinterpret_cast<uintptr_t>(src);
  if (((ds ^ ss) & 15u) == 0) {
    uint64_t head = (16 - (ss & 15u)) & 15u;
    if (head > n) head = n;
    for (uint64_t i = tid; i < head; i += nt) dst[i] = src[i];
    const uint64_t nvec = (n - head) >> 4;
    const char* s = src + head;
    char* d = dst + head;
    constexpr int U = 8;
    uint64_t i = tid;
    for (; i + (U - 1) * nt < nvec; i += U * nt) {
      uint4 v[U];
#pragma unroll
      for (int k = 0; k < U; ++k)
        v[k] = REMOTE_SRC ? ld_volatile_v4(s + ((i + k * nt) << 4)) : ld_v4(s + ((i + k * nt) << 4));
#pragma unroll
      for (int k = 0; k < U; ++k) st_v4(d + ((i + k * nt) << 4), v[k]);
    }
    for (; i < nvec; i += nt) {
      uint4 v = REMOTE_SRC ? ld_volatile_v4(s + (i << 4)) : ld_v4(s + (i << 4));
      st_v4(d + (i << 4), v);
    }
    const uint64_t done = head + (nvec << 4);
    for (uint64_t j = done + tid; j < n; j += nt) dst[j] = src[j];
  } else if (((ds | ss) & 3u) == 0 && (n & 3u) == 0) {
    const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
    uint32_t* d = reinterpret_cast<uint32_t*>(dst);
    for (uint64_t i = tid; i < (n >> 2); i += nt) d[i] = REMOTE_SRC ? ld_relaxed_sys(s + i) : s[i];
  } else {
    const volatile char* s = src;
    for (uint64_t i = tid; i < n; i += nt) dst[i] = s[i];
  }
}

// The same range to several destinations in one pass: every vector is loaded once and stored
// ndst times (a pass per destination pays the load latency ndst times, which is most of the
// time of a small all-gather to seven peers).  Falls back to a pass per destination when the
// pointers do not share their alignment within 16 bytes.
template <bool REMOTE_SRC>
__device__ __forceinline__ void cta_copy_multi(char* const* dsts, int ndst, const char* __restrict__ src, uint64_t n) {
  if (n == 0 || ndst == 0) return;
  const uintptr_t ss = reinterpret_cast<uintptr_t>(src);
  bool congruent = true;
  for (int d = 0; d < ndst; ++d) congruent = congruent && ((reinterpret_cast<uintptr_t>(dsts[d]) ^ ss) & 15u) == 0;
  if (ndst == 1 || !congruent) {
    for (int d = 0; d < ndst; ++d) cta_copy<REMOTE_SRC>(dsts[d], src, n);
    return;
  }
  const uint64_t tid = threadIdx.x, nt = blockDim.x;
  uint64_t head = (16 - (ss & 15u)) & 15u;
  if (head > n) head = n;
  for (uint64_t i = tid; i < head; i += nt) {
    const char b = src[i];
    for (int d = 0; d < ndst; ++d) dsts[d][i] = b;
  }
  const uint64_t nvec = (n - head) >> 4;
  const char* s = src + head;
  constexpr int U = 4;
  uint64_t i = tid;
  for (; i + (U - 1) * nt < nvec; i += U * nt) {
    uint4 v[U];
#pragma unroll
    for (int k = 0; k < U; ++k)
      v[k] = REMOTE_SRC ? ld_volatile_v4(s + ((i + k * nt) << 4)) : ld_v4(s + ((i + k * nt) << 4));
    for (int d = 0; d < ndst; ++d) {
      char* o = dsts[d] + head;
#pragma unroll
      for (int k = 0; k < U; ++k) st_v4(o + ((i + k * nt) << 4), v[k]);
    }
  }
  for (; i < nvec; i += nt) {
    const uint4 v = REMOTE_SRC ? ld_volatile_v4(s + (i << 4)) : ld_v4(s + (i << 4));
    for (int d = 0; d < ndst; ++d) st_v4(dsts[d] + head + (i << 4), v);
  }
  const uint64_t done = head + (nvec << 4);
  for (uint64_t j = done + tid; j < n; j += nt) {
    const char b = src[j];
    for (int d = 0; d < ndst; ++d) dsts[d][j] = b;
  }
}

// ---------------------------------------------------------------- typed 8-element vectors
template <int DT>
struct Elem;
template <>
struct Elem<kBF16> {
  static constexpr int size = 2;
  __device__ static __forceinline__ float load1(const char* p) {
    return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
  }
  __device__ static __forceinline__ void store1(char* p, float f) {
    *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(f);
  }
  __device__ static __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Elem<kF16> {
  static constexpr int size = 2;
  __device__ static __forceinline__ float load1(const char* p) {
    return __half2float(*reinterpret_cast<const __half*>(p));
  }
  __device__ static __forceinline__ void store1(char* p, float f) {
    *reinterpret_cast<__half*>(p) = __float2half_rn(f);
  }
  __device__ static __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Elem<kF32> {
  static constexpr int size = 4;
  __device__ static __forceinline__ float load1(const char* p) { return *reinterpret_cast<const float*>(p); }
  __device__ static __forceinline__ void store1(char* p, float f) { *reinterpret_cast<float*>(p) = f; }
};

// Load 8 consecutive elements as fp32.  p must be 16-byte aligned.
template <int DT, bool REMOTE>
__device__ __forceinline__ void load8(const char* p, float* f) {
  if constexpr (DT == kF32) {
    uint4 a = REMOTE ? ld_volatile_v4(p) : ld_v4(p);
    uint4 b = REMOTE ? ld_volatile_v4(p + 16) : ld_v4(p + 16);
    f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
    f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
  } else {
    uint4 a = REMOTE ? ld_volatile_v4(p) : ld_v4(p);
    Elem<DT>::unpack(a, f);
  }
}
template <int DT>
__device__ __forceinline__ void store8(char* p, const float* f) {
  if constexpr (DT == kF32) {
    st_v4(p, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
    st_v4(p + 16, make_uint4(__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])));
  } else {
    st_v4(p, Elem<DT>::pack(f));
  }
}
template <int DT>
__device__ __forceinline__ float load_scalar(const char* p) {
  return Elem<DT>::load1(p);
}

// ---------------------------------------------------------------- CTA-wide reduction
// out[i] = cast<TOUT>( scale * ( a[i] + sum_k w[k][i] ) ),  i in [0, count)
// `a` has TA elements (may be nullptr), the nw extra sources have TW elements; all sums in
// fp32, one rounding at the store.  REMOTE_W: the w sources may have been written by peers.
constexpr int kMaxReduceSrc = kMaxRanks;

template <int TOUT>
__device__ __forceinline__ void store8_all(char* const* outs, int nout, uint64_t byte_off, const float* f) {
  for (int o = 0; o < nout; ++o) store8<TOUT>(outs[o] + byte_off, f);
}

// outs: nout destinations that all receive the same result (nout > 1: the broadcast half
// of an all-reduce).
// 8 elements of type DT as they sit in memory (one 16-byte vector, two for fp32), and their sum into acc.
template <int DT>
struct Raw8 {
  uint4 v[Elem<DT>::size == 4 ? 2 : 1];
};
template <int DT, bool REMOTE>
__device__ __forceinline__ void load8_raw(const char* p, Raw8<DT>& r) {
  r.v[0] = REMOTE ? ld_volatile_v4(p) : ld_v4(p);
  if constexpr (DT == kF32) r.v[1] = REMOTE ? ld_volatile_v4(p + 16) : ld_v4(p + 16);
}
template <int DT>
__device__ __forceinline__ void add8_raw(const Raw8<DT>& r, float* acc) {
  if constexpr (DT == kF32) {
    acc[0] += __uint_as_float(r.v[0].x); acc[1] += __uint_as_float(r.v[0].y);
    acc[2] += __uint_as_float(r.v[0].z); acc[3] += __uint_as_float(r.v[0].w);
    acc[4] += __uint_as_float(r.v[1].x); acc[5] += __uint_as_float(r.v[1].y);
    acc[6] += __uint_as_float(r.v[1].z); acc[7] += __uint_as_float(r.v[1].w);
  } else {
    float t[8];
    Elem<DT>::unpack(r.v[0], t);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += t[e];
  }
}

// The vector part of cta_reduce: G groups of 8 elements per thread and iteration, every load of
// up to KW sources at a time issued before the first add.  With a loop over the sources that adds as it
// loads, the (volatile) loads of peer memory run one round trip after another: seven peers cost
// seven NVLink latencies per iteration.  Sums are formed in source order, as before.
template <int TA, int TW, int TOUT, bool REMOTE_W, int G, int KW>
__device__ __forceinline__ uint64_t cta_reduce_groups(char* const* outs, int nout, const char* a, const char* const* w,
                                                      int nw, uint64_t i, uint64_t ngroups, float scale) {
  constexpr uint64_t SA = 8 * Elem<TA>::size, SW = 8 * Elem<TW>::size, SO = 8 * Elem<TOUT>::size;
  const uint64_t nt = blockDim.x;
  for (; i + (G - 1) * nt < ngroups; i += G * nt) {
    float acc[G][8];
    Raw8<TW> raw[G][KW];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (a != nullptr) {
        load8<TA, false>(a + (i + g * nt) * SA, acc[g]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
      }
    }
    for (int k0 = 0; k0 < nw; k0 += KW) {            // one pass unless there are more than KW sources
#pragma unroll
      for (int k = 0; k < KW; ++k)
        if (k0 + k < nw) {
#pragma unroll
          for (int g = 0; g < G; ++g) load8_raw<TW, REMOTE_W>(w[k0 + k] + (i + g * nt) * SW, raw[g][k]);
        }
#pragma unroll
      for (int k = 0; k < KW; ++k)
        if (k0 + k < nw) {
#pragma unroll
          for (int g = 0; g < G; ++g) add8_raw<TW>(raw[g][k], acc[g]);
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= scale;
      store8_all<TOUT>(outs, nout, (i + g * nt) * SO, acc[g]);
    }
  }
  return i;
}

template <int TA, int TW, int TOUT, bool REMOTE_W>
__device__ __forceinline__ void cta_reduce(char* const* outs, int nout, const char* a,
                                           const char* const* w, int nw, uint64_t count, float scale) {
  if (count == 0) return;
  const uint64_t tid = threadIdx.x, nt = blockDim.x;
  bool aligned = (a == nullptr || (reinterpret_cast<uintptr_t>(a) & 15u) == 0);
  for (int o = 0; o < nout; ++o) aligned = aligned && (reinterpret_cast<uintptr_t>(outs[o]) & 15u) == 0;
  for (int k = 0; k < nw; ++k) aligned = aligned && (reinterpret_cast<uintptr_t>(w[k]) & 15u) == 0;
  uint64_t done = 0;
  if (aligned) {
    const uint64_t ngroups = count >> 3;
    uint64_t i = tid;
    // at most 32 registers of source vectors in flight per thread
    constexpr int kWide = Elem<TW>::size == 4 ? 2 : 1;      // 16-byte vectors per 8 elements
    if (nw <= 1) i = cta_reduce_groups<TA, TW, TOUT, REMOTE_W, 2, 1>(outs, nout, a, w, nw, i, ngroups, scale);
    i = cta_reduce_groups<TA, TW, TOUT, REMOTE_W, 1, 4 / kWide>(outs, nout, a, w, nw, i, ngroups, scale);
    done = ngroups << 3;
  }
  for (uint64_t i = done + tid; i < count; i += nt) {
    float acc = a != nullptr ? load_scalar<TA>(a + i * Elem<TA>::size) : 0.f;
    for (int k = 0; k < nw; ++k) {
      const char* p = w[k] + i * Elem<TW>::size;
      if constexpr (Elem<TW>::size == 4) {
        acc += __uint_as_float(REMOTE_W ? ld_relaxed_sys(reinterpret_cast<const uint32_t*>(p))
                                        : *reinterpret_cast<const uint32_t*>(p));
      } else {
        unsigned short bits = *reinterpret_cast<const volatile unsigned short*>(p);
        if constexpr (TW == kBF16) acc += __uint_as_float(uint32_t(bits) << 16);
        else acc += __half2float(__ushort_as_half(bits));
      }
    }
    for (int o = 0; o < nout; ++o) Elem<TOUT>::store1(outs[o] + i * Elem<TOUT>::size, acc * scale);
  }
}

// ---------------------------------------------------------------- NVLS (multimem) wrappers
// One instruction addresses the same offset of every GPU bound to the multicast object:
// ld_reduce sums inside the switch (fp32 accumulation for 16-bit types), st writes all.
template <int DT>
__device__ __forceinline__ uint4 multimem_ld_reduce_v4(const char* mc_ptr) {
  uint4 v;
  if constexpr (DT == kBF16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_ptr) : "memory");
  } else if constexpr (DT == kF16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_ptr) : "memory");
  } else {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_ptr) : "memory");
  }
  return v;
}
__device__ __forceinline__ void multimem_st_v4(char* mc_ptr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace pccl
