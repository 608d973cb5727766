// TMA bulk-copy data path of the collective kernels.
//
// A lane (CTA) moves its byte range through a ring of shared-memory stages: one elected
// thread issues cp.async.bulk global->shared loads (completion counted on an mbarrier) and
// cp.async.bulk shared->global stores (bulk groups).  The copy engine of the SM does the
// moving, so a lane keeps hundreds of KB in flight without spending registers or issue
// slots, and a handful of lanes saturates NVLink where a load/store loop needs every SM.
// The same staged data can be stored to several destinations (all-gather push, broadcast):
// local memory is read once per peer set.
//
// Loads may come from a peer's memory and stores may go to a peer's memory; none of the
// copies uses cluster multicast.  Every wait on an mbarrier is bounded.
//
// Requirements of the bulk path: 16-byte aligned addresses and a length that is a
// multiple of 16.  Callers fall back to the load/store loops of primitives.cuh otherwise.
#pragma once
#include <stdint.h>

#include "primitives.cuh"

namespace pccl {

constexpr uint32_t kBulkStageBytes = 32 * 1024;
constexpr int kBulkStages = 6;
constexpr uint32_t kBulkSmemBytes = kBulkStageBytes * kBulkStages + 64;   // stages + mbarriers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded: gives up after the communicator's time limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t timeout_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 255u) == 0u && global_timer_ns() - t0 > timeout_ns) return false;
  }
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All committed groups have finished READING shared memory (their stage may be refilled).
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// All committed groups are complete: their global writes have been performed.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Per-CTA pipeline state.  Lives in registers of every thread, but only the driving thread
// (threadIdx.x == 0) uses `count` for issuing; all threads keep it in step for the waits.
struct BulkPipe {
  char* stages;      // kBulkStages * kBulkStageBytes, 128-byte aligned
  uint64_t* full;    // kBulkStages mbarriers
  uint32_t count;    // chunks pushed through the ring so far (stage = count % N, parity = (count / N) & 1)
  uint64_t timeout_ns;
};

__device__ __forceinline__ void bulk_pipe_init(BulkPipe& p, unsigned char* smem, uint64_t timeout_ns) {
  p.stages = reinterpret_cast<char*>(smem);
  p.full = reinterpret_cast<uint64_t*>(smem + (size_t)kBulkStageBytes * kBulkStages);
  p.count = 0;
  p.timeout_ns = timeout_ns;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kBulkStages; ++i) mbar_init(p.full + i, 1);
    fence_mbar_init();
  }
  __syncthreads();
}

__device__ __forceinline__ bool bulk_ok(const void* a, const void* b, uint64_t bytes) {
  return bytes >= 16 && (bytes & 15u) == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15u) == 0;
}

// Copy `bytes` from src to each of dsts[0..ndst).  Called by all threads; thread 0 drives the
// copy engine.  On return the stores are ISSUED, not complete: call cta_bulk_flush() before
// publishing a flag.  Returns false if a load did not arrive within the time limit.
__device__ __forceinline__ bool cta_bulk_copy(BulkPipe& p, char* const* dsts, int ndst, const char* src, uint64_t bytes) {
  const uint32_t nchunks = (uint32_t)((bytes + kBulkStageBytes - 1) / kBulkStageBytes);
  __shared__ int s_bulk_ok;
  if (threadIdx.x == 0) {
    bool ok = true;
    bulk_wait_read_all();                       // stages of an earlier call are free again
    asm volatile("fence.proxy.async;" ::: "memory");   // flags were acquired through the generic proxy
    const uint32_t k0 = p.count;
    uint32_t loaded = 0;
    auto issue = [&](uint32_t i) {
      const uint32_t st = (k0 + i) % kBulkStages;
      const uint64_t off = (uint64_t)i * kBulkStageBytes;
      const uint32_t len = (uint32_t)((bytes - off) < kBulkStageBytes ? (bytes - off) : kBulkStageBytes);
      mbar_expect_tx(p.full + st, len);
      bulk_load(p.stages + (size_t)st * kBulkStageBytes, src + off, len, p.full + st);
    };
    for (; loaded < nchunks && loaded < (uint32_t)kBulkStages; ++loaded) issue(loaded);
    for (uint32_t i = 0; i < nchunks; ++i) {
      const uint32_t k = k0 + i, st = k % kBulkStages, parity = (k / kBulkStages) & 1u;
      if (!mbar_wait(p.full + st, parity, p.timeout_ns)) {
        ok = false;
        break;
      }
      const uint64_t off = (uint64_t)i * kBulkStageBytes;
      const uint32_t len = (uint32_t)((bytes - off) < kBulkStageBytes ? (bytes - off) : kBulkStageBytes);
      for (int d = 0; d < ndst; ++d) bulk_store(dsts[d] + off, p.stages + (size_t)st * kBulkStageBytes, len);
      bulk_commit();
      if (loaded < nchunks) {
        bulk_wait_read_all();                   // this stage has been read out: refill it
        issue(loaded);
        ++loaded;
      }
    }
    s_bulk_ok = ok ? 1 : 0;
  }
  p.count += nchunks;
  __syncthreads();
  const int ok = s_bulk_ok;
  __syncthreads();
  return ok != 0;
}

// Wait until every store issued by this CTA has been performed (then a release flag may follow).
__device__ __forceinline__ void cta_bulk_flush() {
  if (threadIdx.x == 0) {
    bulk_wait_all();
    asm volatile("fence.proxy.async;" ::: "memory");   // async-proxy writes before the generic-proxy flag
    __threadfence_system();
  }
}

// out[i] = cast<TOUT>(scale * sum_k src_k[i]) for nsrc sources of type TIN (local or peer
// memory), staged through shared memory by the copy engine, summed in fp32 by all threads.
// count elements; every pointer 16-byte aligned; count * size a multiple of 16.
template <int TIN, int TOUT>
__device__ __forceinline__ bool cta_bulk_reduce(BulkPipe& p, char* const* outs, int nout, const char* const* srcs, int nsrc,
                                                uint64_t count, float scale) {
  constexpr uint64_t SI = Elem<TIN>::size, SO = Elem<TOUT>::size;
  // one stage holds nsrc sub-buffers of `sub` bytes each
  const uint32_t sub = (kBulkStageBytes / (uint32_t)nsrc) & ~127u;
  const uint64_t bytes = count * SI;
  const uint32_t nchunks = (uint32_t)((bytes + sub - 1) / sub);
  const uint32_t k0 = p.count;
  bool ok = true;
  auto issue = [&](uint32_t i) {
    const uint32_t st = (k0 + i) % kBulkStages;
    const uint64_t off = (uint64_t)i * sub;
    const uint32_t len = (uint32_t)((bytes - off) < sub ? (bytes - off) : sub);
    mbar_expect_tx(p.full + st, len * (uint32_t)nsrc);
    for (int s = 0; s < nsrc; ++s)
      bulk_load(p.stages + (size_t)st * kBulkStageBytes + (size_t)s * sub, srcs[s] + off, len, p.full + st);
  };
  uint32_t loaded = 0;
  if (threadIdx.x == 0) {
    bulk_wait_read_all();
    asm volatile("fence.proxy.async;" ::: "memory");
    for (; loaded < nchunks && loaded < (uint32_t)kBulkStages; ++loaded) issue(loaded);
  } else {
    loaded = nchunks < (uint32_t)kBulkStages ? nchunks : (uint32_t)kBulkStages;
  }
  for (uint32_t i = 0; i < nchunks; ++i) {
    const uint32_t k = k0 + i, st = k % kBulkStages, parity = (k / kBulkStages) & 1u;
    if (!mbar_wait(p.full + st, parity, p.timeout_ns)) ok = false;
    if (__syncthreads_or(!ok)) {
      ok = false;
      break;
    }
    const uint64_t off = (uint64_t)i * sub;
    const uint32_t len = (uint32_t)((bytes - off) < sub ? (bytes - off) : sub);
    const char* base = p.stages + (size_t)st * kBulkStageBytes;
    const uint32_t nvec = len >> 4;                       // 16-byte vectors per source
    constexpr int EPV = 16 / (int)SI;                     // elements per vector: 8 (16-bit) or 4 (fp32)
    for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int s = 0; s < nsrc; ++s) {
        const uint4 q = *reinterpret_cast<const uint4*>(base + (size_t)s * sub + ((size_t)v << 4));
        float f[8];
        if constexpr (TIN == kF32) {
          f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
        } else {
          Elem<TIN>::unpack(q, f);
        }
#pragma unroll
        for (int e = 0; e < EPV; ++e) acc[e] += f[e];
      }
#pragma unroll
      for (int e = 0; e < EPV; ++e) acc[e] *= scale;
      const uint64_t elem = (off >> (SI == 4 ? 2 : 1)) + (uint64_t)v * EPV;
      for (int o = 0; o < nout; ++o) {
        char* dst = outs[o] + elem * SO;
        if constexpr (TOUT == kF32) {
          st_v4(dst, make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3])));
          if constexpr (EPV == 8)
            st_v4(dst + 16, make_uint4(__float_as_uint(acc[4]), __float_as_uint(acc[5]), __float_as_uint(acc[6]), __float_as_uint(acc[7])));
        } else if constexpr (EPV == 8) {
          st_v4(dst, Elem<TOUT>::pack(acc));
        } else {   // fp32 in, 16-bit out: 4 elements = 8 bytes
          float t[8] = {acc[0], acc[1], acc[2], acc[3], 0.f, 0.f, 0.f, 0.f};
          const uint4 w = Elem<TOUT>::pack(t);
          *reinterpret_cast<uint2*>(dst) = make_uint2(w.x, w.y);
        }
      }
    }
    __syncthreads();                                      // everyone is done reading this stage
    if (threadIdx.x == 0 && loaded < nchunks) issue(loaded);
    if (loaded < nchunks) ++loaded;
  }
  p.count += nchunks;
  return ok;
}

}  // namespace pccl
