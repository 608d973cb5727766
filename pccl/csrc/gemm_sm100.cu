// tcgen05 / TMEM / TMA GEMM for sm_100a, with an optional in-kernel all-gather of the
// weight (see gemm.h for the operation).
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer: A and W tiles (128x64, 256x64 bf16, 128-byte swizzle) into a
//               4-stage shared-memory ring; plain tiled TMA loads, no cluster multicast
//   warp 1      allocates TMEM, issues tcgen05.mma (M128 N256 K16, cta_group::1) from one
//               elected thread; tcgen05.commit releases ring stages and publishes accumulators
//   warps 2-5   epilogue: tcgen05.ld 32x32b from TMEM, bias, bf16, 16-byte stores
// Two 128x256 fp32 accumulators (all 512 TMEM columns) let the epilogue of one tile overlap
// the main loop of the next.
//
// Fused mode: the first `gather_ctas` CTAs do not multiply; they pull 256-row panels of the
// peers' weight shards into the local buffer with the copy engine (bulk.cuh) and raise one
// flag per panel.  The producer of a GEMM CTA waits for the panel's flag before its TMA
// loads read the panel from LOCAL memory; panels of the own shard are read directly from
// the shard, so the math starts immediately.  Remote data crosses NVLink exactly once.
//
// Every wait (mbarrier, panel flag, peer flag) is bounded; on expiry the kernel records an
// error code, lets the other roles drain, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "bulk.cuh"
#include "act.cuh"
#include "gemm.h"
#include "primitives.cuh"

namespace pccl {

namespace {

constexpr int BM = kGemmBM, BN = kGemmBN, BK = kGemmBK;
constexpr int kStages = 4;
constexpr uint32_t kABytes = BM * BK * 2;            // 16 KiB
constexpr uint32_t kBBytes = BN * BK * 2;            // 32 KiB
constexpr uint32_t kStageBytes = kABytes + kBBytes;  // 48 KiB
constexpr uint32_t kBarOff = kStages * kStageBytes;  // 196,608
constexpr uint32_t kGemmSmem = kBarOff + 256 + 1024; // barriers + slack for 1 KiB alignment
constexpr int kGemmThreads = 192;
constexpr uint64_t kWaitNs = 4ull * 1000 * 1000 * 1000;
constexpr uint32_t kTmemCols = 512;

static_assert(kBulkSmemBytes <= kBarOff + 256, "the gatherer's copy ring must fit into the GEMM's shared memory");

// ---- error codes written to *error
constexpr int kErrProducer = 1, kErrMma = 2, kErrEpilogue = 3, kErrPanel = 4, kErrGather = 5;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait that also gives up when another role has failed.
__device__ __forceinline__ bool gemm_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > kWaitNs) return false;
    }
  }
}

// The same for waits that are expected to last microseconds: pauses between polls.
__device__ __forceinline__ bool gemm_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t it = 0;
  for (;;) {
    __nanosleep(64);
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 63u) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > kWaitNs) return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes,
// 8-row groups 1024 bytes apart, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset
  d |= (uint64_t)1 << 46;                              // version
  d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
  return d;
}

// Instruction descriptor: D fp32, A and B bf16, both K-major, N = 256, M = 128.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(kIdesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

struct TileSched {
  int tiles_m, tiles_n, total;
  int tiles_per_rank, P, me;   // fused mode: own panels first, then the peers' in arrival order
  // Tiles are walked in bands of kGroupM row-tiles: the ~148 tiles in flight then cover a
  // 16 x 9 patch of the output instead of 148 x 1, so one wave touches ~17 MB of A and W
  // instead of ~80 MB and the operands are served from L2 rather than HBM.
  // Fused mode walks all row-tiles of a panel before the next panel (group_m = tiles_m):
  // panels are then needed as late as possible, in the order in which they arrive.
  int group_m;
  __device__ __forceinline__ void decode(int t, int* m_idx, int* n_idx) const {
    const int band_tiles = group_m * tiles_n;
    const int band = t / band_tiles;
    const int first_m = band * group_m;
    const int rows = (tiles_m - first_m) < group_m ? (tiles_m - first_m) : group_m;
    const int in_band = t - band * band_tiles;
    const int q = in_band / rows;
    *m_idx = first_m + in_band - q * rows;
    if (tiles_per_rank > 0) {
      const int r = (me + q / tiles_per_rank) % P;
      *n_idx = r * tiles_per_rank + q % tiles_per_rank;
    } else {
      *n_idx = q;
    }
  }
};

// cp.async.bulk.wait_group takes an immediate: wait until at most n groups are pending.
__device__ __forceinline__ void bulk_wait_pending(int n) {
  switch (n) {
    case 1: asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.bulk.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.bulk.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.bulk.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.bulk.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.bulk.wait_group 6;" ::: "memory"); break;
    case 7: asm volatile("cp.async.bulk.wait_group 7;" ::: "memory"); break;
    case 8: asm volatile("cp.async.bulk.wait_group 8;" ::: "memory"); break;
    default: asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); break;   // conservative
  }
}

// ---------------------------------------------------------------- gatherer CTAs
__device__ void gather_role(const GemmArgs& a, unsigned char* smem, int gi) {
  const GroupDev& g = a.g;
  const int P = g.size, me = g.first_local;
  const bool flag_sync = g.sig[0] != nullptr;
  const LaneCtx c{0, me, gi, kCollAgGemm};
  BulkPipe pipe;
  bulk_pipe_init(pipe, smem, g.timeout_ns);
  const int tpr = (a.N / P) / BN;
  const uint64_t panel_bytes = (uint64_t)BN * a.K * 2;
  const unsigned others = others_mask(P, me);
  char* w_full = reinterpret_cast<char*>(const_cast<void*>(a.W));
  if (flag_sync) cta_signal_mask(g, c, kSlotEntry, others);
  bool ok = true;
  if (flag_sync && !cta_wait_mask(g, c, kSlotEntry, others)) ok = false;
  // Every gatherer moves its slice of every panel as ONE continuous stream of 32 KiB chunks
  // through the copy ring, panels in the order in which the GEMM CTAs want them (peers me+1,
  // me+2, ..., the own shard last: the GEMM reads that from the shard itself).  A panel's
  // flag is raised one panel later, when `wait_group` says that everything older than the
  // newest panel's stores has been performed, so the pipeline never drains.
  uint64_t lo, hi;
  lane_range(panel_bytes, 16, gi, a.gather_ctas, &lo, &hi);
  const uint64_t len = hi - lo;
  if (threadIdx.x == 0 && ok && len > 0) {
    const uint32_t cpp = (uint32_t)((len + kBulkStageBytes - 1) / kBulkStageBytes);   // chunks per panel slice
    const uint32_t npanels = (uint32_t)(P * tpr);
    const uint32_t total = npanels * cpp;
    const int nremote = (P - 1) * tpr;
    auto locate = [&](uint32_t ch, const char** src, char** dst, uint32_t* bytes, int* n_tile) {
      const int i = (int)(ch / cpp);
      const uint64_t off = (uint64_t)(ch % cpp) * kBulkStageBytes;
      const int k = i < nremote ? 1 + i / tpr : 0;
      const int j = i < nremote ? i % tpr : i - nremote;
      const int p = (me + k) % P;
      *n_tile = p * tpr + j;
      *src = g.heap[p] + a.shard_off + (uint64_t)j * panel_bytes + lo + off;
      *dst = w_full + (uint64_t)(*n_tile) * panel_bytes + lo + off;
      *bytes = (uint32_t)((len - off) < kBulkStageBytes ? (len - off) : kBulkStageBytes);
    };
    auto issue = [&](uint32_t ch) {
      const char* src; char* dst; uint32_t bytes; int nt;
      locate(ch, &src, &dst, &bytes, &nt);
      const uint32_t st = ch % kBulkStages;
      mbar_expect_tx(pipe.full + st, bytes);
      bulk_load(pipe.stages + (size_t)st * kBulkStageBytes, src, bytes, pipe.full + st);
    };
    auto raise = [&](int n_tile) {
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence();
      atomicAdd(a.panel_flags + n_tile, 1u);
    };
    asm volatile("fence.proxy.async;" ::: "memory");
    uint32_t loaded = 0;
    for (; loaded < total && loaded < (uint32_t)kBulkStages; ++loaded) issue(loaded);
    int prev_tile = -1;
    for (uint32_t ch = 0; ch < total; ++ch) {
      const uint32_t st = ch % kBulkStages, parity = (ch / kBulkStages) & 1u;
      if (!mbar_wait(pipe.full + st, parity, g.timeout_ns)) {
        ok = false;
        break;
      }
      const char* src; char* dst; uint32_t bytes; int nt;
      locate(ch, &src, &dst, &bytes, &nt);
      bulk_store(dst, pipe.stages + (size_t)st * kBulkStageBytes, bytes);
      bulk_commit();
      if (ch % cpp == cpp - 1) {            // the last chunk of a panel has been issued
        if (prev_tile >= 0) {
          bulk_wait_pending((int)cpp);      // everything older than this panel has landed
          raise(prev_tile);
        }
        prev_tile = nt;
      }
      if (loaded < total) {
        bulk_wait_read_all();
        issue(loaded);
        ++loaded;
      }
    }
    bulk_wait_all();
    if (ok && prev_tile >= 0) raise(prev_tile);
    if (!ok) atomicCAS(a.error, 0, kErrGather);
  }
  __syncthreads();
  if (flag_sync) {
    cta_signal_mask(g, c, kSlotExit, others);   // I no longer read your shard
    cta_wait_mask(g, c, kSlotExit, others);     // nobody reads mine any more
  }
}

// Epilogue of one accumulator row segment: 32 fp32 values of row `row`, columns col0..col0+31.
// Adds the bias, rounds to bf16 and stores; with act_out it also stores gelu() of the rounded
// value (what a separate activation kernel would read) to the second output.
__device__ __forceinline__ void epilogue_store32(const GemmArgs& a, const uint32_t (&r)[32], int row, int col0) {
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.C) + (size_t)row * a.N + col0;
  __nv_bfloat16* act = a.act_out != nullptr ? reinterpret_cast<__nv_bfloat16*>(a.act_out) + (size_t)row * a.N + col0 : nullptr;
  const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
  if (col0 + 32 <= a.N) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (bias != nullptr) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(bias + col0 + v * 8));     // N % 8 == 0: 16-byte aligned
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          b[2 * e] = __uint_as_float(qw[e] << 16);
          b[2 * e + 1] = __uint_as_float(qw[e] & 0xffff0000u);
        }
      }
      uint32_t w[4], g[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x0 = __uint_as_float(r[v * 8 + 2 * e]) + b[2 * e], x1 = __uint_as_float(r[v * 8 + 2 * e + 1]) + b[2 * e + 1];
        __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
        w[e] = *reinterpret_cast<uint32_t*>(&h);
        if (act != nullptr) {
          __nv_bfloat162 hg = __floats2bfloat162_rn(gelu_tanh(__low2float(h)), gelu_tanh(__high2float(h)));
          g[e] = *reinterpret_cast<uint32_t*>(&hg);
        }
      }
      *reinterpret_cast<uint4*>(out + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
      if (act != nullptr) *reinterpret_cast<uint4*>(act + v * 8) = make_uint4(g[0], g[1], g[2], g[3]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      if (col0 + e < a.N) {
        float x = __uint_as_float(r[e]);
        if (bias != nullptr) x += __bfloat162float(bias[col0 + e]);
        const __nv_bfloat16 h = __float2bfloat16_rn(x);
        out[e] = h;
        if (act != nullptr) act[e] = __float2bfloat16_rn(gelu_tanh(__bfloat162float(h)));
      }
    }
  }
}


// ---------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                      const __grid_constant__ CUtensorMap tmWown, const __grid_constant__ GemmArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  if ((int)blockIdx.x < a.gather_ctas) {
    gather_role(a, smem, (int)blockIdx.x);
    return;
  }
  const int cta = (int)blockIdx.x - a.gather_ctas, ncta = (int)gridDim.x - a.gather_ctas;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kBarOff);
  uint64_t* empty = full + kStages;
  uint64_t* tmem_full = empty + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full + i, 1);
      mbar_init(tmem_empty + i, 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  TileSched sch;
  sch.tiles_m = (a.M + BM - 1) / BM;
  sch.tiles_n = (a.N + BN - 1) / BN;
  sch.total = sch.tiles_m * sch.tiles_n;
  sch.P = a.g.size;
  sch.me = a.g.first_local;
  sch.tiles_per_rank = a.gather_ctas > 0 ? (a.N / sch.P) / BN : 0;
  sch.group_m = a.gather_ctas > 0 ? sch.tiles_m : (sch.tiles_m < 16 ? sch.tiles_m : 16);
  const int nkb = (a.K + BK - 1) / BK;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ TMA producer
    uint32_t it = 0;
    bool ok = true;
    for (int t = cta; t < sch.total && ok; t += ncta) {
      int m_idx, n_idx;
      sch.decode(t, &m_idx, &n_idx);
      const CUtensorMap* wmap = &tmW;
      int wy = n_idx * BN;
      if (sch.tiles_per_rank > 0) {
        const int owner = n_idx / sch.tiles_per_rank;
        if (owner == sch.me) {
          wmap = &tmWown;                                   // straight from the shard
          wy = (n_idx - owner * sch.tiles_per_rank) * BN;
        } else {
          // wait until a gatherer has landed this panel in the local buffer
          const uint32_t* flag = a.panel_flags + n_idx;
          const uint64_t t0 = global_timer_ns();
          uint32_t spins = 0;
          for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v >= a.flag_target) break;
            if ((++spins & 63u) == 0u) {
              if (*abort_flag != 0 || global_timer_ns() - t0 > kWaitNs) {
                ok = false;
                break;
              }
              __nanosleep(100);
            }
          }
          if (!ok) {
            atomicCAS(a.error, 0, kErrPanel);
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");  // flag came through the generic proxy
        }
      }
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
        if (!gemm_wait(empty + s, ph ^ 1u, abort_flag)) {
          ok = false;
          atomicCAS(a.error, 0, kErrProducer);
          break;
        }
        unsigned char* sa = smem + (size_t)s * kStageBytes;
        mbar_expect_tx(full + s, kStageBytes);
        tma_load_2d(sa, &tmA, kb * BK, m_idx * BM, full + s);
        tma_load_2d(sa + kABytes, wmap, kb * BK, wy, full + s);
      }
    }
    if (!ok) *abort_flag = 1;
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    uint32_t it = 0, tile_count = 0;
    bool ok = true;
    for (int t = cta; t < sch.total && ok; t += ncta, ++tile_count) {
      const uint32_t acc = tile_count & 1u, acc_ph = (tile_count >> 1) & 1u;
      if (!gemm_wait(tmem_empty + acc, acc_ph ^ 1u, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
        if (!gemm_wait(full + s, ph, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes);
        const uint64_t da = smem_desc(sa), db = smem_desc(sa + kABytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          mma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), (kb > 0 || k > 0) ? 1u : 0u);
        mma_commit(empty + s);             // the stage is free once these MMAs have read it
      }
      if (!ok) break;
      mma_commit(tmem_full + acc);         // accumulator complete
    }
    if (!ok) {
      atomicCAS(a.error, 0, kErrMma);
      *abort_flag = 1;
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue
    uint32_t tile_count = 0;
    bool ok = true;
    const int lane_base = (warp & 3) * 32;
    for (int t = cta; t < sch.total && ok; t += ncta, ++tile_count) {
      int m_idx, n_idx;
      sch.decode(t, &m_idx, &n_idx);
      const uint32_t acc = tile_count & 1u, acc_ph = (tile_count >> 1) & 1u;
      if (!gemm_wait(tmem_full + acc, acc_ph, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m_idx * BM + lane_base + lane;
      const uint32_t t_base = tmem_base + acc * BN + ((uint32_t)lane_base << 16);
#pragma unroll 1
      for (int cc = 0; cc < BN / 32; ++cc) {
        uint32_t r[32];
        tmem_ld32(t_base + cc * 32, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col0 = n_idx * BN + cc * 32;
        if (row < a.M && col0 < a.N) epilogue_store32(a, r, row, col0);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + acc);
    }
    if (!ok && lane == 0) {
      atomicCAS(a.error, 0, kErrEpilogue);
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------- 2-SM variant (cta_group::2)
// A pair of CTAs on neighbouring SMs works on one 256x256 tile.  Each CTA stages its own
// 128 rows of A and its own 128 rows of W (32 KiB per stage, six stages), the leader CTA
// issues M=256 MMAs that read both CTAs' shared memory, and each CTA keeps the accumulator
// rows of its half in its own TMEM.  Per FLOP a third less shared-memory traffic than the
// single-SM form.  Loads are plain tiled TMA loads (no cluster multicast); both CTAs' loads
// count on the leader's barrier; commits are sent to each CTA's barrier in turn.
//
// Operand layouts.  An operand whose contraction index is contiguous in memory (A[M,K],
// W[N,K]) is loaded as 128 rows x 64 k ("K-major": rows of 128 bytes, 128-byte swizzle).  An
// operand stored the other way round (A as [K,M], W as [K,N]: what dy^T * x and dy * W read) is
// loaded as 64 k x 128 rows in two blocks of 64 rows ("MN-major": each k is a row of 128 bytes
// holding 64 consecutive rows of the operand; blocks 8 KiB apart).  The MMA reads either
// through its shared-memory descriptor, so no transposing copy exists anywhere.
//
// Epilogue.  Every epilogue warp owns 32 accumulator rows.  It reads 64 columns from TMEM,
// adds the bias, rounds to bf16, writes the 32x64 slab into its own 4 KiB piece of shared
// memory in the 128-byte-swizzled layout and hands it to the copy engine as one tiled TMA
// store (which also clips rows and columns beyond M and N); two pieces per warp alternate.
constexpr int kStages2 = 6;
constexpr uint32_t kHalfBytes = 128 * BK * 2;              // 16 KiB: 128 rows x 64 bf16
constexpr uint32_t kStage2Bytes = 2 * kHalfBytes;          // A half + W half
constexpr uint32_t kEpiOff = kStages2 * kStage2Bytes;      // 196,608
constexpr uint32_t kEpiSlabBytes = 32 * 64 * 2;            // 4 KiB: 32 rows x 64 bf16
constexpr uint32_t kEpiWarpBytes = 2 * kEpiSlabBytes;      // two slabs per epilogue warp
constexpr uint32_t kBar2Off = kEpiOff + 4 * kEpiWarpBytes; // 229,376
constexpr uint32_t kGemm2Smem = kBar2Off + 256 + 1024;     // 230,656 of the 232,448 a CTA may have
static_assert(kBulkSmemBytes <= kBar2Off + 256, "the gatherer's copy ring must fit");
constexpr uint32_t kIdesc2 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

// Descriptor of an MN-major operand tile (64 k x 128 rows as two 8 KiB blocks of 64 rows):
// leading byte offset = distance between the 64-row blocks, stride byte offset = distance
// between groups of eight k (8 rows of 128 bytes), 128-byte swizzle, version 1.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(8192 >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory variable in another CTA of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(leader_bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_u32(smem_src)),
               "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void mma_bf16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Round eight accumulator values (+ bias) to bf16; returns them packed, and gelu() of the
// rounded values in `g` when ACT.
template <bool ACT>
__device__ __forceinline__ uint4 pack8(const uint32_t* r, const float* b, uint4* g) {
  uint32_t w[4], gg[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float x0 = __uint_as_float(r[2 * e]) + b[2 * e], x1 = __uint_as_float(r[2 * e + 1]) + b[2 * e + 1];
    __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
    w[e] = *reinterpret_cast<uint32_t*>(&h);
    if (ACT) {
      __nv_bfloat162 hg = __floats2bfloat162_rn(gelu_tanh(__low2float(h)), gelu_tanh(__high2float(h)));
      gg[e] = *reinterpret_cast<uint32_t*>(&hg);
    }
  }
  if (ACT) *g = make_uint4(gg[0], gg[1], gg[2], gg[3]);
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- tiles drawn at run time.  The producer thread of the leader CTA draws the next tile number
// from the global counter and hands it to every other role of the pair (the peer CTA's producer,
// the MMA issuer, the eight epilogue warps) through a four-slot ring in each CTA's shared memory:
// value written into both CTAs, then one arrival on each CTA's `ready` barrier of the slot; a
// reader copies the value and arrives on the leader's `taken` barrier at once, so a slot is free
// again as soon as all ten readers have looked at it.
constexpr int kSchedSlots = 4;
constexpr uint32_t kSchedReaders = 10;     // peer producer, MMA issuer, 2 x 4 epilogue warps
constexpr int kSchedDone = -1;

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool sched_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++it & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > kWaitNs) return false;
    }
  }
}
struct SchedRing {
  int* tile;            // kSchedSlots values
  uint64_t* ready;      // kSchedSlots barriers, one arrival (the scheduler's)
  uint64_t* taken;      // kSchedSlots barriers in the LEADER CTA, kSchedReaders arrivals
};
// Scheduler (leader CTA's producer thread): draw, publish to both CTAs.  Returns false on a wait that ran out.
__device__ __forceinline__ bool sched_draw(const GemmArgs& a, const SchedRing& r, uint32_t n, int total, volatile int* abort_flag, int* t) {
  const uint32_t slot = n % kSchedSlots, ph = (n / kSchedSlots) & 1u;
  if (!sched_wait(r.taken + slot, ph ^ 1u, abort_flag)) return false;
  const uint32_t v = atomicAdd(a.sched_counter, 1u) - a.sched_base;
  const int tile = v < (uint32_t)total ? (int)v : kSchedDone;
  r.tile[slot] = tile;
  const uint32_t peer_tile = map_to_cta(smem_u32(r.tile + slot), 1);
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(peer_tile), "r"(tile) : "memory");
  mbar_arrive_cluster(map_to_cta(smem_u32(r.ready + slot), 0));
  mbar_arrive_cluster(map_to_cta(smem_u32(r.ready + slot), 1));
  *t = tile;
  return true;
}
// Reader (one thread): wait for slot n, copy the value, give the slot back.
__device__ __forceinline__ bool sched_read(const SchedRing& r, uint32_t n, volatile int* abort_flag, int* t) {
  const uint32_t slot = n % kSchedSlots, ph = (n / kSchedSlots) & 1u;
  if (!sched_wait(r.ready + slot, ph, abort_flag)) return false;
  *t = *reinterpret_cast<volatile int*>(r.tile + slot);
  mbar_arrive_cluster(map_to_cta(smem_u32(r.taken + slot), 0));
  return true;
}

// The work of one CTA pair as a sequence of items (tile, first k-block, end k-block): first its
// run of the k-block sequence of the leading sk_tiles tiles (see GemmArgs), then whole tiles
// sk_tiles + pair, + npairs, ...  Producer, MMA issuer and epilogue walk the same sequence.
struct WorkIter {
  long long cur, end;     // position in the k-block sequence of the split tiles
  int nkb, next_tile, total, stride;
  __device__ __forceinline__ WorkIter(int pair, int npairs, int total_, int nkb_, int sk_tiles)
      : nkb(nkb_), next_tile(sk_tiles + pair), total(total_), stride(npairs) {
    const long long I = (long long)sk_tiles * nkb_;
    cur = I * pair / npairs;
    end = I * (pair + 1) / npairs;
  }
  __device__ __forceinline__ bool next(int* tile, int* kb0, int* kb1) {
    if (cur < end) {
      const int t = (int)(cur / nkb);
      const int k0 = (int)(cur - (long long)t * nkb);
      const long long left = end - cur;
      const int k1 = (long long)(nkb - k0) <= left ? nkb : (int)(k0 + left);
      *tile = t;
      *kb0 = k0;
      *kb1 = k1;
      cur += k1 - k0;
      return true;
    }
    if (next_tile < total) {
      *tile = next_tile;
      *kb0 = 0;
      *kb1 = nkb;
      next_tile += stride;
      return true;
    }
    return false;
  }
};
// The pair whose run of the split sequence (I k-blocks over G pairs) holds k-block i.
__device__ __forceinline__ int sk_pair_of(long long i, long long I, int G) { return (int)(((i + 1) * G + I - 1) / I) - 1; }

// WIDE: the unit of work is two vertically adjacent 256 x 256 tiles that share their W half:
// a stage holds two A halves and one W half (48 KiB, four stages), the MMA issuer feeds both
// accumulators of TMEM from it, and the epilogue drains them as two ordinary tiles.  A quarter
// fewer operand bytes come from L2 per FLOP; the price is that both accumulators belong to one
// unit, so the epilogue of a unit overlaps only the first k-blocks of the next.
template <bool A_MN, bool B_MN, bool WIDE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    gemm_sm100_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                           const __grid_constant__ CUtensorMap tmWown, const __grid_constant__ CUtensorMap tmC,
                           const __grid_constant__ CUtensorMap tmAct, const __grid_constant__ GemmArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  if ((int)blockIdx.x < a.gather_ctas) {      // whole pairs: gather_ctas is even
    gather_role(a, smem, (int)blockIdx.x);
    return;
  }
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = ((int)blockIdx.x - a.gather_ctas) >> 1, npairs = ((int)gridDim.x - a.gather_ctas) >> 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kBar2Off);
  uint64_t* empty = full + kStages2;
  uint64_t* tmem_full = empty + kStages2;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  SchedRing ring;
  ring.ready = reinterpret_cast<uint64_t*>(tmem_slot + 2);
  ring.taken = ring.ready + kSchedSlots;
  ring.tile = reinterpret_cast<int*>(ring.taken + kSchedSlots);
  const bool dynamic = a.sched_counter != nullptr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full + i, 1);
      mbar_init(tmem_empty + i, 8);        // four epilogue warps of each CTA
    }
    for (int i = 0; i < kSchedSlots; ++i) {
      mbar_init(ring.ready + i, 1);
      mbar_init(ring.taken + i, kSchedReaders);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                       // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr int NST = WIDE ? 4 : kStages2;                                  // stages in flight
  constexpr uint32_t SB = WIDE ? 3 * kHalfBytes : kStage2Bytes;             // bytes of one stage in one CTA
  constexpr uint32_t W_OFF = WIDE ? 2 * kHalfBytes : kHalfBytes;            // where the W half sits in a stage
  const int tiles_m = WIDE ? (a.M + 511) / 512 : (a.M + 255) / 256, tiles_n = (a.N + 255) / 256;   // WIDE: units of two row-tiles
  const int total = tiles_m * tiles_n;
  const bool fused = a.panel_flags != nullptr;       // W arrives panel by panel
  // Tiles are walked in bands: `group` row-tiles deep and all column-tiles wide (or, transposed,
  // `group` column-tiles wide and all row-tiles deep), down the short side of the band first.
  const bool walk_n = !fused && a.group_m < 0;            // bands of column-tiles
  // Default depth of a band, from timings of the training shapes with a cold L2: long contractions
  // run up to a fifth faster with shallow bands (the pairs of a round then share few row-tiles and
  // write long contiguous runs of C), outputs that are much taller than wide want deep ones.
  const int auto_depth = tiles_m > 4 * tiles_n ? 16 : (a.K >= 4096 ? 2 : 8);
  const int want = a.group_m > 0 ? a.group_m : (a.group_m < 0 ? -a.group_m : auto_depth);
  const int major = walk_n ? tiles_n : tiles_m, minor = walk_n ? tiles_m : tiles_n;
  const int group = fused ? tiles_m : (major < want ? major : want);
  const int nkb = (a.K + BK - 1) / BK;
  const int P = a.g.size, me = a.g.first_local;
  const int tpr = fused ? (a.N / P) / BN : 0;            // 256-row panels per rank
  auto decode = [&](int t, int* m_idx, int* n_idx) {
    const int band_tiles = group * minor;
    const int band = t / band_tiles;
    const int first = band * group;
    const int depth = (major - first) < group ? (major - first) : group;
    const int in_band = t - band * band_tiles;
    const int q = in_band / depth;
    const int along = first + in_band - q * depth;
    if (walk_n) {
      *n_idx = along;
      *m_idx = q;
      return;
    }
    *m_idx = along;
    // fused: own panels first, then the peers' in the order in which they arrive
    *n_idx = fused ? ((me + q / tpr) % P) * tpr + q % tpr : q;
  };

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    uint32_t it = 0;
    bool ok = true;
    WorkIter work(pair, npairs, total, nkb, a.sk_tiles);
    int t, kb0, kb1;
    uint32_t drawn = 0;
    auto next_item = [&]() -> bool {
      if (!dynamic) return work.next(&t, &kb0, &kb1);
      kb0 = 0;
      kb1 = nkb;
      const bool got = leader ? sched_draw(a, ring, drawn, total, abort_flag, &t) : sched_read(ring, drawn, abort_flag, &t);
      ++drawn;
      if (!got) {
        ok = false;
        atomicCAS(a.error, 0, kErrProducer);
        return false;
      }
      return t != kSchedDone;
    };
    while (ok && next_item()) {
      int m_idx, n_idx;
      decode(t, &m_idx, &n_idx);
      const CUtensorMap* wmap = &tmW;
      int wy = n_idx * 256 + (int)rank * 128;
      if (fused) {
        const int owner = n_idx / tpr;
        if (owner == me) {
          wmap = &tmWown;                                   // straight from the shard
          wy = (n_idx - owner * tpr) * 256 + (int)rank * 128;
        } else {
          const uint32_t* flag = a.panel_flags + n_idx;
          const uint64_t t0 = global_timer_ns();
          uint32_t spins = 0;
          for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v >= a.flag_target) break;
            if ((++spins & 63u) == 0u) {
              if (*abort_flag != 0 || global_timer_ns() - t0 > kWaitNs) {
                ok = false;
                break;
              }
              __nanosleep(100);
            }
          }
          if (!ok) {
            atomicCAS(a.error, 0, kErrPanel);
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
      }
      const int ay = m_idx * (WIDE ? 512 : 256) + (int)rank * 128;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const uint32_t s = it % NST, ph = (it / NST) & 1u;
        if (!gemm_wait(empty + s, ph ^ 1u, abort_flag)) {
          ok = false;
          atomicCAS(a.error, 0, kErrProducer);
          break;
        }
        unsigned char* sa = smem + (size_t)s * SB;
        if (leader) mbar_expect_tx(full + s, 2 * SB);                // both CTAs' bytes land on this barrier
        const uint32_t bar = map_to_cta(smem_u32(full + s), 0);      // the leader's barrier, from either CTA
        if (A_MN) tma_load_3d_pair(sa, &tmA, 0, kb * BK, ay >> 6, bar);
        else tma_load_2d_pair(sa, &tmA, kb * BK, ay, bar);
        if (WIDE) {
          // the lower row-tile of the unit (rows past M read zeros)
          if (A_MN) tma_load_3d_pair(sa + kHalfBytes, &tmA, 0, kb * BK, (ay + 256) >> 6, bar);
          else tma_load_2d_pair(sa + kHalfBytes, &tmA, kb * BK, ay + 256, bar);
        }
        if (B_MN) tma_load_3d_pair(sa + W_OFF, wmap, 0, kb * BK, wy >> 6, bar);
        else tma_load_2d_pair(sa + W_OFF, wmap, kb * BK, wy, bar);
      }
    }
    if (!ok) *abort_flag = 1;
  } else if (warp == 1 && lane == 0 && leader) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    constexpr uint32_t idesc = kIdesc2 | (A_MN ? (1u << 15) : 0u) | (B_MN ? (1u << 16) : 0u);
    constexpr uint64_t a_step = A_MN ? (2048 >> 4) : (32 >> 4);   // 16 k further: 16 rows of 128 B, or 32 bytes along the row
    constexpr uint64_t b_step = B_MN ? (2048 >> 4) : (32 >> 4);
    uint32_t it = 0, tile_count = 0, draws = 0;
    bool ok = true;
    WorkIter work(pair, npairs, total, nkb, a.sk_tiles);
    int t, kb0, kb1;
    auto next_item = [&]() -> bool {
      if (!dynamic) return work.next(&t, &kb0, &kb1);
      kb0 = 0;
      kb1 = nkb;
      if (!sched_read(ring, draws++, abort_flag, &t)) {      // draws, not tiles: a unit of two tiles is one draw
        ok = false;
        return false;
      }
      return t != kSchedDone;
    };
    for (; ok && next_item(); tile_count += WIDE ? 2 : 1) {
      // WIDE: a unit fills both accumulators, so tile_count stays even and acc is 0
      const uint32_t acc = tile_count & 1u, acc_ph = (tile_count >> 1) & 1u;
      if (!gemm_wait(tmem_empty + acc, acc_ph ^ 1u, abort_flag) ||
          (WIDE && !gemm_wait(tmem_empty + 1, acc_ph ^ 1u, abort_flag))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const uint32_t s = it % NST, ph = (it / NST) & 1u;
        if (!gemm_wait(full + s, ph, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + (size_t)s * SB);
        const uint64_t da = A_MN ? smem_desc_mn(sa) : smem_desc(sa);
        const uint64_t db = B_MN ? smem_desc_mn(sa + W_OFF) : smem_desc(sa + W_OFF);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          mma_bf16_pair(d_tmem, da + (uint64_t)k * a_step, db + (uint64_t)k * b_step, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        if (WIDE) {
          const uint64_t da1 = A_MN ? smem_desc_mn(sa + kHalfBytes) : smem_desc(sa + kHalfBytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            mma_bf16_pair(d_tmem + BN, da1 + (uint64_t)k * a_step, db + (uint64_t)k * b_step, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        const uint32_t eb = smem_u32(empty + s);
        mma_commit_pair(map_to_cta(eb, 0));     // free the stage in both CTAs
        mma_commit_pair(map_to_cta(eb, 1));
      }
      if (!ok) break;
      const uint32_t fb = smem_u32(tmem_full + acc);
      mma_commit_pair(map_to_cta(fb, 0));       // accumulator complete: wake both epilogues
      mma_commit_pair(map_to_cta(fb, 1));
      if (WIDE) {
        const uint32_t fb1 = smem_u32(tmem_full + 1);
        mma_commit_pair(map_to_cta(fb1, 0));
        mma_commit_pair(map_to_cta(fb1, 1));
      }
    }
    if (!ok) {
      atomicCAS(a.error, 0, kErrMma);
      *abort_flag = 1;
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    uint32_t tile_count = 0;
    bool ok = true;
    const int q = warp & 3;                     // the quarter of the TMEM lanes this warp may read
    const int lane_base = q * 32;
    unsigned char* ebuf = smem + kEpiOff + (size_t)q * kEpiWarpBytes;
    const bool has_act = a.act_out != nullptr;
    const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
    const uint32_t sw = (uint32_t)(lane & 7);   // 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r % 8)
    uint32_t nstore = 0;                        // slabs stored so far: picks the piece, across tiles too
    uint32_t draws = 0;                         // tiles (or units) taken from the run-time scheduler so far
    WorkIter work(pair, npairs, total, nkb, a.sk_tiles);
    const long long sk_I = (long long)a.sk_tiles * nkb;
    // this warp's 32 x 256 fp32 block inside a pair's scratch slot, and its flag word
    const size_t sk_warp = ((size_t)rank * 4 + (size_t)q) * (32 * 256);
    const uint32_t sk_word = rank * 4 + (uint32_t)q;
    int t, kb0, kb1;
    auto next_item = [&]() -> bool {
      if (!dynamic) return work.next(&t, &kb0, &kb1);
      kb0 = 0;
      kb1 = nkb;
      int got = 1;
      if (lane == 0) got = sched_read(ring, draws, abort_flag, &t) ? 1 : 0;
      ++draws;
      got = __shfl_sync(0xffffffffu, got, 0);
      t = __shfl_sync(0xffffffffu, t, 0);
      if (!got) {
        ok = false;
        return false;
      }
      return t != kSchedDone;
    };
    int sub = 1;                                // WIDE: which row-tile of the current unit comes next
    auto next_tile = [&]() -> bool {
      if (!WIDE) return next_item();
      if (sub == 0) {
        sub = 1;
        return true;                            // the lower row-tile of the unit already drawn
      }
      if (!next_item()) return false;
      sub = 0;
      return true;
    };
    for (; ok && next_tile(); ++tile_count) {
      int m_idx, n_idx;
      decode(t, &m_idx, &n_idx);
      if (WIDE) m_idx = 2 * m_idx + sub;
      const uint32_t acc = tile_count & 1u, acc_ph = (tile_count >> 1) & 1u;
      // one lane polls the barrier (with a pause between polls: an accumulator takes microseconds),
      // the others wait at the shuffle: 124 fewer threads hammering shared memory beside the MMAs
      if (lane == 0) ok = gemm_wait_relaxed(tmem_full + acc, acc_ph, abort_flag);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const int row0 = m_idx * 256 + (int)rank * 128 + lane_base;     // first of this warp's 32 rows
      const uint32_t t_base = tmem_base + acc * BN + ((uint32_t)lane_base << 16);
      const bool partial_only = kb0 > 0;                               // a piece of a tile somebody else finishes
      int first_helper = 0, last_helper = -1;                          // pairs whose partial sums this tile still needs
      if (kb0 == 0 && kb1 < nkb) {
        first_helper = pair + 1;
        last_helper = sk_pair_of((long long)(t + 1) * nkb - 1, sk_I, npairs);
        for (int h = first_helper; h <= last_helper && ok; ++h) {
          if (lane == 0) {
            const uint32_t* flag = a.sk_flags + (size_t)h * kGemmSkFlagsPerPair + sk_word;
            const uint64_t t0 = global_timer_ns();
            uint32_t spins = 0;
            for (;;) {
              uint32_t v;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
              if (v == a.sk_epoch) break;
              if ((++spins & 63u) == 0u && (*abort_flag != 0 || global_timer_ns() - t0 > kWaitNs)) {
                ok = false;
                break;
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (!ok) {
          // hand the accumulator back so that the other roles can drain, then give up
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty + acc), 0));
          break;
        }
      }
#pragma unroll 1
      for (int slab = 0; slab < BN / 64; ++slab) {
        uint32_t r[64];
        tmem_ld32(t_base + slab * 64, r);
        tmem_ld32(t_base + slab * 64 + 32, r + 32);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (slab == BN / 64 - 1) {
          // the accumulator is in registers: hand it back to the MMA issuer before storing
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty + acc), 0));
        }
        if (partial_only) {
          // fp32 partial sums to this pair's scratch slot: float4 j of lane l at (j * 32 + l), so a warp's store is contiguous
          float4* dst = reinterpret_cast<float4*>(a.sk_scratch + (size_t)pair * (2 * 128 * 256) + sk_warp) + (size_t)slab * 16 * 32 + lane;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            __stcg(dst + j * 32, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                             __uint_as_float(r[4 * j + 3])));
          if (slab == BN / 64 - 1) {
            __syncwarp();
            if (lane == 0) {
              __threadfence();
              asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.sk_flags + (size_t)pair * kGemmSkFlagsPerPair + sk_word),
                           "r"(a.sk_epoch)
                           : "memory");
            }
          }
          continue;
        }
        for (int h = first_helper; h <= last_helper; ++h) {
          const float4* src = reinterpret_cast<const float4*>(a.sk_scratch + (size_t)h * (2 * 128 * 256) + sk_warp) + (size_t)slab * 16 * 32 + lane;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float4 v = __ldcg(src + j * 32);
            r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v.x);
            r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v.y);
            r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v.z);
            r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v.w);
          }
        }
        const int col0 = n_idx * 256 + slab * 64;
        if (row0 >= a.M || col0 >= a.N) continue;                     // nothing of this slab exists (warp-uniform)
        unsigned char* cbuf = ebuf + (has_act ? 0u : (nstore & 1u)) * kEpiSlabBytes;
        unsigned char* gbuf = ebuf + kEpiSlabBytes;
        ++nstore;
        // the copy engine must have finished reading the piece that is about to be rewritten:
        // with two alternating pieces that is the store before the previous one
        if (lane == 0) {
          if (has_act) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        }
        __syncwarp();
        if (a.gelu_grad_of != nullptr && row0 + lane < a.M) {
          // result *= gelu'(u[row, col]): this thread's 64 columns of u are 128 contiguous bytes
          const __nv_bfloat16* urow = reinterpret_cast<const __nv_bfloat16*>(a.gelu_grad_of) + (size_t)(row0 + lane) * a.N + col0;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            if (col0 + c * 8 < a.N) {
              const uint4 uq = __ldg(reinterpret_cast<const uint4*>(urow + c * 8));
              const uint32_t uw[4] = {uq.x, uq.y, uq.z, uq.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float u0 = __uint_as_float(uw[e] << 16), u1 = __uint_as_float(uw[e] & 0xffff0000u);
                r[c * 8 + 2 * e] = __float_as_uint(__uint_as_float(r[c * 8 + 2 * e]) * gelu_tanh_grad(u0));
                r[c * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(r[c * 8 + 2 * e + 1]) * gelu_tanh_grad(u1));
              }
            }
          }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (bias != nullptr && col0 + c * 8 < a.N) {
            const uint4 qv = __ldg(reinterpret_cast<const uint4*>(bias + col0 + c * 8));     // N % 8 == 0: whole and aligned
            const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              b[2 * e] = __uint_as_float(qw[e] << 16);
              b[2 * e + 1] = __uint_as_float(qw[e] & 0xffff0000u);
            }
          }
          const uint32_t off = (uint32_t)lane * 128u + (((uint32_t)c ^ sw) << 4);
          uint4 g;
          if (has_act) {
            *reinterpret_cast<uint4*>(cbuf + off) = pack8<true>(r + c * 8, b, &g);
            *reinterpret_cast<uint4*>(gbuf + off) = g;
          } else {
            *reinterpret_cast<uint4*>(cbuf + off) = pack8<false>(r + c * 8, b, &g);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes, async-proxy read
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmC, cbuf, col0, row0);
          if (has_act) tma_store_2d(&tmAct, gbuf, col0, row0);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every store has been performed
    if (!ok && lane == 0) {
      atomicCAS(a.error, 0, kErrEpilogue);
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                       // the peer may still be reading this CTA's shared memory or signalling it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------- host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

// [rows, K] bf16 row-major, box = box_rows x 64 elements, 128-byte swizzle, zero fill.
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Operand stored [K, rows] row-major (rows contiguous, rows % 64 == 0), seen as a 3-D tensor
// {64 consecutive rows, k, block of 64 rows}: one box of 64 x 64 x 2 lands in shared memory as
// two 8 KiB blocks, each holding 64 k as rows of 128 bytes (128-byte swizzle).  k beyond K
// reads zeros; blocks beyond the last one read zeros.
bool make_map_mn(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr || rows % 64 != 0) return false;
  cuuint64_t dims[3] = {64, K, rows / 64};
  cuuint64_t strides[2] = {rows * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)BK, 2};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Output [M, N] bf16 row-major written in boxes of 32 rows x 64 columns (128-byte swizzle).
bool make_map_store(CUtensorMap* map, void* base, uint64_t M, uint64_t N) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {N, M};
  cuuint64_t strides[1] = {N * 2};
  cuuint32_t box[2] = {64, 32};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool A_MN, bool B_MN, bool WIDE = false>
cudaError_t launch_pair(const CUtensorMap& mA, const CUtensorMap& mW, const CUtensorMap& mOwn, const CUtensorMap& mC,
                        const CUtensorMap& mAct, const GemmArgs& a, int grid, cudaStream_t stream) {
  // the shared-memory limit is an attribute of the function on the current device
  static thread_local bool configured[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(gemm_sm100_2cta_kernel<A_MN, B_MN, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemm2Smem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  gemm_sm100_2cta_kernel<A_MN, B_MN, WIDE><<<grid, kGemmThreads, kGemm2Smem, stream>>>(mA, mW, mOwn, mC, mAct, a);
  return cudaGetLastError();
}

}  // namespace

int gemm_sk_tiles(int M, int N, int K, int sm_count) {
  const int G = sm_count / 2;
  const long long T = (long long)((M + 255) / 256) * ((N + 255) / 256);
  const int nkb = (K + BK - 1) / BK;
  if (G < 2 || nkb < 8 || T <= 0 || T > (1 << 30)) return 0;
  const int R = (int)(T % G);
  if (R == 0) return 0;
  const long long rounds = (T + G - 1) / G;
  if ((double)T / ((double)G * (double)rounds) > 0.97) return 0;      // the last round is nearly full anyway
  if (T < G) return (T * nkb / G >= 4) ? (int)T : 0;                  // one partial round: split every tile
  return G + R;                                                       // the last full round and the partial one
}

cudaError_t launch_gemm_sm100(const GemmArgs& a_in, int sm_count, cudaStream_t stream) {
  GemmArgs a = a_in;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || (a.K % 8) != 0 || (a.N % 8) != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.W) | reinterpret_cast<uintptr_t>(a.C)) & 15u)
    return cudaErrorInvalidValue;
  if (a.act_out != nullptr && (reinterpret_cast<uintptr_t>(a.act_out) & 15u)) return cudaErrorInvalidValue;
  const bool fused = a.panel_flags != nullptr;
  if (a.gather_ctas > 0 && !fused) return cudaErrorInvalidValue;
  if (fused && a.gather_ctas == 0 && !a.two_cta) return cudaErrorInvalidValue;   // externally filled panels: CTA-pair form only
  if ((a.a_mn || a.b_mn) && (!a.two_cta || fused)) return cudaErrorInvalidValue;   // layouts: plain CTA-pair form only
  if (a.gelu_grad_of != nullptr && (!a.two_cta || a.bias != nullptr || (reinterpret_cast<uintptr_t>(a.gelu_grad_of) & 15u)))
    return cudaErrorInvalidValue;
  if (a.a_mn && (a.M % 64) != 0) return cudaErrorInvalidValue;
  if (a.b_mn && (a.N % 64) != 0) return cudaErrorInvalidValue;
  const void* own = a.W;
  uint64_t own_rows = (uint64_t)a.N;
  if (fused) {
    const int P = a.g.size;
    if (P < 1 || a.N % (P * BN) != 0 || a.gather_ctas >= sm_count) return cudaErrorInvalidValue;
    own = a.g.heap[a.g.first_local] + a.shard_off;
    own_rows = (uint64_t)a.N / P;
    if (reinterpret_cast<uintptr_t>(own) & 15u) return cudaErrorInvalidValue;
    if (a.gather_ctas > 0) a.flag_target = (uint32_t)a.gather_ctas;
    else if (a.flag_target == 0) a.flag_target = 1;
  }
  if (a.two_cta && (a.gather_ctas % 2) == 0) {
    CUtensorMap mA, mW, mOwn, mC, mAct;
    const bool okA = a.a_mn ? make_map_mn(&mA, a.A, (uint64_t)a.M, (uint64_t)a.K) : make_map(&mA, a.A, (uint64_t)a.M, (uint64_t)a.K, 128);
    const bool okW = a.b_mn ? make_map_mn(&mW, a.W, (uint64_t)a.N, (uint64_t)a.K) : make_map(&mW, a.W, (uint64_t)a.N, (uint64_t)a.K, 128);
    if (!okA || !okW) return cudaErrorInvalidValue;
    if (a.b_mn) mOwn = mW;
    else if (!make_map(&mOwn, own, own_rows, (uint64_t)a.K, 128)) return cudaErrorInvalidValue;
    if (!make_map_store(&mC, a.C, (uint64_t)a.M, (uint64_t)a.N)) return cudaErrorInvalidValue;
    if (a.act_out != nullptr) {
      if (!make_map_store(&mAct, a.act_out, (uint64_t)a.M, (uint64_t)a.N)) return cudaErrorInvalidValue;
    } else {
      mAct = mC;
    }
    // units of two row-tiles that share their W half: plain products only, tiles dealt out in advance
    const bool wide = a.wide != 0 && !fused && a.sk_tiles == 0 && a.M > 256;
    const int tiles2 = (wide ? (a.M + 511) / 512 : (a.M + 255) / 256) * ((a.N + 255) / 256);
    int pairs = (sm_count - a.gather_ctas) / 2;
    if (a.sk_tiles > 0) {
      // tiles split along K: every pair takes part, and the partial sums need their scratch
      if (fused || a.sk_scratch == nullptr || a.sk_flags == nullptr || a.sk_tiles > tiles2) return cudaErrorInvalidValue;
    } else if (!fused && tiles2 < pairs) {
      pairs = tiles2;
    }
    if (a.sched_counter != nullptr && a.sk_tiles > 0) return cudaErrorInvalidValue;   // one way of dealing out tiles at a time
    if (!fused && a.max_pairs > 0 && a.max_pairs < pairs) pairs = a.max_pairs;
    if (pairs < 1) return cudaErrorInvalidValue;
    const int grid = a.gather_ctas + pairs * 2;
    if (wide) {
      if (a.a_mn && a.b_mn) return launch_pair<true, true, true>(mA, mW, mOwn, mC, mAct, a, grid, stream);
      if (a.a_mn) return launch_pair<true, false, true>(mA, mW, mOwn, mC, mAct, a, grid, stream);
      if (a.b_mn) return launch_pair<false, true, true>(mA, mW, mOwn, mC, mAct, a, grid, stream);
      return launch_pair<false, false, true>(mA, mW, mOwn, mC, mAct, a, grid, stream);
    }
    if (a.a_mn && a.b_mn) return launch_pair<true, true>(mA, mW, mOwn, mC, mAct, a, grid, stream);
    if (a.a_mn) return launch_pair<true, false>(mA, mW, mOwn, mC, mAct, a, grid, stream);
    if (a.b_mn) return launch_pair<false, true>(mA, mW, mOwn, mC, mAct, a, grid, stream);
    return launch_pair<false, false>(mA, mW, mOwn, mC, mAct, a, grid, stream);
  }
  if (a.a_mn || a.b_mn) return cudaErrorInvalidValue;
  CUtensorMap tmA, tmW, tmWown;
  if (!make_map(&tmA, a.A, (uint64_t)a.M, (uint64_t)a.K, BM)) return cudaErrorInvalidValue;
  if (!make_map(&tmW, a.W, (uint64_t)a.N, (uint64_t)a.K, BN)) return cudaErrorInvalidValue;
  if (!make_map(&tmWown, own, own_rows, (uint64_t)a.K, BN)) return cudaErrorInvalidValue;
  static thread_local bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int tiles = ((a.M + BM - 1) / BM) * ((a.N + BN - 1) / BN);
  int grid = sm_count;
  if (!fused && tiles < grid) grid = tiles;
  gemm_sm100_kernel<<<grid, kGemmThreads, kGemmSmem, stream>>>(tmA, tmW, tmWown, a);
  return cudaGetLastError();
}

}  // namespace pccl
