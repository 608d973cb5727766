// Memory-bound training kernels of the GPT forward and backward pass, each one pass over the
// activations: column sums (bias gradients), GELU forward, GELU backward fused with the
// column sum of its result, layer norm fused with the residual add in front of it, and
// layer-norm backward with its weight/bias gradients and the residual gradient added in.
//
// The reference has no model code; these serve the in-repo ZeRO-3 engine, where the stock
// framework kernels for the same jobs cost about a sixth of the step.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "act.cuh"
#include "optim.h"

namespace pccl {

namespace {

__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ float round_bf16(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }

// ---------------------------------------------------------------- column sum
// out[c] = sum_r X[r, c]; X is [T, N] bf16 row-major with N % 8 == 0.  A block covers 512
// columns (64 threads x 16 bytes: 1 KiB of one row, so a warp reads 512 contiguous bytes) in
// four row lanes, and one slice of the rows; the last block to finish a column tile adds the
// slices' fp32 partial sums and writes bf16.
// GELU form: X is the gradient of the GELU's output and U its input; the kernel writes
// DU = X * gelu'(U) and sums the columns of DU (as rounded to bf16), the bias gradient of
// the linear layer in front of the GELU.
// Concatenating form: the columns are those of three [T, N/3] matrices side by side (the
// gradients of q, k and v); the kernel writes the [T, N] concatenation to DU while it sums.
constexpr int kColTile = 512, kRowLanes = 4;
enum ColMode { kColSum = 0, kColGelu = 1, kColCat3 = 2 };

template <int MODE>
__device__ __forceinline__ void col_item(const uint4& q, const uint4& uq, __nv_bfloat16* DU, int64_t off, float* acc) {
  float f[8];
  unpack8(q, f);
  if (MODE == kColGelu) {
    float u[8];
    unpack8(uq, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] *= gelu_tanh_grad(u[e]);
    const uint4 packed = pack8(f);               // one rounding; the sums below are of the rounded values
    *reinterpret_cast<uint4*>(DU + off) = packed;
    unpack8(packed, f);
  }
  if (MODE == kColCat3) *reinterpret_cast<uint4*>(DU + off) = q;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] += f[e];
}

template <int MODE>
__global__ void __launch_bounds__(256) col_sum_kernel(const __nv_bfloat16* __restrict__ X, int64_t T, int N,
                                                      __nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                                                      int* __restrict__ counters, const __nv_bfloat16* __restrict__ U,
                                                      __nv_bfloat16* __restrict__ DU, const __nv_bfloat16* __restrict__ X2) {
  __shared__ __align__(16) float red[kRowLanes][kColTile];
  __shared__ int s_last;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int col_base = blockIdx.x * kColTile;
  const int col = col_base + tx * 8;
  const int R = gridDim.y;
  const int64_t rows_per = (T + R - 1) / R;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per;
  const int64_t r1 = r0 + rows_per < T ? r0 + rows_per : T;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  if (col < N) {
    // where this thread's 8 columns come from: X itself, or one of the three sources
    const __nv_bfloat16* src = X + col;
    int64_t ld = N;
    if (MODE == kColCat3) {
      const int w = N / 3, which = col / w;
      src = (which == 0 ? X : which == 1 ? U : X2) + (col - which * w);
      ld = w;
    }
    int64_t r = r0 + ty;
    for (; r + 3 * kRowLanes < r1; r += 4 * kRowLanes) {
      uint4 q[4], uq[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        q[k] = *reinterpret_cast<const uint4*>(src + (r + k * kRowLanes) * ld);
        uq[k] = MODE == kColGelu ? *reinterpret_cast<const uint4*>(U + (r + k * kRowLanes) * N + col) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) col_item<MODE>(q[k], uq[k], DU, (r + k * kRowLanes) * N + col, acc);
    }
    for (; r < r1; r += kRowLanes) {
      const uint4 q = *reinterpret_cast<const uint4*>(src + r * ld);
      const uint4 uq = MODE == kColGelu ? *reinterpret_cast<const uint4*>(U + r * N + col) : make_uint4(0, 0, 0, 0);
      col_item<MODE>(q, uq, DU, r * N + col, acc);
    }
  }
  *reinterpret_cast<float4*>(&red[ty][tx * 8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  *reinterpret_cast<float4*>(&red[ty][tx * 8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  __syncthreads();
  for (int c = threadIdx.x; c < kColTile; c += 256)
    if (col_base + c < N) partial[(int64_t)blockIdx.y * N + col_base + c] = red[0][c] + red[1][c] + red[2][c] + red[3][c];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(counters + blockIdx.x, 1) == R - 1;
  __syncthreads();
  if (s_last) {
    __threadfence();
    // the four row lanes split the slices; every thread adds 8 columns of its share
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (col < N) {
      int y = ty;
      for (; y + 3 * kRowLanes < R; y += 4 * kRowLanes) {
        float4 v[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float* src = partial + (int64_t)(y + k * kRowLanes) * N + col;
          v[2 * k] = __ldcg(reinterpret_cast<const float4*>(src));
          v[2 * k + 1] = __ldcg(reinterpret_cast<const float4*>(src + 4));
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          acc[0] += v[2 * k].x, acc[1] += v[2 * k].y, acc[2] += v[2 * k].z, acc[3] += v[2 * k].w;
          acc[4] += v[2 * k + 1].x, acc[5] += v[2 * k + 1].y, acc[6] += v[2 * k + 1].z, acc[7] += v[2 * k + 1].w;
        }
      }
      for (; y < R; y += kRowLanes) {
        const float* src = partial + (int64_t)y * N + col;
        const float4 v0 = __ldcg(reinterpret_cast<const float4*>(src)), v1 = __ldcg(reinterpret_cast<const float4*>(src + 4));
        acc[0] += v0.x, acc[1] += v0.y, acc[2] += v0.z, acc[3] += v0.w;
        acc[4] += v1.x, acc[5] += v1.y, acc[6] += v1.z, acc[7] += v1.w;
      }
    }
    __syncthreads();
    *reinterpret_cast<float4*>(&red[ty][tx * 8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(&red[ty][tx * 8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    __syncthreads();
    for (int c = threadIdx.x; c < kColTile; c += 256)
      if (col_base + c < N) out[col_base + c] = __float2bfloat16_rn(red[0][c] + red[1][c] + red[2][c] + red[3][c]);
    if (threadIdx.x == 0) counters[blockIdx.x] = 0;   // ready for the next call
  }
}

// ---------------------------------------------------------------- layer-norm backward
// One pass over dy and x:  dx = rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dy * gamma,
// and per-block partial sums of dgamma = sum_r dy * xhat, dbeta = sum_r dy.
//
// 128 threads work on one row (EPT = d / 128 elements each, in 16-byte vectors).  A block has
// two such row groups and each group takes RB rows per iteration: all their loads (dy, x and the
// residual gradient, kept packed as bf16) are issued before the first use, so a block keeps
// 2 * RB rows in flight, and the RB row reductions share one pair of block barriers.
// With `resid` the gradient that flows around the layer norm (the residual connection) is added
// to dx in the same pass (in fp32, before the one rounding); with `pdx` the kernel also sums the columns of dx (the
// bias gradient of the linear layer whose output gradient dx is).  The two groups add their
// column sums through shared memory, so a block leaves one partial row per array, and a second
// small kernel adds the blocks' partials.
template <int EPT>
__device__ __forceinline__ void ln_bwd_combine(const float* acc, float* comb, float* out_row, int rg, int t) {
  constexpr int NV = EPT / 8;
  if (rg == 0) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float4* c = reinterpret_cast<float4*>(comb + (t + 128 * k) * 8);
      c[0] = make_float4(acc[8 * k], acc[8 * k + 1], acc[8 * k + 2], acc[8 * k + 3]);
      c[1] = make_float4(acc[8 * k + 4], acc[8 * k + 5], acc[8 * k + 6], acc[8 * k + 7]);
    }
  }
  __syncthreads();
  if (rg == 1) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const float4* c = reinterpret_cast<const float4*>(comb + (t + 128 * k) * 8);
      const float4 a0 = c[0], a1 = c[1];
      float4* o = reinterpret_cast<float4*>(out_row + (t + 128 * k) * 8);
      o[0] = make_float4(a0.x + acc[8 * k], a0.y + acc[8 * k + 1], a0.z + acc[8 * k + 2], a0.w + acc[8 * k + 3]);
      o[1] = make_float4(a1.x + acc[8 * k + 4], a1.y + acc[8 * k + 5], a1.z + acc[8 * k + 6], a1.w + acc[8 * k + 7]);
    }
  }
  __syncthreads();
}

template <int EPT, int RB>
__global__ void __launch_bounds__(256, 1)
    ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const float* __restrict__ mean,
                  const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ gamma,
                  const __nv_bfloat16* __restrict__ resid, __nv_bfloat16* __restrict__ dx, float* __restrict__ pgamma,
                  float* __restrict__ pbeta, float* __restrict__ pdx, int64_t T, int d) {
  constexpr int NV = EPT / 8;
  __shared__ float red[2][RB][4][2];
  __shared__ __align__(16) float comb[128 * EPT];
  const int rg = threadIdx.x >> 7, t = threadIdx.x & 127, warp_in_rg = t >> 5, lane = t & 31;
  uint4 pgam[NV];
  float dgam[EPT], dbet[EPT], dxs[EPT];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    pgam[k] = *reinterpret_cast<const uint4*>(gamma + (t + 128 * k) * 8);
#pragma unroll
    for (int e = 0; e < 8; ++e) dgam[8 * k + e] = dbet[8 * k + e] = dxs[8 * k + e] = 0.f;
  }
  const float inv_d = 1.0f / (float)d;
  const int64_t step = 2 * RB * (int64_t)gridDim.x;
  for (int64_t base = (int64_t)blockIdx.x * 2 * RB; base < T; base += step) {
    uint4 pdy[RB][NV], px[RB][NV], pr[RB][NV];
    float mu[RB], rs[RB];
    // ---- all loads of this group's rows
#pragma unroll
    for (int j = 0; j < RB; ++j) {
      const int64_t r = base + rg * RB + j;
      mu[j] = 0.f;
      rs[j] = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) pdy[j][k] = px[j][k] = pr[j][k] = make_uint4(0, 0, 0, 0);
      if (r < T) {
        mu[j] = mean[r];
        rs[j] = rstd[r];
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const int64_t off = r * d + (t + 128 * k) * 8;
          pdy[j][k] = *reinterpret_cast<const uint4*>(dy + off);
          px[j][k] = *reinterpret_cast<const uint4*>(x + off);
          if (resid != nullptr) pr[j][k] = *reinterpret_cast<const uint4*>(resid + off);
        }
      }
    }
    // ---- row sums and the weight/bias gradient sums (rows past the end hold zeros)
#pragma unroll
    for (int j = 0; j < RB; ++j) {
      float s1 = 0.f, s2 = 0.f;
      const float nmr = -mu[j] * rs[j];
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        float a[8], b[8], g[8];
        unpack8(pdy[j][k], a);
        unpack8(px[j][k], b);
        unpack8(pgam[k], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xhat = fmaf(b[e], rs[j], nmr);
          const float gg = a[e] * g[e];
          s1 += gg;
          s2 = fmaf(gg, xhat, s2);
          dgam[8 * k + e] = fmaf(a[e], xhat, dgam[8 * k + e]);
          dbet[8 * k + e] += a[e];
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
      }
      if (lane == 0) {
        red[rg][j][warp_in_rg][0] = s1;
        red[rg][j][warp_in_rg][1] = s2;
      }
    }
    __syncthreads();
    // ---- dx
#pragma unroll
    for (int j = 0; j < RB; ++j) {
      const int64_t r = base + rg * RB + j;
      if (r < T) {
        const float m1 = (red[rg][j][0][0] + red[rg][j][1][0] + red[rg][j][2][0] + red[rg][j][3][0]) * inv_d;
        const float m2 = (red[rg][j][0][1] + red[rg][j][1][1] + red[rg][j][2][1] + red[rg][j][3][1]) * inv_d;
        // dx = rs * (dy * gamma - m1 - xhat * m2) = dy * (gamma * rs) - x * c2 + c0
        const float c2 = rs[j] * rs[j] * m2;
        const float c0 = fmaf(mu[j], c2, -m1 * rs[j]);
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          float a[8], b[8], g[8], o8[8];
          unpack8(pdy[j][k], a);
          unpack8(px[j][k], b);
          unpack8(pgam[k], g);
#pragma unroll
          for (int e = 0; e < 8; ++e) o8[e] = fmaf(a[e], g[e] * rs[j], fmaf(b[e], -c2, c0));
          if (resid != nullptr) {
            float q8[8];
            unpack8(pr[j][k], q8);
#pragma unroll
            for (int e = 0; e < 8; ++e) o8[e] += q8[e];                        // one rounding, at the store
          }
          *reinterpret_cast<uint4*>(dx + r * d + (t + 128 * k) * 8) = pack8(o8);
          if (pdx != nullptr) {
#pragma unroll
            for (int e = 0; e < 8; ++e) dxs[8 * k + e] += o8[e];
          }
        }
      }
    }
    __syncthreads();
  }
  ln_bwd_combine<EPT>(dgam, comb, pgamma + (int64_t)blockIdx.x * d, rg, t);
  ln_bwd_combine<EPT>(dbet, comb, pbeta + (int64_t)blockIdx.x * d, rg, t);
  if (pdx != nullptr) ln_bwd_combine<EPT>(dxs, comb, pdx + (int64_t)blockIdx.x * d, rg, t);
}

// The d = 2048 form: all 256 threads of a block work on one row (8 elements each), RB rows per
// iteration, two blocks per SM.  The column accumulators then take 24 registers instead of 48, so
// four rows of loads fit beside them in 128 registers; two resident blocks overlap one block's
// loads with the other's arithmetic (measured 1.2x faster than the two-group form at 8192 rows, 1.4x at 32768).
template <int RB>
__global__ void __launch_bounds__(256, 2)
    ln_bwd_row256_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                         const float* __restrict__ mean, const float* __restrict__ rstd,
                         const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ resid,
                         __nv_bfloat16* __restrict__ dx, float* __restrict__ pgamma, float* __restrict__ pbeta,
                         float* __restrict__ pdx, int64_t T) {
  constexpr int d = 2048;
  __shared__ float red[RB][8][2];
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  float g[8], dgam[8], dbet[8], dxs[8];
  unpack8(*reinterpret_cast<const uint4*>(gamma + t * 8), g);
#pragma unroll
  for (int e = 0; e < 8; ++e) dgam[e] = dbet[e] = dxs[e] = 0.f;
  const float inv_d = 1.0f / (float)d;
  const int64_t step = (int64_t)RB * gridDim.x;
  for (int64_t base = (int64_t)blockIdx.x * RB; base < T; base += step) {
    uint4 pdy[RB], px[RB], pr[RB];
    float mu[RB], rs[RB];
#pragma unroll
    for (int j = 0; j < RB; ++j) {
      const int64_t r = base + j;
      mu[j] = rs[j] = 0.f;
      pdy[j] = px[j] = pr[j] = make_uint4(0, 0, 0, 0);
      if (r < T) {
        const int64_t off = r * d + t * 8;
        mu[j] = mean[r];
        rs[j] = rstd[r];
        pdy[j] = *reinterpret_cast<const uint4*>(dy + off);
        px[j] = *reinterpret_cast<const uint4*>(x + off);
        if (resid != nullptr) pr[j] = *reinterpret_cast<const uint4*>(resid + off);
      }
    }
#pragma unroll
    for (int j = 0; j < RB; ++j) {
      float s1 = 0.f, s2 = 0.f, a[8], b[8];
      const float nmr = -mu[j] * rs[j];
      unpack8(pdy[j], a);
      unpack8(px[j], b);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xhat = fmaf(b[e], rs[j], nmr);
        const float gg = a[e] * g[e];
        s1 += gg;
        s2 = fmaf(gg, xhat, s2);
        dgam[e] = fmaf(a[e], xhat, dgam[e]);
        dbet[e] += a[e];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
      }
      if (lane == 0) {
        red[j][warp][0] = s1;
        red[j][warp][1] = s2;
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < RB; ++j) {
      const int64_t r = base + j;
      if (r < T) {
        float m1 = 0.f, m2 = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
          m1 += red[j][w][0];
          m2 += red[j][w][1];
        }
        m1 *= inv_d;
        m2 *= inv_d;
        const float c2 = rs[j] * rs[j] * m2;
        const float c0 = fmaf(mu[j], c2, -m1 * rs[j]);
        float a[8], b[8], o8[8];
        unpack8(pdy[j], a);
        unpack8(px[j], b);
#pragma unroll
        for (int e = 0; e < 8; ++e) o8[e] = fmaf(a[e], g[e] * rs[j], fmaf(b[e], -c2, c0));
        if (resid != nullptr) {
          float q8[8];
          unpack8(pr[j], q8);
#pragma unroll
          for (int e = 0; e < 8; ++e) o8[e] += q8[e];                          // one rounding, at the store
        }
        *reinterpret_cast<uint4*>(dx + r * d + t * 8) = pack8(o8);
        if (pdx != nullptr) {
#pragma unroll
          for (int e = 0; e < 8; ++e) dxs[e] += o8[e];
        }
      }
    }
    __syncthreads();
  }
  auto put = [&](float* row, const float* acc) {
    float4* o = reinterpret_cast<float4*>(row + (int64_t)blockIdx.x * d + t * 8);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  };
  put(pgamma, dgam);
  put(pbeta, dbet);
  if (pdx != nullptr) put(pdx, dxs);
}

// Adds the per-block partial sums of up to three arrays (blockIdx.y picks the array): a block
// owns 32 columns, its 8 warps split the partials.
struct LnBwdFinalizeArgs {
  const float* part[3];
  __nv_bfloat16* out[3];
};

__global__ void __launch_bounds__(256) ln_bwd_finalize_kernel(LnBwdFinalizeArgs f, int nparts, int d) {
  __shared__ float sa[8][33];
  const float* __restrict__ part = f.part[blockIdx.y];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float a = 0.f;
  if (c < d) {
    int p = w;
    for (; p + 56 < nparts; p += 64) {              // eight rows in flight
      float va[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) va[k] = __ldcg(part + (int64_t)(p + 8 * k) * d + c);
#pragma unroll
      for (int k = 0; k < 8; ++k) a += va[k];
    }
    for (; p < nparts; p += 8) a += __ldcg(part + (int64_t)p * d + c);
  }
  sa[w][lane] = a;
  __syncthreads();
  if (w == 0 && c < d) {
#pragma unroll
    for (int k = 1; k < 8; ++k) a += sa[k][lane];
    f.out[blockIdx.y][c] = __float2bfloat16_rn(a);
  }
}

// ---------------------------------------------------------------- GELU forward
__global__ void __launch_bounds__(256) gelu_fwd_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int64_t nvec) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    uint4 q[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) q[k] = in[i + k * stride];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float f[8];
      unpack8(q[k], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = gelu_tanh(f[e]);
      out[i + k * stride] = pack8(f);
    }
  }
  for (; i < nvec; i += stride) {
    float f[8];
    unpack8(in[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = gelu_tanh(f[e]);
    out[i] = pack8(f);
  }
}

// ---------------------------------------------------------------- residual add + layer norm
// One row per 128-thread block iteration.  With `branch` the row is x + branch, rounded to
// bf16 and written back over `branch` (it becomes the new residual stream); the statistics and
// the normalised output are taken from the rounded values, which is what the backward pass
// reads.  Writes y = (v - mean) * rstd * gamma + beta, mean and rstd (biased variance).
__device__ __forceinline__ float block_sum_128(float s, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  s = red[0] + red[1] + red[2] + red[3];
  __syncthreads();
  return s;
}

template <int EPT>
__global__ void __launch_bounds__(128) ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* branch,
                                                     const __nv_bfloat16* __restrict__ gamma,
                                                     const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                                                     float* __restrict__ mean, float* __restrict__ rstd, int64_t T, int d,
                                                     float eps) {
  constexpr int NV = EPT / 8;
  __shared__ float red[4];
  const int t = threadIdx.x;
  const float inv_d = 1.0f / (float)d;
  for (int64_t r = blockIdx.x; r < T; r += gridDim.x) {
    float v[EPT];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t off = r * d + (t + 128 * k) * 8;
      unpack8(*reinterpret_cast<const uint4*>(x + off), v + 8 * k);
      if (branch != nullptr) {
        float b[8];
        unpack8(*reinterpret_cast<const uint4*>(branch + off), b);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[8 * k + e] = round_bf16(v[8 * k + e] + b[e]);
        *reinterpret_cast<uint4*>(branch + off) = pack8(v + 8 * k);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[8 * k + e];
    }
    const float mu = block_sum_128(s, red) * inv_d;
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const float c = v[i] - mu;
      s2 += c * c;
    }
    const float rs = rsqrtf(block_sum_128(s2, red) * inv_d + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c0 = (t + 128 * k) * 8;
      float g[8], b[8], o[8];
      unpack8(*reinterpret_cast<const uint4*>(gamma + c0), g);
      unpack8(*reinterpret_cast<const uint4*>(beta + c0), b);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[8 * k + e] - mu) * rs * g[e] + b[e];
      *reinterpret_cast<uint4*>(y + r * d + c0) = pack8(o);
    }
    if (t == 0) {
      mean[r] = mu;
      rstd[r] = rs;
    }
  }
}

}  // namespace

int col_sum_row_splits(int64_t T, int N) {
  const int tiles = (N + kColTile - 1) / kColTile;
  int R = (148 * 4 + tiles - 1) / tiles;                       // about four blocks per SM (3, 5 and 6 measured slower)
  const int64_t max_r = (T + 4 * kRowLanes - 1) / (4 * kRowLanes);
  if (R > max_r) R = (int)max_r;
  if (R < 1) R = 1;
  return R;
}

cudaError_t launch_col_sum(const void* X, int64_t T, int N, void* out, float* partial, int* counters, int R,
                           cudaStream_t s) {
  if (T <= 0 || N <= 0) return cudaSuccess;
  if (N % 8 != 0) return cudaErrorInvalidValue;
  dim3 grid((N + kColTile - 1) / kColTile, R);
  col_sum_kernel<kColSum><<<grid, 256, 0, s>>>((const __nv_bfloat16*)X, T, N, (__nv_bfloat16*)out, partial, counters, nullptr,
                                               nullptr, nullptr);
  return cudaGetLastError();
}

cudaError_t launch_gelu_bwd_col_sum(const void* dg, const void* u, void* du, int64_t T, int N, void* out, float* partial,
                                    int* counters, int R, cudaStream_t s) {
  if (T <= 0 || N <= 0) return cudaSuccess;
  if (N % 8 != 0) return cudaErrorInvalidValue;
  dim3 grid((N + kColTile - 1) / kColTile, R);
  col_sum_kernel<kColGelu><<<grid, 256, 0, s>>>((const __nv_bfloat16*)dg, T, N, (__nv_bfloat16*)out, partial, counters,
                                                (const __nv_bfloat16*)u, (__nv_bfloat16*)du, nullptr);
  return cudaGetLastError();
}

cudaError_t launch_cat3_col_sum(const void* a, const void* b, const void* c, void* cat, int64_t T, int N, void* out,
                                float* partial, int* counters, int R, cudaStream_t s) {
  if (T <= 0 || N <= 0) return cudaSuccess;
  if (N % 24 != 0) return cudaErrorInvalidValue;          // three sources of a multiple of 8 columns each
  dim3 grid((N + kColTile - 1) / kColTile, R);
  col_sum_kernel<kColCat3><<<grid, 256, 0, s>>>((const __nv_bfloat16*)a, T, N, (__nv_bfloat16*)out, partial, counters,
                                                (const __nv_bfloat16*)b, (__nv_bfloat16*)cat, (const __nv_bfloat16*)c);
  return cudaGetLastError();
}

cudaError_t launch_gelu_fwd(const void* in, void* out, int64_t n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  if (n % 8 != 0) return cudaErrorInvalidValue;
  const int64_t nvec = n / 8;
  int64_t blocks = (nvec + 256 * 4 - 1) / (256 * 4);
  if (blocks > 148 * 8) blocks = 148 * 8;
  gelu_fwd_kernel<<<(int)blocks, 256, 0, s>>>((const uint4*)in, (uint4*)out, nvec);
  return cudaGetLastError();
}

cudaError_t launch_ln_fwd(const void* x, void* branch, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                          int64_t T, int d, float eps, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  int64_t blocks = T < 148 * 8 ? T : 148 * 8;
  auto* X = (const __nv_bfloat16*)x;
  auto* B = (__nv_bfloat16*)branch;
  auto* G = (const __nv_bfloat16*)gamma;
  auto* Be = (const __nv_bfloat16*)beta;
  auto* Y = (__nv_bfloat16*)y;
  switch (d / 128) {
    case 8: ln_fwd_kernel<8><<<(int)blocks, 128, 0, s>>>(X, B, G, Be, Y, mean, rstd, T, d, eps); break;
    case 16: ln_fwd_kernel<16><<<(int)blocks, 128, 0, s>>>(X, B, G, Be, Y, mean, rstd, T, d, eps); break;
    case 32: ln_fwd_kernel<32><<<(int)blocks, 128, 0, s>>>(X, B, G, Be, Y, mean, rstd, T, d, eps); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

int ln_bwd_blocks() { return 296; }      // at most two blocks per SM; each leaves one partial row per array

cudaError_t launch_ln_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma, void* dx,
                          const void* resid, void* dgamma, void* dbeta, void* dx_col_sum, float* scratch, int64_t T, int d,
                          cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  // d = 2048: one row per 256 threads, four rows per iteration, two blocks per SM; other widths: two
  // row groups of 128 threads per block, one block per SM, rows per group limited by registers
  const bool row256 = d == 2048;
  const int rows_per_iter = row256 ? 4 : 2 * (d <= 2048 ? 4 : 1);
  int blocks = row256 ? ln_bwd_blocks() : 148;
  if ((int64_t)blocks * rows_per_iter > T) blocks = (int)((T + rows_per_iter - 1) / rows_per_iter);
  auto* DY = (const __nv_bfloat16*)dy;
  auto* X = (const __nv_bfloat16*)x;
  auto* G = (const __nv_bfloat16*)gamma;
  auto* RS = (const __nv_bfloat16*)resid;
  auto* DX = (__nv_bfloat16*)dx;
  float* pgamma = scratch;
  float* pbeta = scratch + (int64_t)ln_bwd_blocks() * d;
  float* pdx = dx_col_sum != nullptr ? scratch + 2 * (int64_t)ln_bwd_blocks() * d : nullptr;
  switch (d / 128) {
    case 8: ln_bwd_kernel<8, 4><<<blocks, 256, 0, s>>>(DY, X, mean, rstd, G, RS, DX, pgamma, pbeta, pdx, T, d); break;
    case 16: ln_bwd_row256_kernel<4><<<blocks, 256, 0, s>>>(DY, X, mean, rstd, G, RS, DX, pgamma, pbeta, pdx, T); break;
    case 32: ln_bwd_kernel<32, 1><<<blocks, 256, 0, s>>>(DY, X, mean, rstd, G, RS, DX, pgamma, pbeta, pdx, T, d); break;
    default: return cudaErrorInvalidValue;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  LnBwdFinalizeArgs f;
  f.part[0] = pgamma, f.part[1] = pbeta, f.part[2] = pdx;
  f.out[0] = (__nv_bfloat16*)dgamma, f.out[1] = (__nv_bfloat16*)dbeta, f.out[2] = (__nv_bfloat16*)dx_col_sum;
  ln_bwd_finalize_kernel<<<dim3((d + 31) / 32, pdx != nullptr ? 3 : 2), 256, 0, s>>>(f, blocks, d);
  return cudaGetLastError();
}

}  // namespace pccl
