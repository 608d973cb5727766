// Reduction-shaped training kernels of the GPT backward pass: column sums (bias gradients)
// and layer-norm backward with its weight/bias gradients in one pass over the activations.
//
// The reference has no model code; these serve the in-repo ZeRO-3 engine, where the stock
// framework kernels for the same jobs cost about a tenth of the step.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

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

// ---------------------------------------------------------------- column sum
// out[c] = sum_r X[r, c]; X is [T, N] bf16 row-major with N % 8 == 0.  A block covers 64
// columns (8 threads x 16 bytes: one 128-byte line per row) and one slice of the rows; the
// last block to finish a column tile adds the slices' fp32 partial sums and writes bf16.
constexpr int kColTile = 64, kColRowsPerBlock = 32;

__global__ void __launch_bounds__(256) col_sum_kernel(const __nv_bfloat16* __restrict__ X, int64_t T, int N,
                                                      __nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                                                      int* __restrict__ counters) {
  __shared__ float red[kColRowsPerBlock][kColTile + 1];
  __shared__ int s_last;
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  const int col = blockIdx.x * kColTile + tx * 8;
  const int R = gridDim.y;
  const int64_t rows_per = (T + R - 1) / R;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per;
  const int64_t r1 = r0 + rows_per < T ? r0 + rows_per : T;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  if (col < N) {
    const __nv_bfloat16* base = X + col;
    int64_t r = r0 + ty;
    for (; r + 3 * kColRowsPerBlock < r1; r += 4 * kColRowsPerBlock) {
      uint4 q[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) q[k] = *reinterpret_cast<const uint4*>(base + (r + k * kColRowsPerBlock) * N);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f[8];
        unpack8(q[k], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += f[e];
      }
    }
    for (; r < r1; r += kColRowsPerBlock) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(base + r * N), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[ty][tx * 8 + e] = acc[e];
  __syncthreads();
  if (threadIdx.x < kColTile) {
    float s = 0.f;
#pragma unroll 8
    for (int y = 0; y < kColRowsPerBlock; ++y) s += red[y][threadIdx.x];
    const int c = blockIdx.x * kColTile + threadIdx.x;
    if (c < N) partial[(int64_t)blockIdx.y * N + c] = s;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(counters + blockIdx.x, 1) == R - 1;
  __syncthreads();
  if (s_last && threadIdx.x < kColTile) {
    __threadfence();
    const int c = blockIdx.x * kColTile + threadIdx.x;
    if (c < N) {
      float s = 0.f;
      for (int y = 0; y < R; ++y) s += __ldcg(partial + (int64_t)y * N + c);
      out[c] = __float2bfloat16_rn(s);
    }
    if (threadIdx.x == 0) counters[blockIdx.x] = 0;   // ready for the next call
  }
}

// ---------------------------------------------------------------- layer-norm backward
// One pass over dy and x:  dx = rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dy * gamma,
// and per-block partial sums of dgamma = sum_r dy * xhat, dbeta = sum_r dy.
// 128 threads work on one row (EPT = d / 128 elements each, in 16-byte vectors), two rows per
// block iteration; a second small kernel adds the partials.
template <int EPT>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                     const float* __restrict__ mean, const float* __restrict__ rstd,
                                                     const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ dx,
                                                     float* __restrict__ pgamma, float* __restrict__ pbeta, int64_t T, int d) {
  constexpr int NV = EPT / 8;
  __shared__ float red[2][4][2];
  const int rg = threadIdx.x >> 7, t = threadIdx.x & 127, warp_in_rg = t >> 5, lane = t & 31;
  float gam[EPT], dgam[EPT], dbet[EPT];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    unpack8(*reinterpret_cast<const uint4*>(gamma + (t + 128 * k) * 8), gam + 8 * k);
#pragma unroll
    for (int e = 0; e < 8; ++e) dgam[8 * k + e] = dbet[8 * k + e] = 0.f;
  }
  const float inv_d = 1.0f / (float)d;
  const int64_t iters = (T + 2 * (int64_t)gridDim.x - 1) / (2 * (int64_t)gridDim.x);
  for (int64_t it = 0; it < iters; ++it) {
    const int64_t r = (it * gridDim.x + blockIdx.x) * 2 + rg;
    const bool live = r < T;
    float g[EPT], xh[EPT];
    float s1 = 0.f, s2 = 0.f;
    float rs = 0.f;
    if (live) {
      const float mu = mean[r];
      rs = rstd[r];
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        float a[8], b[8];
        unpack8(*reinterpret_cast<const uint4*>(dy + r * d + (t + 128 * k) * 8), a);
        unpack8(*reinterpret_cast<const uint4*>(x + r * d + (t + 128 * k) * 8), b);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xhat = (b[e] - mu) * rs;
          const float gg = a[e] * gam[8 * k + e];
          xh[8 * k + e] = xhat;
          g[8 * k + e] = gg;
          s1 += gg;
          s2 += gg * xhat;
          dgam[8 * k + e] += a[e] * xhat;
          dbet[8 * k + e] += a[e];
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane == 0) {
      red[rg][warp_in_rg][0] = s1;
      red[rg][warp_in_rg][1] = s2;
    }
    __syncthreads();
    s1 = red[rg][0][0] + red[rg][1][0] + red[rg][2][0] + red[rg][3][0];
    s2 = red[rg][0][1] + red[rg][1][1] + red[rg][2][1] + red[rg][3][1];
    __syncthreads();
    if (live) {
      const float m1 = s1 * inv_d, m2 = s2 * inv_d;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        float o8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o8[e] = (g[8 * k + e] - m1 - xh[8 * k + e] * m2) * rs;
        *reinterpret_cast<uint4*>(dx + r * d + (t + 128 * k) * 8) = pack8(o8);
      }
    }
  }
  float* pg = pgamma + ((int64_t)blockIdx.x * 2 + rg) * d;
  float* pb = pbeta + ((int64_t)blockIdx.x * 2 + rg) * d;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int c = (t + 128 * k) * 8;
    *reinterpret_cast<float4*>(pg + c) = make_float4(dgam[8 * k], dgam[8 * k + 1], dgam[8 * k + 2], dgam[8 * k + 3]);
    *reinterpret_cast<float4*>(pg + c + 4) = make_float4(dgam[8 * k + 4], dgam[8 * k + 5], dgam[8 * k + 6], dgam[8 * k + 7]);
    *reinterpret_cast<float4*>(pb + c) = make_float4(dbet[8 * k], dbet[8 * k + 1], dbet[8 * k + 2], dbet[8 * k + 3]);
    *reinterpret_cast<float4*>(pb + c + 4) = make_float4(dbet[8 * k + 4], dbet[8 * k + 5], dbet[8 * k + 6], dbet[8 * k + 7]);
  }
}

// Adds the per-block partial sums: a block owns 32 columns, its 8 warps split the partials.
__global__ void __launch_bounds__(256) ln_bwd_finalize_kernel(const float* __restrict__ pgamma, const float* __restrict__ pbeta,
                                                              int nparts, int d, __nv_bfloat16* __restrict__ dgamma,
                                                              __nv_bfloat16* __restrict__ dbeta) {
  __shared__ float sa[8][33], sb[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float a = 0.f, b = 0.f;
  if (c < d)
    for (int p = w; p < nparts; p += 8) {
      a += pgamma[(int64_t)p * d + c];
      b += pbeta[(int64_t)p * d + c];
    }
  sa[w][lane] = a;
  sb[w][lane] = b;
  __syncthreads();
  if (w == 0 && c < d) {
#pragma unroll
    for (int k = 1; k < 8; ++k) {
      a += sa[k][lane];
      b += sb[k][lane];
    }
    dgamma[c] = __float2bfloat16_rn(a);
    dbeta[c] = __float2bfloat16_rn(b);
  }
}

}  // namespace

int col_sum_row_splits(int64_t T, int N) {
  const int tiles = (N + kColTile - 1) / kColTile;
  int R = (148 * 4 + tiles - 1) / tiles;
  const int64_t max_r = (T + 4 * kColRowsPerBlock - 1) / (4 * kColRowsPerBlock);
  if (R > max_r) R = (int)max_r;
  if (R < 1) R = 1;
  if (R > 64) R = 64;
  return R;
}

cudaError_t launch_col_sum(const void* X, int64_t T, int N, void* out, float* partial, int* counters, int R,
                           cudaStream_t s) {
  if (T <= 0 || N <= 0) return cudaSuccess;
  if (N % 8 != 0) return cudaErrorInvalidValue;
  dim3 grid((N + kColTile - 1) / kColTile, R);
  col_sum_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)X, T, N, (__nv_bfloat16*)out, partial, counters);
  return cudaGetLastError();
}

int ln_bwd_blocks() { return 148; }

cudaError_t launch_ln_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma, void* dx,
                          void* dgamma, void* dbeta, float* pgamma, float* pbeta, int64_t T, int d, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  int blocks = ln_bwd_blocks();
  if ((int64_t)blocks * 2 > T) blocks = (int)((T + 1) / 2);
  auto* DY = (const __nv_bfloat16*)dy;
  auto* X = (const __nv_bfloat16*)x;
  auto* G = (const __nv_bfloat16*)gamma;
  auto* DX = (__nv_bfloat16*)dx;
  switch (d / 128) {
    case 8: ln_bwd_kernel<8><<<blocks, 256, 0, s>>>(DY, X, mean, rstd, G, DX, pgamma, pbeta, T, d); break;
    case 16: ln_bwd_kernel<16><<<blocks, 256, 0, s>>>(DY, X, mean, rstd, G, DX, pgamma, pbeta, T, d); break;
    case 32: ln_bwd_kernel<32><<<blocks, 256, 0, s>>>(DY, X, mean, rstd, G, DX, pgamma, pbeta, T, d); break;
    default: return cudaErrorInvalidValue;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  ln_bwd_finalize_kernel<<<(d + 31) / 32, 256, 0, s>>>(pgamma, pbeta, blocks * 2, d, (__nv_bfloat16*)dgamma,
                                                         (__nv_bfloat16*)dbeta);
  return cudaGetLastError();
}

}  // namespace pccl
