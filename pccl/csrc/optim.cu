// Elementwise training kernels of the ZeRO-3 engine: fused AdamW on a parameter shard,
// squared-norm partial sums for gradient clipping, and softmax cross-entropy computed
// forward and backward in one pass over the logits.
//
// The reference contains none of this (it hooks DeepSpeed, pccl/patch_deepspeed.py:95-126,
// and DeepSpeed brings its own optimizer); they exist here because the engine that stands
// in for DeepSpeed has to do the optimizer step inside the timed region.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "optim.h"

namespace pccl {

namespace {

constexpr int kOptThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <bool MAX>
__device__ __forceinline__ float block_reduce(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = MAX ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = MAX ? -INFINITY : 0.f;
  for (int i = 0; i < nw; ++i) r = MAX ? fmaxf(r, smem[i]) : r + smem[i];
  return r;
}

// ---------------------------------------------------------------- squared norm
// Grid-stride partial sums over 16-byte vectors (four in flight per thread), one atomicAdd per
// block into *out (zeroed by the caller).
template <typename T>
__device__ __forceinline__ float sq8(const uint4& q);
template <>
__device__ __forceinline__ float sq8<__nv_bfloat16>(const uint4& q) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  float a = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
    a += lo * lo + hi * hi;
  }
  return a;
}
template <>
__device__ __forceinline__ float sq8<float>(const uint4& q) {
  const float a = __uint_as_float(q.x), b = __uint_as_float(q.y), c = __uint_as_float(q.z), d = __uint_as_float(q.w);
  return a * a + b * b + c * c + d * d;
}

template <typename T>
__global__ void __launch_bounds__(kOptThreads) sq_norm_kernel(const T* __restrict__ x, uint64_t n, float* out) {
  __shared__ float red[32];
  constexpr uint64_t EPV = 16 / sizeof(T);
  float acc = 0.f;
  uint64_t done = 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
    const uint64_t nvec = n / EPV;
    const uint4* v = reinterpret_cast<const uint4*>(x);
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      const uint4 a = v[i], b = v[i + stride], c = v[i + 2 * stride], d = v[i + 3 * stride];
      acc += sq8<T>(a) + sq8<T>(b) + sq8<T>(c) + sq8<T>(d);
    }
    for (; i < nvec; i += stride) acc += sq8<T>(v[i]);
    done = nvec * EPV;
  }
  for (uint64_t i = done + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const float f = (float)x[i];
    acc += f * f;
  }
  acc = block_reduce<false>(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

// ---------------------------------------------------------------- AdamW
// One pass over the shard: reads grad, master, m, v; writes master, m, v and the bf16
// working copy that the next all-gather sends out.  total_sq_norm (device scalar, may be
// null) holds the squared global gradient norm; the clip factor is derived on the device,
// so no host synchronisation sits between the norm all-reduce and the update.
template <typename G>
__global__ void __launch_bounds__(kOptThreads)
    adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, const G* __restrict__ grad,
                 __nv_bfloat16* __restrict__ param, uint64_t n, AdamWArgs a, const float* total_sq_norm) {
  float clip = 1.0f;
  if (total_sq_norm != nullptr && a.max_grad_norm > 0.f) {
    const float norm = sqrtf(*total_sq_norm) * a.grad_scale;
    clip = fminf(1.0f, a.max_grad_norm / (norm + 1e-6f));
  }
  const float gs = a.grad_scale * clip;
  auto update = [&](float g, float& p, float& mi, float& vi) {
    g *= gs;
    mi = a.beta1 * mi + (1.f - a.beta1) * g;
    vi = a.beta2 * vi + (1.f - a.beta2) * g * g;
    const float mhat = mi * a.bias1, vhat = vi * a.bias2;
    p = p * (1.f - a.lr * a.weight_decay) - a.lr * mhat / (sqrtf(vhat) + a.eps);
  };
  // Four elements per thread and iteration through 16-byte accesses (8 bytes for the bf16 sides),
  // two such groups in flight: the pass is pure streaming (28 bytes per parameter) and wants many
  // wide requests outstanding.  Pointers that are not 16-byte aligned take the scalar loop.
  uint64_t done = 0;
  const uintptr_t align = reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                          reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(param);
  if ((align & 15u) == 0) {
    const uint64_t nvec = n / 4;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    float4* pm = reinterpret_cast<float4*>(master);
    float4* mm = reinterpret_cast<float4*>(m);
    float4* vv = reinterpret_cast<float4*>(v);
    auto load_g = [&](uint64_t i, float* g) {
      if constexpr (sizeof(G) == 2) {
        const uint2 q = __ldcs(reinterpret_cast<const uint2*>(grad) + i);
        g[0] = __uint_as_float(q.x << 16); g[1] = __uint_as_float(q.x & 0xffff0000u);
        g[2] = __uint_as_float(q.y << 16); g[3] = __uint_as_float(q.y & 0xffff0000u);
      } else {
        const float4 q = __ldcs(reinterpret_cast<const float4*>(grad) + i);
        g[0] = q.x; g[1] = q.y; g[2] = q.z; g[3] = q.w;
      }
    };
    auto one = [&](uint64_t i, const float* g, float4 p4, float4 m4, float4 v4) {
      update(g[0], p4.x, m4.x, v4.x);
      update(g[1], p4.y, m4.y, v4.y);
      update(g[2], p4.z, m4.z, v4.z);
      update(g[3], p4.w, m4.w, v4.w);
      __stcs(pm + i, p4);
      __stcs(mm + i, m4);
      __stcs(vv + i, v4);
      const __nv_bfloat162 lo = __floats2bfloat162_rn(p4.x, p4.y), hi = __floats2bfloat162_rn(p4.z, p4.w);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&lo);
      o.y = *reinterpret_cast<const uint32_t*>(&hi);
      reinterpret_cast<uint2*>(param)[i] = o;          // the working copy is read again soon: default caching
    };
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < nvec; i += 2 * stride) {
      float g0[4], g1[4];
      load_g(i, g0);
      load_g(i + stride, g1);
      const float4 p0 = __ldcs(pm + i), m0 = __ldcs(mm + i), v0 = __ldcs(vv + i);
      const float4 p1 = __ldcs(pm + i + stride), m1 = __ldcs(mm + i + stride), v1 = __ldcs(vv + i + stride);
      one(i, g0, p0, m0, v0);
      one(i + stride, g1, p1, m1, v1);
    }
    for (; i < nvec; i += stride) {
      float g0[4];
      load_g(i, g0);
      one(i, g0, __ldcs(pm + i), __ldcs(mm + i), __ldcs(vv + i));
    }
    done = nvec * 4;
  }
  for (uint64_t i = done + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    float p = master[i], mi = m[i], vi = v[i];
    update((float)grad[i], p, mi, vi);
    master[i] = p;
    m[i] = mi;
    v[i] = vi;
    param[i] = __float2bfloat16_rn(p);
  }
}

// ---------------------------------------------------------------- softmax cross-entropy, fwd + bwd
// One CTA per row.  The row of logits is read from HBM once into shared memory, reduced
// (max, sum of exponentials), and overwritten in place with d(loss)/d(logits) =
// (softmax - onehot) * grad_scale.  loss_sum accumulates the per-row losses.
__global__ void __launch_bounds__(512) ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                         float* loss_sum, int vocab, int64_t row_stride, float grad_scale,
                                                         int64_t ignore_index, int* bad_targets) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* row_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __shared__ float red[32];
  __nv_bfloat16* row = logits + (int64_t)blockIdx.x * row_stride;
  const int64_t tgt = targets[blockIdx.x];
  const int nvec = vocab >> 3;  // 8 bf16 = 16 bytes (row_stride and vocab are multiples of 8)
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 q = reinterpret_cast<const uint4*>(row)[i];
    reinterpret_cast<uint4*>(row_s)[i] = q;
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      mx = fmaxf(mx, fmaxf(f.x, f.y));
    }
  }
  for (int i = (nvec << 3) + threadIdx.x; i < vocab; i += blockDim.x) {
    row_s[i] = row[i];
    mx = fmaxf(mx, __bfloat162float(row[i]));
  }
  mx = block_reduce<true>(mx, red);
  float sum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) sum += __expf(__bfloat162float(row_s[i]) - mx);
  sum = block_reduce<false>(sum, red);
  // A target outside [0, vocab) that is not the ignore index would index past the row in shared
  // memory: such a row counts as ignored (no loss, zero gradient) and is reported through
  // *bad_targets, so a corrupt label never becomes an out-of-bounds access.
  const bool out_of_range = tgt != ignore_index && (tgt < 0 || tgt >= (int64_t)vocab);
  if (out_of_range && threadIdx.x == 0 && bad_targets != nullptr) atomicAdd(bad_targets, 1);
  const bool ignored = tgt == ignore_index || out_of_range;
  if (threadIdx.x == 0 && !ignored) {
    const float lt = __bfloat162float(row_s[tgt]);
    atomicAdd(loss_sum, (mx + logf(sum) - lt));
  }
  const float inv = ignored ? 0.f : grad_scale / sum;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 q = reinterpret_cast<const uint4*>(row_s)[i];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      const int c = (i << 3) + 2 * k;
      f.x = __expf(f.x - mx) * inv - ((c == tgt && !ignored) ? grad_scale : 0.f);
      f.y = __expf(f.y - mx) * inv - ((c + 1 == tgt && !ignored) ? grad_scale : 0.f);
      h[k] = __floats2bfloat162_rn(f.x, f.y);
    }
    reinterpret_cast<uint4*>(row)[i] = q;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < vocab; i += blockDim.x) {
    const float p = __expf(__bfloat162float(row_s[i]) - mx) * inv - ((i == tgt && !ignored) ? grad_scale : 0.f);
    row[i] = __float2bfloat16_rn(p);
  }
}

int grid_for(uint64_t n, int threads, int per_thread) {
  uint64_t blocks = (n + (uint64_t)threads * per_thread - 1) / ((uint64_t)threads * per_thread);
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return (int)blocks;
}

}  // namespace

cudaError_t launch_sq_norm(const void* x, int dtype_is_bf16, uint64_t n, float* out, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const int grid = grid_for(n, kOptThreads, 16);
  if (dtype_is_bf16) sq_norm_kernel<<<grid, kOptThreads, 0, s>>>((const __nv_bfloat16*)x, n, out);
  else sq_norm_kernel<<<grid, kOptThreads, 0, s>>>((const float*)x, n, out);
  return cudaGetLastError();
}

cudaError_t launch_adamw(float* master, float* m, float* v, const void* grad, int grad_is_bf16, void* param_bf16,
                         uint64_t n, const AdamWArgs& a, const float* total_sq_norm, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const int grid = grid_for(n, kOptThreads, 8);
  if (grad_is_bf16)
    adamw_kernel<<<grid, kOptThreads, 0, s>>>(master, m, v, (const __nv_bfloat16*)grad, (__nv_bfloat16*)param_bf16, n, a,
                                              total_sq_norm);
  else
    adamw_kernel<<<grid, kOptThreads, 0, s>>>(master, m, v, (const float*)grad, (__nv_bfloat16*)param_bf16, n, a,
                                              total_sq_norm);
  return cudaGetLastError();
}

cudaError_t launch_ce_fwd_bwd(void* logits_bf16, const int64_t* targets, float* loss_sum, int64_t rows, int vocab,
                              int64_t row_stride, float grad_scale, int64_t ignore_index, int* bad_targets,
                              cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  const size_t smem = (size_t)vocab * sizeof(__nv_bfloat16);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;   // the row must fit into shared memory
  // the shared-memory limit is a per-device attribute of the function
  static bool configured[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(ce_fwd_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  ce_fwd_bwd_kernel<<<(unsigned)rows, 512, smem, s>>>((__nv_bfloat16*)logits_bf16, targets, loss_sum, vocab, row_stride,
                                                      grad_scale, ignore_index, bad_targets);
  return cudaGetLastError();
}

}  // namespace pccl
