// Launchers of the elementwise training kernels (optim.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace pccl {

struct AdamWArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias1, bias2;      // 1/(1-beta1^t), 1/(1-beta2^t)
  float grad_scale;        // multiplies the stored gradient (e.g. loss-scale inverse)
  float max_grad_norm;     // <= 0: no clipping
};

// *out += sum(x^2); out must be zeroed by the caller.
cudaError_t launch_sq_norm(const void* x, int dtype_is_bf16, uint64_t n, float* out, cudaStream_t s);

cudaError_t launch_adamw(float* master, float* m, float* v, const void* grad, int grad_is_bf16, void* param_bf16,
                         uint64_t n, const AdamWArgs& a, const float* total_sq_norm, cudaStream_t s);

// In place: logits (bf16, rows x vocab) become d(loss)/d(logits) * grad_scale; *loss_sum += sum of row losses.
// A target that is neither ignore_index nor inside [0, vocab) makes its row count as ignored and
// adds one to *bad_targets (device int, may be nullptr); nothing is read out of bounds.
cudaError_t launch_ce_fwd_bwd(void* logits_bf16, const int64_t* targets, float* loss_sum, int64_t rows, int vocab,
                              int64_t row_stride, float grad_scale, int64_t ignore_index, int* bad_targets,
                              cudaStream_t s);

// out[c] = sum over rows of X[T, N] (bf16, N % 8 == 0).  partial: R*N floats, counters: ceil(N/64)
// ints that are zero on entry and zero again on exit.
int col_sum_row_splits(int64_t T, int N);
cudaError_t launch_col_sum(const void* X, int64_t T, int N, void* out, float* partial, int* counters, int R,
                           cudaStream_t s);

// du = dg * gelu'(u) (tanh form, bf16, [T, N]) and out[c] = sum over rows of du, in one pass.
// Scratch as for launch_col_sum.
cudaError_t launch_gelu_bwd_col_sum(const void* dg, const void* u, void* du, int64_t T, int N, void* out, float* partial,
                                    int* counters, int R, cudaStream_t s);

// cat = [a | b | c] (three [T, N/3] bf16 matrices side by side, N % 24 == 0) and out[c] = column
// sums of cat, in one pass.  Scratch as for launch_col_sum.
cudaError_t launch_cat3_col_sum(const void* a, const void* b, const void* c, void* cat, int64_t T, int N, void* out,
                                float* partial, int* counters, int R, cudaStream_t s);

// out = gelu(in), tanh form, bf16, n % 8 == 0, both 16-byte aligned.
cudaError_t launch_gelu_fwd(const void* in, void* out, int64_t n, cudaStream_t s);

// Layer norm over rows of d in {1024, 2048, 4096} bf16 elements.  branch != nullptr: the row is
// x + branch, written back over branch.  mean / rstd: T floats each.
cudaError_t launch_ln_fwd(const void* x, void* branch, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                          int64_t T, int d, float eps, cudaStream_t s);

// Layer-norm backward for bf16 activations with d in {1024, 2048, 4096}: writes dx (+ resid when
// given), dgamma, dbeta and, when dx_col_sum is given, the column sums of the stored dx.
// scratch: 3 * ln_bwd_blocks() * d floats.
int ln_bwd_blocks();
cudaError_t launch_ln_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma, void* dx,
                          const void* resid, void* dgamma, void* dbeta, void* dx_col_sum, float* scratch, int64_t T, int d,
                          cudaStream_t s);

}  // namespace pccl
