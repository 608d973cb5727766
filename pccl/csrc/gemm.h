// Blackwell GEMM and fused all-gather+GEMM (gemm_sm100.cu).
//
//   C[M,N] = A[M,K] * W[N,K]^T (+ bias[N])      bf16 in, fp32 accumulation in TMEM, bf16 out
//
// The CTA-pair form also takes either operand "transposed in memory" (a_mn / b_mn below), which
// gives the three products of a linear layer without a transposing copy:
//   forward        y  = x  * W^T      A = x  [M,K],            W = W  [N,K]
//   data gradient  dx = dy * W        A = dy [M,K],            W = W  stored [K,N]  (b_mn)
//   weight grad.   dW = dy^T * x      A = dy stored [K,M] (a_mn), W = x stored [K,N]  (b_mn)
//
// Plain mode: W is one [N,K] matrix in local memory.
// Fused mode: W is sharded by rows over the P members of a group (member p owns rows
// [p*N/P, (p+1)*N/P) in its symmetric heap).  The same kernel gathers the shards into a
// local [N,K] buffer over NVLink (a few "gatherer" CTAs driving the copy engine, one flag
// per 256-row panel) and multiplies: tiles whose panel is local start at once, the others
// as their panel lands.  The gathered matrix stays in the local buffer for later use.
//
// The reference has no GEMM at all; this is the "parameter all-gather fused with the
// first GEMM that consumes the gathered shard" of the ZeRO-3 path
// (hook point: pccl/patch_deepspeed.py:29-40 of the reference).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_types.h"

namespace pccl {

constexpr int kGemmBM = 128, kGemmBN = 256, kGemmBK = 64;

struct GemmArgs {
  int M, N, K;
  const void* A;        // [M,K] bf16 row-major, 16-byte aligned, K % 8 == 0
  const void* W;        // [N,K] bf16 row-major (plain mode: the weight; fused mode: the local gather buffer)
  void* C;              // [M,N] bf16 row-major, N % 8 == 0
  const void* bias;     // [N] bf16 or nullptr
  void* act_out;        // [M,N] bf16 or nullptr: second output, gelu(C) in the tanh form (C keeps the pre-activation)
  const void* gelu_grad_of;  // [M,N] bf16 or nullptr (CTA-pair form): every result is multiplied by gelu'(u) of the
                        // element of this tensor at its place before it is rounded: with A = dy, W = the second
                        // MLP weight and u = the first layer's pre-activation this is the whole GELU backward
  int* error;           // device int, set non-zero when a bounded wait ran out
  int two_cta;          // use the 2-SM MMA form (cta_group::2, one 256x256 tile per CTA pair); fused mode
                        // then needs an even gather_ctas (gatherers are whole pairs)
  // ---- operand layouts (CTA-pair form only; both 0 is the plain A[M,K], W[N,K] case)
  int a_mn;             // A is stored [K, M] row-major (M contiguous); M % 64 == 0
  int b_mn;             // W is stored [K, N] row-major (N contiguous); N % 64 == 0
  // ---- fused all-gather (gather_ctas == 0: plain GEMM)
  int gather_ctas;      // CTAs that move shards instead of multiplying
  GroupDev g;           // group, epoch, flags (filled by Comm::begin_call)
  uint64_t shard_off;   // offset of the [N/P, K] shard inside every member's heap
  uint32_t* panel_flags;  // device, ceil(N/256) counters, zeroed before the launch
  // A panel may be read once its counter has reached flag_target.  With gatherer CTAs that is
  // their number (each adds one per panel).  With gather_ctas == 0 and panel_flags set, somebody
  // else fills the local buffer and raises the counters (the copy engines, followed by
  // stream-ordered 32-bit writes of 1): then flag_target is 1 and all CTAs multiply.
  uint32_t flag_target;
  // ---- split of the last wave along K (CTA-pair form, plain mode; sk_tiles == 0: off)
  // With T tiles on G CTA pairs the last of ceil(T/G) rounds is only partly filled.  The first
  // sk_tiles tiles (in schedule order) are therefore not dealt out whole: their k-blocks form one
  // sequence that is cut into G equal runs, one per pair, so a tile may be computed by two (or
  // more) pairs.  The pair that holds a tile's first k-block finishes the tile; every other pair
  // with a piece of it writes its fp32 partial sums to its slot of sk_scratch and publishes
  // sk_epoch in sk_flags; the finisher adds them in its epilogue.  A pair works on its run first
  // and on whole tiles afterwards, so a partial is ready long before its finisher asks for it.
  int sk_tiles;
  float* sk_scratch;    // per pair 2 x 128 x 256 floats (256 KiB)
  uint32_t* sk_flags;   // per pair 8 words (one per epilogue warp of the pair), holding the last epoch written
  uint32_t sk_epoch;    // differs from launch to launch on the same scratch
  // ---- tiles handed out at run time (CTA-pair form; sched_counter == nullptr: static round-robin)
  // A persistent kernel that deals its tiles out in advance assumes that all its CTA pairs start
  // together.  Beside a collective kernel that holds a few SMs (a gradient reduction overlapping the
  // backward pass) some pairs start late and would then work through their whole share alone.  With
  // a counter, every pair takes the next tile when it is ready for one: late pairs simply take fewer.
  // The counter is never reset: a launch's tiles are counter values sched_base .. sched_base+tiles-1,
  // and the host advances its base by tiles + pairs per launch (every pair draws one value too many).
  uint32_t* sched_counter;   // device word, shared by the launches of one stream
  uint32_t sched_base;
  // ---- tuning knobs (0: the default)
  int max_pairs;        // use at most this many CTA pairs (plain mode)
  int group_m;          // row-tiles per band of the tile walk (plain mode; default 8); negative: bands of
                        // -group_m column-tiles walked along M instead
  // Plain CTA-pair products only: work in units of two vertically adjacent 256 x 256 tiles that share
  // their W half in shared memory (three quarters of the operand bytes per FLOP from L2; both TMEM
  // accumulators belong to one unit).  Ignored with sk_tiles, panel flags or M <= 256.
  int wide;
};

// Bytes of sk_scratch / words of sk_flags needed for `pairs` CTA pairs.
constexpr size_t kGemmSkScratchBytesPerPair = 2 * 128 * 256 * sizeof(float);
constexpr size_t kGemmSkFlagsPerPair = 8;

// How many leading tiles launch_gemm_sm100 would split along K for this shape on `sm_count` SMs
// (0: none).  The caller provides scratch for sm_count / 2 pairs when this is non-zero.
int gemm_sk_tiles(int M, int N, int K, int sm_count);

// Launches on `stream`.  Returns cudaErrorInvalidValue for shapes the kernel does not take.
cudaError_t launch_gemm_sm100(const GemmArgs& a, int sm_count, cudaStream_t stream);

}  // namespace pccl
