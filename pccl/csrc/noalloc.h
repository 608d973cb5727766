// A reduce-scatter that never allocates.  This entry point has no counterpart in the
// reference: there every call takes its workspaces from the torch caching allocator
// (pccl/src/pccl.cpp:54-59,67-73).
//
// Who needs it.  Some programs that want to run this library's reduce-scatter kernel on
// one GPU (all ranks emulated by a single launch: the pre-flight self check of a training
// job, a unit test inside somebody else's process) are not allowed to allocate device
// memory when they call us: the host framework has already claimed the whole HBM for its
// own pool, so cudaMalloc simply fails; or the call sits on a latency-critical path where
// the device-wide synchronisation that cudaMalloc and cudaFree imply is not acceptable;
// or the caller is plain C and has no torch allocator to hand us.  The regular path needs
// a communicator whose heaps, staging areas and signal pads are allocated up front.
//
// What it does instead.  The staging areas for the partial sums, the signal pads and the
// status words of all emulated ranks live in ONE file-scope `static __device__` array of
// kNoAllocScratchBytes (about 8.6 MiB), which every GPU that loads the library holds until
// the process exits.  The caller passes only inputs and outputs.
//
// Rules for callers.
//  * Limits: 1..8 ranks, at most kNoAllocMaxBlockElems elements per rank's result; larger
//    requests are refused with an error message, nothing is launched.
//  * The first call on each device looks up the device address of the array
//    (cudaGetSymbolAddress, with that device current).  Make that first call outside of
//    any stream capture.
//  * All calls share the array and it keeps what the previous call left in it.  The flags
//    carry a per-device call number, so they need no clearing; the status words are cleared
//    on `stream` before every launch.  Two calls whose kernels overlap on the GPU (different
//    streams, no dependency) race on the array: order them.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PCCL_NOALLOC_MAX_RANKS 8
#define PCCL_NOALLOC_MAX_BLOCK_ELEMS 32768

// SUM reduce-scatter over `world` ranks emulated on the current device.
//   inputs[r]  : rank r's input, world * block_elems elements of `in_dtype`
//   outputs[r] : rank r's result, block_elems elements of `out_dtype`:
//                outputs[r][i] = scale * sum_s inputs[s][r * block_elems + i]   (fp32 accumulation)
//   dtypes     : 0 = bfloat16, 1 = float16, 2 = float32; out_dtype is in_dtype or float32
//   algo       : 0 = direct, 1 = ring, 2 = recursive halving (power-of-two world only)
//   stream     : the stream the work is enqueued on (the call does not wait for it)
// Returns 0 when the arguments were accepted and the work was ENQUEUED on `stream`; that says
// nothing yet about how the kernel fares.  Every wait inside the kernel is bounded (2 s): a wait
// that runs out leaves the outputs incomplete and records a status code in the static array,
// which pccl_reduce_scatter_noalloc_status reads back.  On a rejected argument or a failed
// enqueue the function returns a negative number and, when `err` is not null, writes a
// NUL-terminated explanation of at most `err_len` bytes into it.
int pccl_reduce_scatter_noalloc(const void* const* inputs, void* const* outputs, int world, uint64_t block_elems,
                                int in_dtype, int out_dtype, int algo, float scale, cudaStream_t stream, char* err,
                                size_t err_len);

// Outcome of the LAST call on the current device: waits for `stream`, then copies the status
// code of each of the `world` emulated ranks into codes[0..world) (0 = completed, 1 = a bounded
// wait ran out, 2 = gave up because another lane had failed).  Allocates nothing.  Returns 0
// when every rank completed, 1 when some code is non-zero, a negative number on a CUDA error
// or when no call has been made on this device yet.
int pccl_reduce_scatter_noalloc_status(cudaStream_t stream, int world, uint32_t* codes, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
