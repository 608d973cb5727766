// Python bindings of the native layer (module pccl._C).
//
// Role of pccl/src/pccl.cpp in the reference (reduce_scatter_mpi / all_gather_mpi with
// their argument checks, :11-148) and of the unbuilt pccl/src/yacl.cpp (all_reduce_mpi,
// :146-184).  Differences: sizes are 64-bit, bf16/fp16/fp32 are accepted for the
// reductions (the reference takes fp32 only, pccl.cpp:42-45), the algorithm is an enum
// that includes ring all-gather, and errors surface as Python exceptions.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <optional>

#include "comm.h"
#include "schedule.h"
#include "segments.h"

namespace py = pybind11;
using namespace pccl;

namespace {

int to_dtype(at::ScalarType t) {
  switch (t) {
    case at::kBFloat16: return kBF16;
    case at::kHalf: return kF16;
    case at::kFloat: return kF32;
    default: throw Error("unsupported dtype for a reduction: expected bfloat16, float16 or float32");
  }
}

py::tuple step_tuple(const Step& s) { return py::make_tuple(s.dst, s.src, s.send_first, s.recv_first, s.nblocks); }

cudaStream_t current_stream(int device) { return at::cuda::getCurrentCUDAStream(device).stream(); }

void check_tensor(const at::Tensor& t, const char* name, int device) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.get_device() == device, name, " lives on cuda:", t.get_device(), ", the communicator on cuda:", device);
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

struct LocalList {
  int n;          // number of local ranks driven by this call
  int first;      // group index of local slot 0
};

LocalList local_list(Comm& c, int gid, size_t given, const char* what) {
  const GroupState& gs = c.group(gid);
  TORCH_CHECK(gs.my_index >= 0, "this rank is not a member of the group");
  LocalList l;
  l.n = c.nlocal() > 1 ? (int)gs.ranks.size() : 1;
  l.first = c.nlocal() > 1 ? 0 : gs.my_index;
  TORCH_CHECK((int)given == l.n, what, ": expected ", l.n, " tensor(s), one per local rank, got ", given);
  return l;
}

// Offset of tensor i inside the heap of the rank that owns local slot i; all slots must
// agree (the buffer is symmetric) or none may be in the heap.
int64_t symmetric_offset(Comm& c, int gid, const LocalList& l, const std::vector<at::Tensor>& ts) {
  const GroupState& gs = c.group(gid);
  int64_t off = -2;
  for (int i = 0; i < l.n; ++i) {
    const int owner = gs.ranks[l.first + i];
    const int64_t o = c.offset_of((uint64_t)ts[i].data_ptr(), (uint64_t)ts[i].nbytes(), owner);
    if (off == -2) off = o;
    if (o != off) return -1;   // emulated ranks at different offsets: treat as private memory
  }
  return off;
}

// ------------------------------------------------------------------ flat all-gather
void all_gather(Comm& c, int gid, std::vector<at::Tensor> outs, std::vector<at::Tensor> ins, int algo, int nlanes) {
  const LocalList l = local_list(c, gid, outs.size(), "all_gather outputs");
  TORCH_CHECK(ins.size() == outs.size(), "all_gather: need one input per output");
  const int P = c.group_size(gid);
  const int dev = c.device();
  c10::cuda::CUDAGuard guard(dev);
  for (int i = 0; i < l.n; ++i) {
    check_tensor(outs[i], "output_tensor", dev);
    check_tensor(ins[i], "input_tensor", dev);
    TORCH_CHECK(outs[i].scalar_type() == ins[i].scalar_type(), "input and output dtypes differ");
    TORCH_CHECK(outs[i].numel() == ins[i].numel() * P, "output_tensor must hold world_size * input elements (", P, " * ",
                ins[i].numel(), "), got ", outs[i].numel());
    TORCH_CHECK(ins[i].nbytes() == ins[0].nbytes(), "all ranks must contribute the same number of bytes");
  }
  const uint64_t n = (uint64_t)ins[0].nbytes();
  if (n == 0) return;
  cudaStream_t stream = current_stream(dev);
  if (P == 1) {
    // A group of one: the gather is a device-to-device copy, which the copy engine does
    // without occupying an SM.
    if (outs[0].data_ptr() != ins[0].data_ptr())
      PCCL_CUDA(cudaMemcpyAsync(outs[0].data_ptr(), ins[0].data_ptr(), n, cudaMemcpyDeviceToDevice, stream));
    return;
  }
  const int64_t out_off = symmetric_offset(c, gid, l, outs);
  const int64_t in_off = symmetric_offset(c, gid, l, ins);

  AllGatherArgs a;
  std::memset(&a, 0, sizeof(a));
  a.algo = algo;
  a.nsub = 1;
  a.out_src_stride = n;
  a.in_sub_stride = n;
  if (algo == kMultimem) TORCH_CHECK(n % 16 == 0, "multimem all-gather needs a multiple of 16 bytes per rank");

  if (algo == kEager) {
    // Small messages on the world group: the direct schedule into this call's half of the eager
    // area, no entry handshake; the result is copied out of the area by the same kernel.
    TORCH_CHECK(gid == 0, "the eager variant runs on the world group only");
    TORCH_CHECK(c.eager_capacity() >= (uint64_t)P * n, "message too large for the eager area: ", P * n, " bytes, capacity ",
                c.eager_capacity());
    const uint64_t slot = c.eager_capacity() / (uint64_t)P / 16 * 16;
    a.algo = kDirect;
    a.eager = 1;
    a.recv_off = c.next_eager_half();
    a.src_stride = slot;
    a.sub_bytes = n;
    for (int i = 0; i < l.n; ++i) {
      a.in[i] = (const char*)ins[i].data_ptr();
      a.out[i] = (char*)outs[i].data_ptr();
    }
    c.all_gather(gid, a, nlanes, stream);
    return;
  }

  if (algo == kPull) {
    // Results go straight to the outputs; only a private input needs staging.
    uint64_t cap = n;
    if (in_off < 0) {
      cap = c.staging_bytes() / 16 * 16;
      TORCH_CHECK(cap > 0, "no staging area configured for non-symmetric tensors");
    }
    for (uint64_t e0 = 0; e0 < n; e0 += cap) {
      const uint64_t len = std::min(cap, n - e0);
      a.sub_bytes = len;
      for (int i = 0; i < l.n; ++i) {
        a.in[i] = in_off < 0 ? (const char*)ins[i].data_ptr() + e0 : nullptr;
        a.out[i] = (char*)outs[i].data_ptr() + e0;
      }
      a.in_off = in_off < 0 ? c.staging_off() : (uint64_t)in_off + e0;
      a.recv_off = 0;
      c.all_gather(gid, a, nlanes, stream);
    }
    return;
  }

  if (out_off >= 0) {
    // Zero-copy: peers write into the symmetric output.
    if (algo == kMultimem) TORCH_CHECK(out_off % 16 == 0, "multimem needs a 16-byte aligned symmetric output");
    a.recv_off = (uint64_t)out_off;
    a.src_stride = n;
    a.sub_bytes = n;
    for (int i = 0; i < l.n; ++i) {
      const bool aliased = (const char*)ins[i].data_ptr() == (const char*)outs[i].data_ptr() + (uint64_t)(l.first + i) * n;
      a.in[i] = aliased ? nullptr : (const char*)ins[i].data_ptr();
      a.out[i] = nullptr;
    }
    c.all_gather(gid, a, nlanes, stream);
    return;
  }

  // Private output: land in the staging area, then copy out inside the same kernel.
  const uint64_t cap = c.staging_bytes() / P / 16 * 16;
  TORCH_CHECK(cap > 0, "no staging area configured for non-symmetric tensors");
  for (uint64_t e0 = 0; e0 < n; e0 += cap) {
    const uint64_t len = std::min(cap, n - e0);
    a.recv_off = c.staging_off();
    a.src_stride = cap;
    a.sub_bytes = len;
    for (int i = 0; i < l.n; ++i) {
      a.in[i] = (const char*)ins[i].data_ptr() + e0;
      a.out[i] = (char*)outs[i].data_ptr() + e0;
    }
    c.all_gather(gid, a, nlanes, stream);
  }
}

// All-gather by the GPU's copy engines: this rank copies every peer's contribution out of the
// peer's symmetric heap into its own output, one cudaMemcpyAsync per peer on the current stream,
// peers in ring order (me+1, me+2, ...) so that at any moment every source serves one reader.
// No kernel runs and no SM is occupied, which is what a gather that overlaps GEMMs wants.
// There is no handshake with the peers either: the caller guarantees that the peers' inputs are
// complete before the call and stay unchanged until every rank's copy has finished (parameter
// shards between two optimizer steps, behind a barrier).  One rank per process only.
void all_gather_copy_engine(Comm& c, int gid, at::Tensor out, at::Tensor in) {
  TORCH_CHECK(c.nlocal() == 1, "the copy-engine all-gather runs one rank per process");
  const GroupState& gs = c.group(gid);
  TORCH_CHECK(gs.my_index >= 0, "this rank is not a member of the group");
  const int P = (int)gs.ranks.size(), me = gs.my_index;
  const int dev = c.device();
  c10::cuda::CUDAGuard guard(dev);
  check_tensor(out, "output_tensor", dev);
  check_tensor(in, "input_tensor", dev);
  TORCH_CHECK(out.scalar_type() == in.scalar_type(), "input and output dtypes differ");
  TORCH_CHECK(out.numel() == in.numel() * P, "output_tensor must hold world_size * input elements");
  const uint64_t n = (uint64_t)in.nbytes();
  if (n == 0) return;
  const int64_t in_off = c.offset_of((uint64_t)in.data_ptr(), n, c.rank());
  TORCH_CHECK(in_off >= 0 || P == 1, "the copy-engine all-gather reads the peers' inputs: allocate input_tensor with "
                                     "pccl.empty_symmetric");
  cudaStream_t stream = current_stream(dev);
  char* o = (char*)out.data_ptr();
  for (int k = 1; k < P; ++k) {
    const int p = (me + k) % P;
    PCCL_CUDA(cudaMemcpyAsync(o + (uint64_t)p * n, (const void*)(c.heap_base(gs.ranks[p]) + (uint64_t)in_off), n,
                              cudaMemcpyDeviceToDevice, stream));
  }
  if (o + (uint64_t)me * n != (char*)in.data_ptr())
    PCCL_CUDA(cudaMemcpyAsync(o + (uint64_t)me * n, in.data_ptr(), n, cudaMemcpyDeviceToDevice, stream));
}

// Layout-general all-gather used by the 2-D hierarchy: every quantity is given in bytes.
void all_gather_raw(Comm& c, int gid, int algo, int nlanes, std::vector<uint64_t> in_ptrs, std::vector<uint64_t> out_ptrs,
                    uint64_t recv_off, uint64_t out_src_stride, uint64_t out_sub_stride, uint64_t src_stride,
                    uint64_t sub_stride, uint64_t sub_bytes, uint64_t in_sub_stride, int nsub, uint64_t in_off) {
  const LocalList l = local_list(c, gid, in_ptrs.size(), "all_gather_raw inputs");
  TORCH_CHECK(out_ptrs.size() == in_ptrs.size(), "all_gather_raw: need one output slot per input");
  c10::cuda::CUDAGuard guard(c.device());
  AllGatherArgs a;
  std::memset(&a, 0, sizeof(a));
  a.algo = algo;
  for (int i = 0; i < l.n; ++i) {
    a.in[i] = (const char*)in_ptrs[i];
    a.out[i] = (char*)out_ptrs[i];
  }
  a.recv_off = recv_off;
  a.out_src_stride = out_src_stride;
  a.out_sub_stride = out_sub_stride;
  a.src_stride = src_stride;
  a.sub_stride = sub_stride;
  a.sub_bytes = sub_bytes;
  a.in_sub_stride = in_sub_stride;
  a.nsub = nsub;
  a.in_off = in_off;
  if (sub_bytes == 0) return;
  c.all_gather(gid, a, nlanes, current_stream(c.device()));
}

// ------------------------------------------------------------------ flat reduce-scatter
void reduce_scatter(Comm& c, int gid, std::vector<at::Tensor> outs, std::vector<at::Tensor> ins, int algo, int nlanes,
                    double scale, std::optional<at::ScalarType> wire) {
  const LocalList l = local_list(c, gid, outs.size(), "reduce_scatter outputs");
  TORCH_CHECK(ins.size() == outs.size(), "reduce_scatter: need one input per output");
  const int P = c.group_size(gid);
  const int dev = c.device();
  c10::cuda::CUDAGuard guard(dev);
  for (int i = 0; i < l.n; ++i) {
    check_tensor(outs[i], "output_tensor", dev);
    check_tensor(ins[i], "input_tensor", dev);
    TORCH_CHECK(ins[i].numel() % P == 0, "input_tensor numel (", ins[i].numel(), ") must be divisible by world size ", P);
    TORCH_CHECK(outs[i].numel() == ins[i].numel() / P, "output_tensor must hold input numel / world_size elements");
    TORCH_CHECK(ins[i].numel() == ins[0].numel() && ins[i].scalar_type() == ins[0].scalar_type() &&
                    outs[i].scalar_type() == outs[0].scalar_type(),
                "all ranks must pass tensors of the same size and dtype");
  }
  const int tin = to_dtype(ins[0].scalar_type());
  const int tout = to_dtype(outs[0].scalar_type());
  const int tw = wire.has_value() ? to_dtype(*wire) : tin;
  TORCH_CHECK(tw == tin || tw == kF32, "partial sums travel in the input dtype or in float32");
  TORCH_CHECK(tout == tin || tout == kF32 || (tin == kF32 && tout == kBF16),
              "output dtype must be the input dtype or float32");
  const uint64_t n = (uint64_t)outs[0].numel();
  if (n == 0) return;
  cudaStream_t stream = current_stream(dev);
  if (P == 1 && tin == tout && scale == 1.0) {
    // A group of one with nothing to scale or convert: the result is the input, and the copy
    // engine moves it without occupying an SM (as the one-rank all-gather does).
    if (outs[0].data_ptr() != ins[0].data_ptr())
      PCCL_CUDA(cudaMemcpyAsync(outs[0].data_ptr(), ins[0].data_ptr(), outs[0].nbytes(), cudaMemcpyDeviceToDevice, stream));
    return;
  }
  const int64_t in_off = symmetric_offset(c, gid, l, ins);
  const uint64_t si = dtype_size(tin), sw = dtype_size(tw), so = dtype_size(tout);

  ReduceScatterArgs a;
  std::memset(&a, 0, sizeof(a));
  a.algo = algo;
  a.in_dtype = tin;
  a.wire_dtype = tw;
  a.out_dtype = tout;
  a.nsub = 1;
  a.scale = (float)scale;
  a.dst_stride = n * si;
  a.out_sub_stride = n * so;

  if (algo == kPull || algo == kMultimem) {
    TORCH_CHECK(in_off >= 0, "the pull and multimem reduce-scatter read the peers' inputs: allocate input_tensor "
                             "with pccl.empty_symmetric or pick another algorithm");
    if (algo == kMultimem) {
      TORCH_CHECK(in_off % 16 == 0 && (n * si) % 16 == 0, "multimem reduce-scatter needs 16-byte aligned blocks");
      TORCH_CHECK(tw == tin, "multimem reduce-scatter has no wire dtype");
    }
    a.in_off = (uint64_t)in_off;
    a.sub_elems = n;
    for (int i = 0; i < l.n; ++i) {
      a.in[i] = nullptr;
      a.out[i] = (char*)outs[i].data_ptr();
    }
    c.reduce_scatter(gid, a, nlanes, stream);
    return;
  }

  if (algo == kEager) {
    // Small messages on the world group: every rank pushes block d of its input into rank d's half
    // of the eager area (no entry handshake) and sums what it received.
    TORCH_CHECK(gid == 0, "the eager variant runs on the world group only");
    TORCH_CHECK(P == 1 || c.eager_capacity() >= (uint64_t)(P - 1) * n * sw, "message too large for the eager area");
    a.algo = kDirect;
    a.eager = 1;
    a.stage_off = c.next_eager_half();
    a.sub_elems = n;
    for (int i = 0; i < l.n; ++i) {
      a.in[i] = (const char*)ins[i].data_ptr();
      a.out[i] = (char*)outs[i].data_ptr();
    }
    c.reduce_scatter(gid, a, nlanes, stream);
    return;
  }

  // Push variants: partial sums land in the staging area of the receiver.
  uint64_t cap = n;
  if (P > 1) {
    cap = c.staging_bytes() / (uint64_t)(P - 1) / sw / 8 * 8;
    TORCH_CHECK(cap > 0, "staging area too small for a reduce-scatter");
  }
  for (uint64_t e0 = 0; e0 < n; e0 += cap) {
    const uint64_t len = std::min(cap, n - e0);
    a.stage_off = c.staging_off();
    a.sub_elems = len;
    for (int i = 0; i < l.n; ++i) {
      a.in[i] = (const char*)ins[i].data_ptr() + e0 * si;
      a.out[i] = (char*)outs[i].data_ptr() + e0 * so;
    }
    c.reduce_scatter(gid, a, nlanes, stream);
  }
}

void reduce_scatter_raw(Comm& c, int gid, int algo, int nlanes, int in_dtype, int wire_dtype, int out_dtype,
                        std::vector<uint64_t> in_ptrs, std::vector<uint64_t> out_ptrs, uint64_t in_off, uint64_t stage_off,
                        uint64_t dst_stride, uint64_t sub_stride, uint64_t sub_elems, uint64_t out_sub_stride, int nsub,
                        double scale) {
  const LocalList l = local_list(c, gid, in_ptrs.size(), "reduce_scatter_raw inputs");
  TORCH_CHECK(out_ptrs.size() == in_ptrs.size(), "reduce_scatter_raw: need one output per input");
  c10::cuda::CUDAGuard guard(c.device());
  ReduceScatterArgs a;
  std::memset(&a, 0, sizeof(a));
  a.algo = algo;
  a.in_dtype = in_dtype;
  a.wire_dtype = wire_dtype;
  a.out_dtype = out_dtype;
  for (int i = 0; i < l.n; ++i) {
    a.in[i] = (const char*)in_ptrs[i];
    a.out[i] = (char*)out_ptrs[i];
  }
  a.in_off = in_off;
  a.stage_off = stage_off;
  a.dst_stride = dst_stride;
  a.sub_stride = sub_stride;
  a.sub_elems = sub_elems;
  a.out_sub_stride = out_sub_stride;
  a.nsub = nsub;
  a.scale = (float)scale;
  if (sub_elems == 0) return;
  c.reduce_scatter(gid, a, nlanes, current_stream(c.device()));
}

// ------------------------------------------------------------------ all-reduce (in place)
void all_reduce(Comm& c, int gid, std::vector<at::Tensor> ts, int algo, int nlanes, double scale) {
  const LocalList l = local_list(c, gid, ts.size(), "all_reduce tensors");
  const int dev = c.device();
  c10::cuda::CUDAGuard guard(dev);
  for (int i = 0; i < l.n; ++i) {
    check_tensor(ts[i], "tensor", dev);
    TORCH_CHECK(ts[i].numel() == ts[0].numel() && ts[i].scalar_type() == ts[0].scalar_type(),
                "all ranks must pass tensors of the same size and dtype");
  }
  const int dt = to_dtype(ts[0].scalar_type());
  const uint64_t n = (uint64_t)ts[0].numel(), s = dtype_size(dt);
  if (n == 0) return;
  cudaStream_t stream = current_stream(dev);
  const int64_t off = symmetric_offset(c, gid, l, ts);
  const int P = c.group_size(gid);
  if ((algo == kRing || algo == kRecursive) && P > 1 && n % (uint64_t)P == 0) {
    // The reference's composition (pccl/src/yacl.cpp:146-177): reduce-scatter, then all-gather, both
    // ring or both recursive; here one launch per chunk, in place (each rank's block of the sum
    // is formed in its own slot of the tensor and gathered from there).
    const uint64_t blk = n / (uint64_t)P;            // elements per rank
    uint64_t cap = blk;
    if (off < 0) {
      // private tensors: partial sums and gathered blocks both pass through the staging area
      cap = std::min(c.staging_bytes() / (uint64_t)(P - 1) / s, c.staging_bytes() / (uint64_t)P / s) / 8 * 8;
      TORCH_CHECK(cap > 0, "staging area too small for an all-reduce");
    } else {
      cap = c.staging_bytes() / (uint64_t)(P - 1) / s / 8 * 8;   // the reduce-scatter phase stages partial sums
      TORCH_CHECK(cap > 0, "staging area too small for an all-reduce");
    }
    for (uint64_t e0 = 0; e0 < blk; e0 += cap) {
      const uint64_t len = std::min(cap, blk - e0);
      AllReduceRsAgArgs a;
      std::memset(&a, 0, sizeof(a));
      a.rs.algo = a.ag.algo = algo;
      a.rs.in_dtype = a.rs.wire_dtype = a.rs.out_dtype = dt;
      a.rs.nsub = 1;
      a.rs.scale = (float)scale;
      a.rs.dst_stride = blk * s;                     // block d of the input starts at d * blk
      a.rs.out_sub_stride = blk * s;
      a.rs.stage_off = c.staging_off();
      a.rs.sub_elems = len;
      a.ag.nsub = 1;
      a.ag.sub_bytes = len * s;
      a.ag.in_sub_stride = blk * s;
      a.ag.out_src_stride = blk * s;
      for (int i = 0; i < l.n; ++i) {
        char* base = (char*)ts[i].data_ptr();
        const int me = l.first + i;
        a.rs.in[i] = base + e0 * s;
        a.rs.out[i] = base + ((uint64_t)me * blk + e0) * s;    // this rank's block of the sum, in its own slot
        if (off >= 0) {
          a.ag.in[i] = nullptr;                                  // already in place in the landing zone
          a.ag.out[i] = nullptr;
        } else {
          a.ag.in[i] = base + ((uint64_t)me * blk + e0) * s;
          a.ag.out[i] = base + e0 * s;
        }
      }
      if (off >= 0) {
        a.ag.recv_off = (uint64_t)off + e0 * s;      // peers write straight into the symmetric tensor
        a.ag.src_stride = blk * s;
      } else {
        a.ag.recv_off = c.staging_off();
        a.ag.src_stride = cap * s;
      }
      c.all_reduce_rsag(gid, a, nlanes, stream);
    }
    return;
  }
  AllReduceArgs a;
  std::memset(&a, 0, sizeof(a));
  a.algo = algo == kMultimem ? kMultimem : kDirect;
  a.dtype = dt;
  a.scale = (float)scale;
  if (off >= 0) {
    if (a.algo == kMultimem) TORCH_CHECK(off % 16 == 0 && (n * s) % 16 == 0, "multimem all-reduce needs 16-byte aligned data");
    a.buf_off = (uint64_t)off;
    a.elems = n;
    c.all_reduce(gid, a, nlanes, stream);
    return;
  }
  const uint64_t cap = c.staging_bytes() / s / 8 * 8;
  TORCH_CHECK(cap > 0, "no staging area configured for non-symmetric tensors");
  for (uint64_t e0 = 0; e0 < n; e0 += cap) {
    const uint64_t len = std::min(cap, n - e0);
    if (a.algo == kMultimem && (len * s) % 16 != 0) a.algo = kDirect;
    a.buf_off = c.staging_off();
    a.elems = len;
    for (int i = 0; i < l.n; ++i) a.data[i] = (char*)ts[i].data_ptr() + e0 * s;
    c.all_reduce(gid, a, nlanes, stream);
  }
}

// ------------------------------------------------------------------ broadcast
void broadcast(Comm& c, int gid, std::vector<at::Tensor> ts, int root, int nlanes, bool use_multimem) {
  const LocalList l = local_list(c, gid, ts.size(), "broadcast tensors");
  const int dev = c.device();
  c10::cuda::CUDAGuard guard(dev);
  for (int i = 0; i < l.n; ++i) {
    check_tensor(ts[i], "tensor", dev);
    TORCH_CHECK(ts[i].nbytes() == ts[0].nbytes(), "all ranks must pass tensors of the same size");
  }
  const uint64_t n = (uint64_t)ts[0].nbytes();
  if (n == 0) return;
  cudaStream_t stream = current_stream(dev);
  const int64_t off = symmetric_offset(c, gid, l, ts);
  BroadcastArgs a;
  std::memset(&a, 0, sizeof(a));
  a.root = root;
  a.use_multimem = use_multimem && c.has_multimem() ? 1 : 0;
  if (off >= 0) {
    if (a.use_multimem && (off % 16 != 0 || n % 16 != 0)) a.use_multimem = 0;
    a.buf_off = (uint64_t)off;
    a.bytes = n;
    c.broadcast(gid, a, nlanes, stream);
    return;
  }
  const uint64_t cap = c.staging_bytes() / 16 * 16;
  TORCH_CHECK(cap > 0, "no staging area configured for non-symmetric tensors");
  for (uint64_t e0 = 0; e0 < n; e0 += cap) {
    const uint64_t len = std::min(cap, n - e0);
    BroadcastArgs b = a;
    if (b.use_multimem && (len % 16 != 0 || ((uint64_t)ts[0].data_ptr() + e0) % 16 != 0)) b.use_multimem = 0;
    b.buf_off = c.staging_off();
    b.bytes = len;
    for (int i = 0; i < l.n; ++i) b.data[i] = (char*)ts[i].data_ptr() + e0;
    c.broadcast(gid, b, nlanes, stream);
  }
}

// ------------------------------------------------------------------ entry points under the reference's names
// pccl.all_gather_mpi / reduce_scatter_mpi(output, input, comm, algorithm) of the reference
// (pccl/src/pccl.cpp:11-14,87-90) and all_reduce_mpi(tensor, comm, algorithm) of its unbuilt
// pccl/src/yacl.cpp:146-149.  `comm` is a pccl.Group where the reference takes an mpi4py
// communicator; `algorithm` is "recursive" (halving / doubling) or "ring".  The argument
// checks are the reference's (contiguous, 1-D, sizes, dtypes); unlike it, the reductions also
// take bf16 and fp16, the all-gather has a real ring, and sizes are 64-bit.
struct GroupRef {
  std::shared_ptr<Comm> comm;
  int gid;
};

GroupRef group_from_python(const py::object& g) {
  TORCH_CHECK(py::hasattr(g, "comm") && py::hasattr(g, "gid"),
              "expected a pccl.Group as the communicator argument (it stands where the reference takes an mpi4py communicator)");
  py::object comm = g.attr("comm");
  TORCH_CHECK(!comm.is_none() && !comm.attr("native").is_none(), "the group has no native communicator (no CUDA device?)");
  GroupRef r{comm.attr("native").cast<std::shared_ptr<Comm>>(), g.attr("gid").cast<int>()};
  TORCH_CHECK(r.comm->nlocal() == 1, "the *_mpi entry points take one tensor per process");
  return r;
}

int algo_from_name(const std::string& algorithm, const char* fn) {
  if (algorithm == "recursive") return kRecursive;
  if (algorithm == "ring") return kRing;
  TORCH_CHECK(false, "Unknown algorithm specified for ", fn, ": ", algorithm);
  return -1;
}

int default_lanes(const Comm& c, uint64_t bytes) {
  const uint64_t want = std::max<uint64_t>(1, bytes / (128u << 10));
  return (int)std::min<uint64_t>(want, (uint64_t)std::min(64, c.max_lanes()));
}

void check_1d(const at::Tensor& out, const at::Tensor* in) {
  TORCH_CHECK(out.is_contiguous(), in ? "output tensor must be contiguous." : "input tensor must be contiguous.");
  if (in) TORCH_CHECK(in->is_contiguous(), "input tensor must be contiguous.");
  TORCH_CHECK(out.dim() == 1, in ? "output tensor must be 1D" : "input tensor must be 1D");
  if (in) TORCH_CHECK(in->dim() == 1, "input tensor must be 1D");
}

void all_gather_mpi(const at::Tensor& output_tensor, const at::Tensor& input_tensor, py::object py_comm,
                    const std::string& algorithm) {
  check_1d(output_tensor, &input_tensor);
  TORCH_CHECK(input_tensor.dtype() == output_tensor.dtype(), "Input and output tensors must have the same dtype.");
  GroupRef g = group_from_python(py_comm);
  const int size = g.comm->group_size(g.gid);
  TORCH_CHECK(output_tensor.numel() == input_tensor.numel() * size,
              "Output tensor must have total_elem elements (input tensor numel() *world_size)");
  const int algo = algo_from_name(algorithm, "all_gather_mpi");
  all_gather(*g.comm, g.gid, {output_tensor}, {input_tensor}, algo, default_lanes(*g.comm, (uint64_t)input_tensor.nbytes()));
}

void reduce_scatter_mpi(const at::Tensor& output_tensor, const at::Tensor& input_tensor, py::object py_comm,
                        const std::string& algorithm) {
  check_1d(output_tensor, &input_tensor);
  GroupRef g = group_from_python(py_comm);
  const int size = g.comm->group_size(g.gid);
  TORCH_CHECK(input_tensor.numel() % size == 0, "Input tensor size must be divisible by number of processes");
  TORCH_CHECK(output_tensor.numel() == input_tensor.numel() / size,
              "Output tensor must have block_size elements (input tensor numel()/world_size)");
  const int algo = algo_from_name(algorithm, "reduce_scatter_mpi");
  reduce_scatter(*g.comm, g.gid, {output_tensor}, {input_tensor}, algo,
                 default_lanes(*g.comm, (uint64_t)output_tensor.nbytes()), 1.0, std::nullopt);
}

void all_reduce_mpi(const at::Tensor& input_tensor, py::object py_comm, const std::string& algorithm) {
  check_1d(input_tensor, nullptr);
  GroupRef g = group_from_python(py_comm);
  const int size = g.comm->group_size(g.gid);
  TORCH_CHECK(input_tensor.numel() % size == 0, "Input tensor size must be divisible by number of processes");
  const int algo = algo_from_name(algorithm, "all_reduce_mpi");
  all_reduce(*g.comm, g.gid, {input_tensor}, algo, default_lanes(*g.comm, (uint64_t)input_tensor.nbytes() / (uint64_t)size), 1.0);
}

at::Tensor heap_tensor(Comm& c, int64_t off, int64_t numel, at::ScalarType dtype, int world_rank) {
  TORCH_CHECK(off >= 0 && (uint64_t)off + (uint64_t)numel * c10::elementSize(dtype) <= c.heap_bytes(),
              "range outside the symmetric heap");
  void* p = (void*)(c.heap_base(world_rank) + (uint64_t)off);
  auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, c.device());
  return at::from_blob(p, {numel}, opts);
}

// Tensors that own a heap block: the block returns to the allocator when the last of them
// (views included, since they share the storage) is destroyed.
struct HeapBlock {
  std::shared_ptr<Comm> comm;
  int64_t off;
  HeapBlock(std::shared_ptr<Comm> c, int64_t o) : comm(std::move(c)), off(o) {}
  HeapBlock(const HeapBlock&) = delete;
  HeapBlock& operator=(const HeapBlock&) = delete;
  ~HeapBlock() {
    try {
      comm->free(off);
    } catch (...) {
    }
  }
};

std::vector<at::Tensor> owned_tensors(std::shared_ptr<Comm> c, int64_t off, int64_t numel, at::ScalarType dtype,
                                      std::vector<int> owners) {
  TORCH_CHECK(off >= 0 && (uint64_t)off + (uint64_t)numel * c10::elementSize(dtype) <= c->heap_bytes(),
              "range outside the symmetric heap");
  auto blk = std::make_shared<HeapBlock>(c, off);
  auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, c->device());
  std::vector<at::Tensor> out;
  for (int r : owners) {
    void* p = (void*)(c->heap_base(r) + (uint64_t)off);
    out.push_back(at::from_blob(p, {numel}, [blk](void*) {}, opts));
  }
  return out;
}

py::dict status_dict(Comm& c, int li) {
  const Status s = c.status(li);
  py::dict d;
  d["code"] = s.code;
  d["epoch"] = s.epoch;
  d["rank"] = s.rank;
  d["peer"] = s.peer;
  d["lane"] = s.lane;
  d["slot_kind"] = s.slot_kind;
  d["seen"] = s.seen;
  d["collective"] = s.collective;
  return d;
}

}  // namespace

void bind_gemm(py::module_& m);   // gemm_bindings.cpp
void bind_optim(py::module_& m);  // optim_bindings.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "pccl native layer: sm_100a collective kernels, symmetric heap, tcgen05 GEMMs";
  py::register_exception<pccl::Error>(m, "Error", PyExc_RuntimeError);

  m.attr("MAX_RANKS") = kMaxRanks;
  m.attr("MAX_LANES") = kMaxLanes;
  m.attr("REGION_BYTES") = kRegionBytes;
  m.attr("DIRECT") = (int)kDirect;
  m.attr("RING") = (int)kRing;
  m.attr("RECURSIVE") = (int)kRecursive;
  m.attr("PULL") = (int)kPull;
  m.attr("MULTIMEM") = (int)kMultimem;
  m.attr("EAGER") = (int)kEager;
  m.attr("STATUS_OK") = (int)kStatusOk;
  m.attr("STATUS_TIMEOUT") = (int)kStatusTimeout;
  m.attr("STATUS_POISONED") = (int)kStatusPoisoned;

  // Read / write one 32-bit word at a device address of this process (own or peer-mapped):
  // used by the bootstrap self-check to prove that a mapping reaches the peer's memory.
  m.def("peek_u32", [](uint64_t addr) {
    uint32_t v = 0;
    PCCL_CUDA(cudaMemcpy(&v, (const void*)addr, 4, cudaMemcpyDeviceToHost));
    return v;
  });
  m.def("poke_u32", [](uint64_t addr, uint32_t v) {
    PCCL_CUDA(cudaMemcpy((void*)addr, &v, 4, cudaMemcpyHostToDevice));
    PCCL_CUDA(cudaDeviceSynchronize());
  });
  m.def("all_gather_mpi", &all_gather_mpi, py::arg("output_tensor"), py::arg("input_tensor"), py::arg("comm"),
        py::arg("algorithm") = "recursive", "all-gather on a pccl.Group; algorithm: 'recursive' (doubling) or 'ring'");
  m.def("reduce_scatter_mpi", &reduce_scatter_mpi, py::arg("output_tensor"), py::arg("input_tensor"), py::arg("comm"),
        py::arg("algorithm") = "recursive", "reduce-scatter (SUM) on a pccl.Group; algorithm: 'recursive' (halving) or 'ring'");
  m.def("all_reduce_mpi", &all_reduce_mpi, py::arg("input_tensor"), py::arg("comm"), py::arg("algorithm") = "recursive",
        "in-place all-reduce (SUM) on a pccl.Group as reduce-scatter + all-gather of one schedule family, one launch");
  m.def("num_steps", [](int algo, int P) { return num_steps(algo, P); });
  m.def("ag_step", [](int algo, int P, int r, int t) { return step_tuple(ag_step(algo, P, r, t)); });
  m.def("rs_step", [](int algo, int P, int r, int t) { return step_tuple(rs_step(algo, P, r, t)); });
  m.def("rs_stage_offset", [](int algo, int P, int t) { return rs_stage_offset(algo, P, t); });
  m.def("rs_dep_mask", [](int algo, int P, int t) { return rs_dep_mask(algo, P, t); });
  m.def("slot_index", [](int lane, int kind, int src) { return slot_index(lane, kind, src); });

  py::class_<IpcSegment>(m, "IpcSegment")
      .def(py::init<int, uint64_t>(), py::arg("device"), py::arg("bytes"))
      .def(py::init([](int device, py::bytes handle, uint64_t bytes) {
             return new IpcSegment(device, std::string(handle), bytes);
           }),
           py::arg("device"), py::arg("handle"), py::arg("bytes"))
      .def_property_readonly("ptr", &IpcSegment::ptr)
      .def_property_readonly("bytes", &IpcSegment::bytes)
      .def("handle", [](IpcSegment& s) { return py::bytes(s.handle()); })
      .def("close", &IpcSegment::close);

  py::class_<VmmSegment>(m, "VmmSegment")
      .def(py::init<int, uint64_t, int>(), py::arg("device"), py::arg("bytes"), py::arg("world_for_multicast") = 0)
      // a named factory, not an overload: (device, fd, bytes) and (device, bytes, world) are
      // both three integers and overload resolution would silently pick the allocating one
      .def_static("from_fd", [](int device, int fd, uint64_t bytes) { return new VmmSegment(device, fd, bytes); },
                  py::arg("device"), py::arg("fd"), py::arg("bytes"), py::return_value_policy::take_ownership)
      .def_property_readonly("ptr", &VmmSegment::ptr)
      .def_property_readonly("bytes", &VmmSegment::bytes)
      .def("export_fd", &VmmSegment::export_fd)
      .def_static("multicast_supported", &VmmSegment::multicast_supported)
      .def("multicast_create", &VmmSegment::multicast_create)
      .def("multicast_import", &VmmSegment::multicast_import)
      .def("multicast_add_device", &VmmSegment::multicast_add_device)
      .def("multicast_bind_and_map", &VmmSegment::multicast_bind_and_map)
      .def("multicast_release", &VmmSegment::multicast_release)
      .def("close", &VmmSegment::close);

  py::class_<OffsetAllocator>(m, "OffsetAllocator",
                              "first-fit allocator over byte offsets: the bookkeeping of the symmetric heap (no device memory involved)")
      .def(py::init<uint64_t>(), py::arg("size"))
      .def("alloc", &OffsetAllocator::alloc, py::arg("bytes"), py::arg("align") = 256, "offset, or -1 when it does not fit")
      .def("free", &OffsetAllocator::free, py::arg("offset"))
      .def_property_readonly("used", &OffsetAllocator::used)
      .def_property_readonly("size", &OffsetAllocator::size)
      .def("largest_free", &OffsetAllocator::largest_free);

  py::class_<Comm, std::shared_ptr<Comm>>(m, "Comm")
      .def(py::init<int, int, int, int, std::vector<uint64_t>, std::vector<uint64_t>, uint64_t, uint64_t, uint64_t, uint64_t>(),
           py::arg("world"), py::arg("rank"), py::arg("nlocal"), py::arg("device"), py::arg("heaps"), py::arg("sigs"),
           py::arg("mc_heap"), py::arg("heap_bytes"), py::arg("sig_bytes"), py::arg("staging_bytes"))
      .def_property_readonly("world", &Comm::world)
      .def_property_readonly("rank", &Comm::rank)
      .def_property_readonly("nlocal", &Comm::nlocal)
      .def_property_readonly("device", &Comm::device)
      .def_property_readonly("has_multimem", &Comm::has_multimem)
      .def_property_readonly("heap_bytes", &Comm::heap_bytes)
      .def_property_readonly("heap_used", &Comm::heap_used)
      .def_property_readonly("staging_off", &Comm::staging_off)
      .def_property_readonly("staging_bytes", &Comm::staging_bytes)
      .def_property_readonly("max_lanes", &Comm::max_lanes)
      .def_property_readonly("eager_capacity", &Comm::eager_capacity,
                             "bytes of one half of the eager area (0: none): an eager all-gather needs P * bytes per rank, "
                             "an eager reduce-scatter (P-1) * bytes per block")
      .def_property_readonly("kernels_launched", &Comm::kernels_launched)
      .def("heap_base", &Comm::heap_base)
      .def("alloc", &Comm::alloc, py::arg("bytes"), py::arg("align") = 256)
      .def("free", &Comm::free)
      .def("offset_of", &Comm::offset_of)
      .def("tensor", &heap_tensor, py::arg("off"), py::arg("numel"), py::arg("dtype"), py::arg("world_rank"))
      .def("owned_tensors", &owned_tensors)
      .def("new_group", &Comm::new_group)
      .def("group_size", &Comm::group_size)
      .def("group_rank", &Comm::group_rank)
      .def("set_timeout_ms", &Comm::set_timeout_ms)
      .def("set_debug", &Comm::set_debug, py::arg("jitter_ns") = 0, py::arg("trace_events") = 0,
           "stress-mode jitter before every wait/signal and capacity of the device-side trace (0 = off)")
      .def("read_trace",
           [](Comm& c) {
             uint64_t dropped = 0;
             std::vector<TraceEvent> ev = c.read_trace(&dropped);
             py::list rows;
             for (const TraceEvent& e : ev)
               rows.append(py::make_tuple(e.t_ns, e.epoch, (int)e.rank, (int)e.lane, (int)(e.what & 63), (e.what & 64) != 0,
                                          e.collective));
             return py::make_tuple(rows, dropped);
           },
           "([(t_ns, epoch, rank, lane, slot_kind, is_signal, collective)], dropped); empties the trace")
      .def("timeout_ms", &Comm::timeout_ms)
      .def("status", &status_dict, py::arg("local_slot") = 0)
      .def("poisoned", &Comm::poisoned)
      .def("reset_after_failure", &Comm::reset_after_failure)
      .def("all_gather", &all_gather, py::arg("gid"), py::arg("outs"), py::arg("ins"), py::arg("algo"), py::arg("nlanes"))
      .def("all_gather_raw", &all_gather_raw)
      .def("all_gather_copy_engine", &all_gather_copy_engine, py::arg("gid"), py::arg("out"), py::arg("input"),
           "peer-to-local copies on the current stream, no kernel; the caller keeps the peers' inputs stable")
      .def("reduce_scatter", &reduce_scatter, py::arg("gid"), py::arg("outs"), py::arg("ins"), py::arg("algo"),
           py::arg("nlanes"), py::arg("scale") = 1.0, py::arg("wire_dtype") = py::none())
      .def("reduce_scatter_raw", &reduce_scatter_raw)
      .def("all_reduce", &all_reduce, py::arg("gid"), py::arg("tensors"), py::arg("algo"), py::arg("nlanes"),
           py::arg("scale") = 1.0)
      .def("broadcast", &broadcast, py::arg("gid"), py::arg("tensors"), py::arg("root"), py::arg("nlanes"),
           py::arg("use_multimem") = false)
      .def("barrier", [](Comm& c, int gid) {
        c10::cuda::CUDAGuard guard(c.device());
        c.barrier(gid, current_stream(c.device()));
      });

  bind_gemm(m);
  bind_optim(m);
}
