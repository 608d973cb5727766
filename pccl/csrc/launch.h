// Host-callable launchers of the collective kernels (defined in collectives.cu).
// They take fully-resolved argument blocks and enqueue exactly one kernel on `stream`.
#pragma once
#include <cuda_runtime.h>

#include "device_types.h"

namespace pccl {

cudaError_t launch_all_gather(const AllGatherArgs& a, int nlanes, cudaStream_t stream);
cudaError_t launch_reduce_scatter(const ReduceScatterArgs& a, int nlanes, cudaStream_t stream);
cudaError_t launch_all_reduce(const AllReduceArgs& a, int nlanes, cudaStream_t stream);
cudaError_t launch_all_reduce_rsag(const AllReduceRsAgArgs& a, int nlanes, cudaStream_t stream);
cudaError_t launch_broadcast(const BroadcastArgs& a, int nlanes, cudaStream_t stream);
cudaError_t launch_barrier(const BarrierArgs& a, cudaStream_t stream);

// Largest lane count (grid.x) that is guaranteed to be co-resident on `device`.
int max_resident_lanes(int device);

}  // namespace pccl
