#!/usr/bin/env bash
# Launches one raw-collective benchmark on the GPUs of ONE NVSwitch node, one process per GPU.
#
#   benchmark_raw_collectives/run_raw_collectives_benchmark.sh all_gather 8 --library pccl --algorithm all --test
#   benchmark_raw_collectives/run_raw_collectives_benchmark.sh reduce_scatter 4 --library xccl
#   benchmark_raw_collectives/run_raw_collectives_benchmark.sh gemm 8 --fused
#
# Counterpart of the reference's cluster launchers (scripts/perlmutter/run_raw_collectives_benchmark.sh,
# scripts/frontier/run_raw_collectives_benchmark.sh, scripts/get_rank.sh): those export the rendezvous
# variables, NIC / libfabric settings and a per-rank GPU binding for srun.  On one node none of the
# network settings apply; what is left is the rendezvous (loopback), one connection queue per
# device so that copy and compute kernels of different streams are not serialised behind each
# other, and the launcher.  Under SLURM (`srun --ntasks-per-node=N`) the script starts the
# benchmark directly and the ranks come from SLURM_PROCID / SLURM_NTASKS / SLURM_LOCALID.
set -euo pipefail

here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
what="${1:?benchmark name: all_gather | reduce_scatter | gemm}"
ngpu="${2:?number of GPUs}"
shift 2

case "$what" in
  all_gather|reduce_scatter) extra=(--num-gpus-per-node "$ngpu" --machine b200) ;;
  gemm) extra=() ;;
  *) echo "unknown benchmark '$what'" >&2; exit 2 ;;
esac

export MASTER_ADDR="${MASTER_ADDR:-127.0.0.1}"
export MASTER_PORT="${MASTER_PORT:-29500}"
export CUDA_DEVICE_MAX_CONNECTIONS="${CUDA_DEVICE_MAX_CONNECTIONS:-8}"
export NCCL_DEBUG="${NCCL_DEBUG:-WARN}"
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-4}"

if [[ -n "${SLURM_PROCID:-}" ]]; then
  export WORLD_SIZE="${SLURM_NTASKS}"
  exec python "$here/$what.py" "${extra[@]}" "$@"
fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$ngpu" \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" "$here/$what.py" "${extra[@]}" "$@"
