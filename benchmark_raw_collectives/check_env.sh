#!/usr/bin/env bash
# Checks the software this library needs and builds the native extension in-tree.
#
# Counterpart of the reference's environment builders (scripts/perlmutter/create_python_env.sh,
# scripts/frontier/create_python_env.sh): those create a venv, pip-install torch / deepspeed and
# compile mpi4py against the site's MPI.  Nothing here needs MPI or a package index: the
# requirements are a CUDA 12.8+ toolkit with sm_100a support, PyTorch with the NCCL backend, and
# a host compiler; DeepSpeed is optional (pccl.patch_deepspeed patches it when it is importable).
set -euo pipefail
root="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
cd "$root"

fail=0
need() { if ! command -v "$1" >/dev/null 2>&1; then echo "missing: $1" >&2; fail=1; fi; }
need python
need nvcc
need g++
[[ $fail -eq 0 ]] || exit 1

nvcc --version | tail -n 2
if ! nvcc --list-gpu-arch 2>/dev/null | grep -q "compute_100"; then
  echo "this nvcc cannot compile for sm_100a (need CUDA 12.8 or newer)" >&2
  exit 1
fi
python - <<'PY'
import importlib.util, torch, torch.distributed as dist
print("torch", torch.__version__, "cuda", torch.version.cuda, "nccl backend:", dist.is_nccl_available())
if torch.cuda.is_available():
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        print(f"gpu {i}: {p.name} sm_{p.major}{p.minor} {p.total_memory >> 30} GiB {p.multi_processor_count} SMs")
        if (p.major, p.minor) != (10, 0):
            print("  warning: the kernels are built for sm_100a only")
else:
    print("no GPU visible: the extension still builds, the CPU tests still run")
print("deepspeed:", "found" if importlib.util.find_spec("deepspeed") else "not installed (optional)")
PY
python -m pccl.build_kernels
python -m pytest tests -q -m "not gpu" -x
