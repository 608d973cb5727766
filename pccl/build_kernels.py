"""Build and load the native extension ``pccl._C`` for sm_100a.

Counterpart of ``pccl/build_kernels.py:22-116`` in the reference (a JIT
``torch.utils.cpp_extension.load`` of four sources with an sm_70..sm_90 gencode list and
the mpi4py include path).  Differences:

* one target, ``-gencode arch=compute_100a,code=sm_100a``; no MPI, no HIP branch;
* the shared object is kept inside the package (``pccl/_build/pccl_C.so``) together with
  a digest of the sources, and is imported directly when the digest matches, so a
  machine that received a built tree never runs the compiler;
* the module is called ``pccl_C`` and is reachable as ``pccl._C``: it does not shadow the
  Python package the way the reference's extension named ``pccl`` does.

``build()`` is idempotent.  Callers that start one process per GPU should let rank 0 build
first (``build_rank0_first``), as the reference's callers do with an MPI barrier
(``benchmark_raw_collectives/all_gather.py:45-51``).
"""
from __future__ import annotations

import hashlib
import importlib.machinery
import importlib.util
import os
import sys
from pathlib import Path
from typing import List

_HERE = Path(__file__).resolve().parent
CSRC = _HERE / "csrc"
BUILD_DIR = _HERE / "_build"
MODULE_NAME = "pccl_C"
_SO = BUILD_DIR / f"{MODULE_NAME}.so"
_DIGEST = BUILD_DIR / f"{MODULE_NAME}.digest"

SOURCES = [
    "bindings.cpp",
    "gemm_bindings.cpp",
    "optim_bindings.cpp",
    "comm.cpp",
    "segments.cpp",
    "collectives.cu",
    "gemm_sm100.cu",
    "optim.cu",
    "train_ops.cu",
    "noalloc.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--expt-extended-lambda",
    "-Xptxas", "-v",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-Wall", "-Wno-unused-function"]

BUILT = False
_module = None


def _existing_sources() -> List[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def source_digest() -> str:
    h = hashlib.sha256()
    files = sorted(p for p in CSRC.iterdir() if p.suffix in (".cpp", ".cu", ".cuh", ".h"))
    for p in files:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


def is_built() -> bool:
    return _SO.exists() and _DIGEST.exists() and _DIGEST.read_text().strip() == source_digest()


def _import_so():
    global _module
    if _module is not None:
        return _module
    import torch  # noqa: F401  (the extension links against libtorch)

    loader = importlib.machinery.ExtensionFileLoader(MODULE_NAME, str(_SO))
    spec = importlib.util.spec_from_file_location(MODULE_NAME, str(_SO), loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules[MODULE_NAME] = mod
    _module = mod
    return mod


def build(verbose: bool = False, force: bool = False):
    """Compile the extension if the shared object is missing or stale, then import it."""
    global BUILT, _module
    if BUILT and not force and _module is not None:
        return _module
    if force or not is_built():
        from torch.utils import cpp_extension

        BUILD_DIR.mkdir(exist_ok=True)
        # A toolchain that only ships a static libstdc++ gives the extension its own,
        # never-initialised copy of the iostream locale (integer formatting then crashes).
        # The distribution compiler links the shared libstdc++ that torch itself uses.
        for var, path in (("CXX", "/usr/bin/g++"), ("CC", "/usr/bin/gcc")):
            if os.path.exists(path) and os.environ.get("PCCL_KEEP_COMPILER") != "1":
                os.environ[var] = path
        cuda_home = cpp_extension.CUDA_HOME
        if cuda_home is None or not (Path(cuda_home) / "bin" / "nvcc").exists():
            raise RuntimeError("pccl: nvcc not found; the native extension cannot be built on this machine")
        mod = cpp_extension.load(
            name=MODULE_NAME,
            sources=[str(p) for p in _existing_sources()],
            extra_cflags=CXX_FLAGS,
            extra_cuda_cflags=NVCC_FLAGS,
            extra_include_paths=[str(CSRC)],
            build_directory=str(BUILD_DIR),
            with_cuda=True,
            verbose=verbose,
        )
        _DIGEST.write_text(source_digest())
        if _module is None:
            _module = mod
            sys.modules[MODULE_NAME] = mod
    mod = _import_so()
    BUILT = True
    return mod


def load(allow_build: bool = True):
    """Import ``pccl._C``; build it first when that is needed and possible."""
    if _module is not None:
        return _module
    if is_built():
        return _import_so()
    if not allow_build or os.environ.get("PCCL_NO_BUILD") == "1":
        raise ImportError(
            "pccl native extension is missing or stale; run `python -m pccl.build_kernels` on a machine with nvcc"
        )
    return build()


def build_rank0_first(barrier) -> None:
    """Rank 0 compiles, the others wait at ``barrier()`` and then load the result."""
    rank = int(os.environ.get("RANK", os.environ.get("SLURM_PROCID", "0")))
    if rank == 0:
        build()
        barrier()
    else:
        barrier()
        build()


if __name__ == "__main__":
    m = build(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(f"built {m.__name__} -> {_SO}")
