"""The allocation-free reduce-scatter, called the way its users call it: through the C
symbol exported by the shared object, with raw device pointers.

Those users are programs that may not allocate device memory at the moment they call the
library: a self check running inside a job whose framework already owns all of the HBM
(cudaMalloc would fail), code on a path where the implicit synchronisation of
cudaMalloc/cudaFree is not tolerable, or a plain C caller without any tensor allocator.
The entry point keeps its staging areas, flags and status words in a static device array
instead.  This test checks it against the regular entry point (a communicator with its
own heap), twice in a row, because the second call finds the array as the first left it.

This file sorts last on purpose: it must pass on its own in a fresh process and also
after every other test has run in the same process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _entry():
    import pccl
    from pccl import build_kernels

    pccl.build()                                   # makes sure the shared object exists and torch's libraries are loaded
    lib = ctypes.CDLL(str(build_kernels._SO))
    fn = lib.pccl_reduce_scatter_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_uint64,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p,
                   ctypes.c_size_t]
    return fn


def _call(fn, ins, outs, world, n, tin, tout, algo, scale):
    arr = ctypes.c_void_p * world
    err = ctypes.create_string_buffer(256)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = fn(arr(*[t.data_ptr() for t in ins]), arr(*[t.data_ptr() for t in outs]), world, n, tin, tout, algo, scale,
            stream, err, 256)
    return rc, err.value.decode()


_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _status(world):
    """Status codes of the last call, one per emulated rank, read through the exported query."""
    from pccl import build_kernels

    lib = ctypes.CDLL(str(build_kernels._SO))
    q = lib.pccl_reduce_scatter_noalloc_status
    q.restype = ctypes.c_int
    q.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_uint32), ctypes.c_char_p, ctypes.c_size_t]
    codes = (ctypes.c_uint32 * world)()
    err = ctypes.create_string_buffer(256)
    rc = q(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), world, codes, err, 256)
    assert rc in (0, 1), err.value.decode()
    return list(codes)


@pytest.mark.parametrize("world,algo", [(8, 0), (8, 1), (8, 2), (4, 2), (3, 1), (2, 0), (1, 0)])
@pytest.mark.parametrize("dtypes", [(torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16),
                                    (torch.float32, torch.float32), (torch.float16, torch.float16)])
def test_matches_regular_entry_point_twice(world, algo, dtypes):
    import pccl

    fn = _entry()
    tin, tout = dtypes
    comm = pccl.Communicator.emulated_world(world, device=0, heap_bytes=16 << 20, staging_bytes=4 << 20)
    g = torch.Generator(device=DEV).manual_seed(17 * world + algo)
    for call, n in enumerate((32768, 1001)):        # two calls in a row on the same static array
        ins = [torch.randn(world * n, device=DEV, generator=g).to(tin) for _ in range(world)]
        want = [torch.zeros(n, device=DEV, dtype=tout) for _ in range(world)]
        comm.native.reduce_scatter(comm.world_group.gid, want, ins, algo, 4, 0.5, None)
        comm.check()
        got = [torch.full((n,), float("nan"), device=DEV, dtype=tout) for _ in range(world)]
        rc, msg = _call(fn, ins, got, world, n, _CODE[tin], _CODE[tout], algo, 0.5)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert _status(world) == [0] * world       # the return code only says "enqueued"; this says "completed"
        ref = (sum(t.float() for t in ins).view(world, n) * 0.5)
        for r in range(world):
            tol = dict(rtol=1e-5, atol=1e-5) if tout == torch.float32 and (tin == torch.float32 or algo == 0) \
                else dict(rtol=3e-2, atol=3e-2)
            torch.testing.assert_close(got[r].float(), want[r].float(), **tol)       # the existing entry point
            torch.testing.assert_close(got[r].float(), ref[r], rtol=3e-2, atol=3e-2)  # and plain fp32 PyTorch


def test_rejects_what_does_not_fit():
    fn = _entry()
    x = [torch.zeros(8, device=DEV)]
    rc, msg = _call(fn, x * 2, x * 2, 2, 32769, 2, 2, 0, 1.0)
    assert rc != 0 and "exceeds the built-in scratch" in msg
    rc, msg = _call(fn, x * 9, x * 9, 9, 8, 2, 2, 0, 1.0)
    assert rc != 0 and "world size" in msg
    rc, msg = _call(fn, x * 3, x * 3, 3, 8, 2, 2, 2, 1.0)
    assert rc != 0 and "power-of-two" in msg
    rc, msg = _call(fn, x * 2, x * 2, 2, 8, 2, 0, 0, 1.0)
    assert rc != 0 and "dtype" in msg
    # nothing was launched and the device is fine
    assert float(torch.ones(4, device=DEV).sum()) == 4.0
