"""The allocation-free all-reduce entry point (stdmlc_all_reduce_noalloc).

Some users of the library may not allocate device memory, directly or through a
library call: code that lives inside a host application which owns all device
memory through its own allocator, and steady-state loops that cannot afford the
device-wide synchronisation hidden in cudaMalloc / cudaFree.  For them the
library exports one C symbol whose scratch memory is a fixed array inside the
library image.  This test calls that symbol directly (ctypes, as a C program
would) and checks it, bit for bit, against the regular loopback device session
on the same inputs, twice in a row (the second call reuses the scratch that the
first one left behind).  The file name sorts last on purpose: it runs after
every other test, and it also passes when run alone in a fresh process."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from stdml_collective_experimental_b200 import DeviceSession, _native  # noqa: E402
from stdml_collective_experimental_b200.ops.device import dtype_code, op_code  # noqa: E402
from stdml_collective_experimental_b200.utils.oracle import reduce_many  # noqa: E402

MAX_BYTES = 512 << 10
MAX_RANKS = 8


def entry_point():
    lib = _native.lib()
    fn = lib.stdmlc_all_reduce_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                   ctypes.c_ulonglong, ctypes.c_int, ctypes.c_int, ctypes.c_double,
                   ctypes.c_void_p]
    return lib, fn


def status(lib):
    """(return code, the seven status words) of the calls enqueued so far."""
    fn = lib.stdmlc_all_reduce_noalloc_status
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_void_p]
    out = (ctypes.c_int * 7)()
    rc = fn(out, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, tuple(out)


def ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def call(fn, ins, outs, op, scale):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(ptrs(ins), ptrs(outs), len(ins), ins[0].numel(), dtype_code(ins[0].dtype),
              op_code(op), scale, ctypes.c_void_p(stream))


@pytest.mark.parametrize("world,dtype,op,n,scale", [
    (4, torch.float32, "sum", 100_003, 0.25),
    (8, torch.bfloat16, "sum", 262_144, 1.0),     # exactly the size limit
    (2, torch.int32, "max", 17, 1.0),
    (3, torch.float16, "prod", 4099, 1.0),
    (6, torch.float64, "sum", 10_007, 1.0 / 3.0),  # a scale that is not a float
])
def test_noalloc_matches_device_session_twice(world, dtype, op, n, scale):
    lib, fn = entry_point()
    g = torch.Generator().manual_seed(n)
    with DeviceSession.loopback(world, heap_bytes=1 << 20, staging_bytes=2 << 20) as sess:
        for round_ in range(2):  # two calls in a row share the scratch array
            if dtype.is_floating_point:
                host = [(torch.rand(n, generator=g) + 0.5).to(dtype) for _ in range(world)]
            else:
                host = [torch.randint(-1000, 1000, (n,), generator=g).to(dtype)
                        for _ in range(world)]
            ins = [h.cuda() for h in host]
            want = [torch.empty_like(t) for t in ins]
            sess.all_reduce(ins, out=want, op=op, scale=None if scale == 1.0 else scale,
                            algo="oneshot")
            got = [torch.full_like(t, 7) for t in ins]
            rc = call(fn, ins, got, op, scale)
            assert rc == 0, lib.stdmlc_last_error().decode()
            torch.cuda.synchronize()
            sess.check()
            assert status(lib) == (0, (0, 0, 0, 0, 0, 0, 0)), "no bounded wait ran out"
            # two oracles that share no code with the kernel: the host reducer
            # (bit for bit) and a plain float64 PyTorch reduction (within rounding)
            cpu_want = reduce_many(host, op, scale)
            wide = torch.stack([h.double() for h in host])
            wide = {"sum": wide.sum(0), "max": wide.max(0).values,
                    "prod": wide.prod(0)}[op] * scale
            tol = {torch.float32: 1e-6, torch.float64: 1e-14, torch.bfloat16: 1e-2,
                   torch.float16: 2e-3, torch.int32: 0}[dtype]
            for r in range(world):
                assert torch.equal(got[r].view(torch.uint8), want[r].view(torch.uint8)), \
                    (round_, r)
                assert torch.equal(got[r].cpu().view(torch.uint8), cpu_want.view(torch.uint8))
                assert torch.allclose(got[r].cpu().double(), wide, rtol=tol, atol=tol)
                assert torch.equal(ins[r].cpu(), host[r]), "inputs must stay untouched"
        # in place: out[r] == in[r]
        ins = [h.cuda() for h in host]
        assert call(fn, ins, ins, op, scale) == 0
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(ins[r].view(torch.uint8), want[r].view(torch.uint8))


def test_noalloc_rejects_what_does_not_fit():
    lib, fn = entry_point()
    x = [torch.zeros(MAX_BYTES // 4 + 1, device="cuda") for _ in range(2)]
    assert call(fn, x, x, "sum", 1.0) == 2
    assert b"exceed the fixed scratch" in lib.stdmlc_last_error()
    y = [torch.zeros(8, device="cuda") for _ in range(MAX_RANKS + 1)]
    assert call(fn, y, y, "sum", 1.0) == 2
    assert b"nranks" in lib.stdmlc_last_error()
    z = [torch.zeros(8, device="cuda")]
    assert call(fn, z, z, "bit_xor", 1.0) == 2      # xor is not defined for floats
    assert call(fn, z, z, "sum", 1.0) == 0          # one rank: a scaled copy
    torch.cuda.synchronize()
