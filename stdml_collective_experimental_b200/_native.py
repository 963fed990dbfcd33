"""Loader of the native runtime (``libstdml_collective_b200.so``).

The library is built in-tree by ``make -C csrc`` (``build()`` below runs it) and
is loaded with ctypes.  Nothing in this package works without it: a missing
library is an ImportError with the build command, never a silent Python
fallback.
"""
import ctypes
import os
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libstdml_collective_b200.so")

_lock = threading.Lock()
_lib = None


def build(jobs=None, verbose=False, target="all"):
    """Compile the native runtime and its programs for sm_100a (needs nvcc, no GPU)."""
    jobs = jobs or max(2, (os.cpu_count() or 4))
    cmd = ["make", "-C", CSRC, f"-j{jobs}", target]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("native build failed: " + " ".join(cmd))
    return LIB_PATH


def lib():
    """The loaded library (loads it on first use)."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                # a fresh checkout has sources only: compile once (needs nvcc, ~2 minutes)
                try:
                    build(target="lib")
                except Exception as e:
                    raise ImportError(
                        f"{LIB_PATH} is missing and could not be built ({e}); build it with "
                        f"`make -C {CSRC}`") from e
            _lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
            _declare(_lib)
        return _lib


class NativeError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(message)
        self.code = code


class DeviceTimeoutError(NativeError):
    """A device-side bounded wait ran out (a peer never arrived)."""


class PeerFailure(NativeError):
    """Host path: a peer this rank was sending to or waiting for has gone."""


def check(rc):
    if rc != 0:
        msg = lib().stdmlc_last_error().decode("utf-8", "replace")
        if rc == 4:
            raise DeviceTimeoutError(rc, msg)
        if rc == 5:
            raise PeerFailure(rc, msg)
        if rc == 2:
            raise ValueError(msg)
        if rc == 3:
            raise MemoryError(msg)
        raise NativeError(rc, msg)


def _declare(l):
    c = ctypes
    vp, vpp = c.c_void_p, c.POINTER(c.c_void_p)
    u64 = c.c_ulonglong
    l.stdmlc_last_error.restype = c.c_char_p
    l.stdmlc_cuda_device_count.restype = c.c_int
    l.stdmlc_pointer_kind.argtypes = [vp]
    l.stdmlc_dw_create.argtypes = [vpp, c.c_int, c.c_int, c.c_int, c.c_int, u64, u64, c.c_char_p,
                                   c.c_char_p, c.c_int, c.c_int, u64]
    l.stdmlc_dw_destroy.argtypes = [vp]
    l.stdmlc_dw_info.argtypes = [vp, c.c_int, c.POINTER(u64)]
    l.stdmlc_dw_alloc.argtypes = [vp, u64, c.POINTER(u64)]
    l.stdmlc_dw_release.argtypes = [vp, u64]
    l.stdmlc_dw_ptr.argtypes = [vp, c.c_int, u64, vpp]
    l.stdmlc_dw_mc_ptr.argtypes = [vp, u64, vpp]
    l.stdmlc_dw_set_tuning.argtypes = [vp, c.c_int, c.c_longlong, c.c_longlong, c.c_longlong]
    l.stdmlc_dw_set_knob.argtypes = [vp, c.c_char_p, c.c_longlong]
    l.stdmlc_dw_drop_registrations.argtypes = [vp]
    l.stdmlc_dw_all_reduce.argtypes = [vp, vpp, vpp, u64, c.c_int, c.c_int, c.c_double, c.c_int, vp]
    l.stdmlc_dw_reduce.argtypes = [vp, vpp, vpp, u64, c.c_int, c.c_int, c.c_int, c.c_double, vp]
    l.stdmlc_dw_group_all_reduce.argtypes = [vp, u64, vpp, vpp, c.POINTER(u64), c.c_int, c.c_int,
                                             c.c_int, c.c_double, c.c_int, vp]
    l.stdmlc_dw_all_gather.argtypes = [vp, vpp, vpp, u64, c.c_int, vp]
    l.stdmlc_dw_broadcast.argtypes = [vp, vpp, vpp, u64, c.c_int, c.c_int, vp]
    l.stdmlc_dw_barrier.argtypes = [vp, vp]
    l.stdmlc_dw_raw_all_reduce.argtypes = [vp, u64, vpp, vpp, u64, c.c_int, c.c_int, c.c_int,
                                           c.c_int, c.c_int, c.c_int, c.c_int, c.c_double, vp]
    l.stdmlc_dw_status.argtypes = [vp, c.POINTER(c.c_int)]
    l.stdmlc_dw_check.argtypes = [vp]
    l.stdmlc_dw_recover.argtypes = [vp]
    l.stdmlc_dw_barrier_rows.argtypes = [vp, c.c_int, vp]
    l.stdmlc_version.restype = c.c_char_p
    l.stdmlc_dtype_size.argtypes = [c.c_int]
    l.stdmlc_reduce_many.argtypes = [vp, vpp, u64, u64, c.c_int, c.c_int, c.c_double]
    l.stdmlc_reduce.argtypes = [vp, vp, vp, u64, c.c_int, c.c_int]
