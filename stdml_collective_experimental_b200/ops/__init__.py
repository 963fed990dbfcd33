"""Device collectives: thin Python layer over the sm_100a kernels."""
from .device import (ALGO_NVLS, ALGO_NVLS_ONESHOT, ALGO_ONESHOT, ALGO_TWOSHOT, DeviceSession,
                     dtype_code, op_code)

__all__ = ["DeviceSession", "dtype_code", "op_code", "ALGO_ONESHOT", "ALGO_TWOSHOT", "ALGO_NVLS",
           "ALGO_NVLS_ONESHOT"]
