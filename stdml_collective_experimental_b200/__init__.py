"""B200-native collective communication library with the capabilities of
stdml-collective: peer/session model, all_reduce / group_all_reduce / all_gather /
broadcast / reduce / send / recv, star and ring strategies, async task runtime,
elastic resize, MPI-compatible C interface; the device paths are hand-written
sm_100a kernels over NVLink peer memory."""
from . import _native
from ._native import DeviceTimeoutError, NativeError, PeerFailure, build
from .ops.device import DeviceSession

__all__ = ["DeviceSession", "DeviceTimeoutError", "NativeError", "PeerFailure", "build", "_native"]
__version__ = "0.1.0"
