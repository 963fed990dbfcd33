"""CPU oracle of the reducers: the native host `reduce_many` (rank-ascending,
16-bit floats accumulated in f32 and rounded once), called on CPU tensors."""
import ctypes

import torch

from .. import _native
from ..ops.device import dtype_code, op_code


def reduce_many(tensors, op="sum", scale=None):
    """Reduce a list of equally shaped CPU tensors; returns a new CPU tensor."""
    ts = [t.detach().cpu().contiguous() for t in tensors]
    out = torch.empty_like(ts[0])
    arr = (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    rc = _native.lib().stdmlc_reduce_many(
        out.data_ptr(), arr, len(ts), out.numel(), dtype_code(out.dtype), op_code(op),
        1.0 if scale is None else float(scale))
    if rc != 0:
        raise ValueError(f"reduce_many: {op} is not defined for {out.dtype}")
    return out
