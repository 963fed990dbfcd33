"""The collectives as PyTorch custom operators (`torch.ops.stdml_collective.*`),
so that they can be called like any other op (also from traced / compiled
programs, where they appear as opaque mutating calls).  The operators run on a
default `DeviceSession` set with `set_default_session`.

The reference's framework bindings live in separate repositories (README:15-16);
this is their counterpart for PyTorch.
"""
from typing import List

import torch

_default = None


def set_default_session(sess):
    global _default
    _default = sess


def default_session():
    if _default is None:
        raise RuntimeError("no default DeviceSession: call set_default_session(sess) first")
    return _default


@torch.library.custom_op("stdml_collective::all_reduce_", mutates_args=("tensor",),
                         device_types="cuda")
def all_reduce_(tensor: torch.Tensor, op: str = "sum", scale: float = 1.0) -> None:
    default_session().all_reduce(tensor, op=op, scale=None if scale == 1.0 else scale)


@torch.library.custom_op("stdml_collective::group_all_reduce_", mutates_args=("tensors",),
                         device_types="cuda")
def group_all_reduce_(tensors: List[torch.Tensor], op: str = "sum", scale: float = 1.0) -> None:
    default_session().group_all_reduce(list(tensors), op=op,
                                       scale=None if scale == 1.0 else scale)


@torch.library.custom_op("stdml_collective::all_gather", mutates_args=(), device_types="cuda")
def all_gather(tensor: torch.Tensor) -> torch.Tensor:
    sess = default_session()
    out = tensor.new_empty((sess.world * tensor.numel(),))
    sess.all_gather(tensor.contiguous(), out)
    return out


@all_gather.register_fake
def _(tensor):
    return tensor.new_empty((default_session().world * tensor.numel(),))


@torch.library.custom_op("stdml_collective::broadcast_", mutates_args=("tensor",),
                         device_types="cuda")
def broadcast_(tensor: torch.Tensor, root: int = 0) -> None:
    default_session().broadcast(tensor, root=root)


@torch.library.custom_op("stdml_collective::reduce_", mutates_args=("tensor",),
                         device_types="cuda")
def reduce_(tensor: torch.Tensor, op: str = "sum", root: int = 0) -> None:
    default_session().reduce(tensor, op=op, root=root)
