"""Membership, sessions, data-parallel helpers."""
from .optimizer import DistributedOptimizer, broadcast_parameters
from .peer import Peer, Session, Task, enable_trace, resized_cluster, write_trace

__all__ = ["DistributedOptimizer", "broadcast_parameters", "Peer", "Session", "Task", "enable_trace", "resized_cluster", "write_trace"]
