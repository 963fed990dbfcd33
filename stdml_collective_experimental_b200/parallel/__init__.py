"""Membership, sessions, data-parallel helpers."""
from .peer import Peer, Session, Task, enable_trace, resized_cluster, write_trace

__all__ = ["Peer", "Session", "Task", "enable_trace", "resized_cluster", "write_trace"]
