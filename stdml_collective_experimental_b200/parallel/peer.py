"""Python face of the native peer / session model.

    peer = Peer.from_env()          # KungFu, OpenMPI or torchrun variables
    sess = peer.join()
    sess.all_reduce(t)              # torch tensor, CPU (TCP path) or CUDA (NVLink kernels)

Mirrors the reference's C++ API (include/stdml/bits/collective/peer.hpp:16-73,
session.hpp:25-178): all_reduce / group_all_reduce / all_gather / broadcast /
reduce / gather / send / recv / consistent / barrier and the elastic
`peer.resize(sess, ...)`.  CUDA tensors are enqueued on the current CUDA stream.
"""
import ctypes
import os
import json
import weakref

import torch

from .. import _native
from ..ops.device import dtype_code, op_code

_declared = False


def _lib():
    global _declared
    lib = _native.lib()
    if not _declared:
        c = ctypes
        vp, vpp, u64 = c.c_void_p, c.POINTER(c.c_void_p), c.c_ulonglong
        lib.stdmlc_peer_from_env.argtypes = [vpp]
        lib.stdmlc_peer_create.argtypes = [vpp, c.c_int, c.c_char_p, c.c_int, u64, c.c_char_p]
        lib.stdmlc_peer_destroy.argtypes = [vp]
        lib.stdmlc_peer_self.argtypes = [vp, c.c_char_p, u64]
        lib.stdmlc_peer_ping.argtypes = [vp, c.c_char_p, c.c_int, c.POINTER(c.c_double)]
        lib.stdmlc_peer_join.argtypes = [vp, vpp]
        lib.stdmlc_session_destroy.argtypes = [vp]
        lib.stdmlc_session_subgroup.argtypes = [vp, c.POINTER(u64), u64, c.c_char_p, vpp]
        lib.stdmlc_session_info.argtypes = [vp, c.c_int, c.POINTER(u64)]
        lib.stdmlc_session_cluster_json.argtypes = [vp, c.c_char_p, u64]
        lib.stdmlc_session_all_reduce.argtypes = [vp, vp, vp, u64, c.c_int, c.c_int, c.c_char_p, vp]
        lib.stdmlc_session_reduce.argtypes = [vp, vp, vp, u64, c.c_int, c.c_int, c.c_char_p, vp]
        lib.stdmlc_session_group_all_reduce.argtypes = [
            vp, u64, vpp, vpp, c.POINTER(u64), c.c_int, c.c_int, c.POINTER(c.c_char_p),
            c.c_double, vp]
        lib.stdmlc_session_all_gather.argtypes = [vp, vp, vp, u64, c.c_int, c.c_char_p, vp]
        lib.stdmlc_session_gather.argtypes = [vp, vp, vp, u64, c.c_int, c.c_char_p]
        lib.stdmlc_session_broadcast.argtypes = [vp, vp, vp, u64, c.c_int, c.c_char_p, vp]
        lib.stdmlc_session_broadcast_from.argtypes = [vp, vp, vp, u64, c.c_int, c.c_int, c.c_char_p,
                                                      vp]
        lib.stdmlc_session_reduce_to.argtypes = [vp, vp, vp, u64, c.c_int, c.c_int, c.c_int,
                                                 c.c_char_p, vp]
        lib.stdmlc_session_gather_to.argtypes = [vp, vp, vp, u64, c.c_int, c.c_int, c.c_char_p]
        lib.stdmlc_session_reduce_scatter.argtypes = [vp, vp, vp, u64, c.c_int, c.c_int, c.c_char_p, vp]
        lib.stdmlc_session_all_to_all.argtypes = [vp, vp, vp, u64, c.c_int, c.c_char_p, vp]
        lib.stdmlc_session_send.argtypes = [vp, vp, u64, c.c_int, c.c_int, c.c_char_p]
        lib.stdmlc_session_recv.argtypes = [vp, vp, u64, c.c_int, c.c_int, c.c_char_p]
        lib.stdmlc_session_barrier.argtypes = [vp]
        lib.stdmlc_session_symm_alloc.argtypes = [vp, u64, vpp]
        lib.stdmlc_session_symm_free.argtypes = [vp, vp]
        lib.stdmlc_session_device_launches.argtypes = [vp, c.POINTER(u64)]
        lib.stdmlc_session_device_set_knob.argtypes = [vp, c.c_char_p, c.c_longlong]
        lib.stdmlc_session_device_drop_registrations.argtypes = [vp]
        lib.stdmlc_session_device_setup_ms.argtypes = [vp, c.POINTER(c.c_double)]
        lib.stdmlc_session_consistent.argtypes = [vp, vp, u64, c.POINTER(c.c_int)]
        lib.stdmlc_peer_resize.argtypes = [vp, vp, c.c_longlong, c.c_char_p, c.POINTER(c.c_int),
                                           c.POINTER(c.c_int)]
        lib.stdmlc_peer_recover.argtypes = [vp, vp, c.c_int, c.POINTER(c.c_int)]
        lib.stdmlc_cluster_resize_json.argtypes = [c.c_char_p, u64, c.c_char_p, u64]
        lib.stdmlc_session_all_reduce_async.argtypes = [vp, vp, vp, u64, c.c_int, c.c_int,
                                                        c.c_char_p, vp, vpp]
        lib.stdmlc_session_send_async.argtypes = [vp, vp, u64, c.c_int, c.c_int, c.c_char_p, vp, vpp]
        lib.stdmlc_session_recv_async.argtypes = [vp, vp, u64, c.c_int, c.c_int, c.c_char_p, vp, vpp]
        lib.stdmlc_task_poll.argtypes = [vp, c.POINTER(c.c_int)]
        lib.stdmlc_task_finish.argtypes = [vp]
        lib.stdmlc_task_destroy.argtypes = [vp]
        lib.stdmlc_trace_enable.argtypes = [c.c_int]
        lib.stdmlc_trace_write.argtypes = [c.c_char_p]
        _declared = True
    return lib


def _stream_of(t):
    if t.is_cuda:
        return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
    return None


def _checked(t, what):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{what}: torch tensor expected")
    if not t.is_contiguous():
        raise ValueError(f"{what}: contiguous tensor expected")
    return t


class Task:
    """A started operation (the reference's polled `task`): poll() makes progress
    without blocking, wait() polls to completion.  Keeps its tensors alive."""

    def __init__(self, handle, keep):
        self._h = handle
        self._keep = keep
        self._lib = _lib()
        self._done = False

    def poll(self):
        if not self._done:
            fin = ctypes.c_int()
            _native.check(self._lib.stdmlc_task_poll(self._h, ctypes.byref(fin)))
            self._done = bool(fin.value)
        return self._done

    @property
    def finished(self):
        return self.poll()

    def wait(self):
        if not self._done:
            _native.check(self._lib.stdmlc_task_finish(self._h))
            self._done = True
        return self._keep[-1]

    def release(self):
        """Finish the operation if it is still running and free the native task."""
        if self._h is not None:
            if not self._done:
                self._lib.stdmlc_task_finish(self._h)
                self._done = True
            self._lib.stdmlc_task_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class Session:
    """One fixed membership.  Created by Peer.join(); replaced in place by Peer.resize()."""

    def __init__(self, handle):
        self._h = handle
        self._lib = _lib()
        self._tasks = weakref.WeakSet()  # started operations: finished before the session goes

    def _info(self, what):
        v = ctypes.c_ulonglong()
        _native.check(self._lib.stdmlc_session_info(self._h, what, ctypes.byref(v)))
        return int(v.value)

    @property
    def rank(self):
        return self._info(0)

    @property
    def size(self):
        return self._info(1)

    @property
    def version(self):
        return self._info(2)

    @property
    def strategy(self):
        return {1: "ring", 2: "binary_tree", 3: "clique"}.get(self._info(3), "star")

    @property
    def cluster(self):
        """{"Runners": [...], "Workers": [...]} of this session."""
        buf = ctypes.create_string_buffer(1 << 16)
        _native.check(self._lib.stdmlc_session_cluster_json(self._h, buf, len(buf)))
        return json.loads(buf.value.decode())

    def subgroup(self, ranks, scope):
        """A Session of the listed ranks, in that order (like a communicator split).
        Collective among them: all pass the same list and the same `scope`, a name
        unique among the sub-groups alive at one time.  Ranks that are not listed
        get None.  Close it before the parent."""
        arr = (ctypes.c_ulonglong * len(ranks))(*[int(r) for r in ranks])
        h = ctypes.c_void_p()
        _native.check(self._lib.stdmlc_session_subgroup(self._h, arr, len(ranks), scope.encode(),
                                                        ctypes.byref(h)))
        return Session(h) if h.value else None

    def _release_tasks(self):
        """Finish and free every operation started on this session.  A task polls
        the native session it was started on, so none may outlive it: not when the
        session is closed, and not when resize()/recover() replace it in place."""
        for task in list(getattr(self, "_tasks", ())):
            try:
                task.release()
            except Exception:
                pass

    def close(self):
        if self._h is not None:
            self._release_tasks()
            h, self._h = self._h, None
            _native.check(self._lib.stdmlc_session_destroy(h))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------ collectives
    def all_reduce(self, tensor, out=None, op="sum", name=""):
        t = _checked(tensor, "all_reduce")
        o = t if out is None else _checked(out, "all_reduce")
        _native.check(self._lib.stdmlc_session_all_reduce(
            self._h, t.data_ptr(), o.data_ptr(), t.numel(), dtype_code(t.dtype), op_code(op),
            name.encode(), _stream_of(t)))
        return o

    def all_reduce_async(self, tensor, out=None, op="sum", name=""):
        """Start an all_reduce and return a Task.  CPU tensors: the chunk graph runs
        as polled tasks (no thread blocks); CUDA tensors: the kernel is enqueued on
        the current stream and the task finishes when the GPU has run it."""
        t = _checked(tensor, "all_reduce_async")
        o = t if out is None else _checked(out, "all_reduce_async")
        h = ctypes.c_void_p()
        _native.check(self._lib.stdmlc_session_all_reduce_async(
            self._h, t.data_ptr(), o.data_ptr(), t.numel(), dtype_code(t.dtype), op_code(op),
            name.encode(), _stream_of(t), ctypes.byref(h)))
        task = Task(h, (t, o))
        self._tasks.add(task)
        return task

    def reduce(self, tensor, out=None, op="sum", name="", root=0):
        """Result on rank `root` only; `out` of the other ranks is left alone."""
        t = _checked(tensor, "reduce")
        o = t if out is None else _checked(out, "reduce")
        _native.check(self._lib.stdmlc_session_reduce_to(
            self._h, t.data_ptr(), o.data_ptr(), t.numel(), dtype_code(t.dtype), op_code(op),
            int(root), name.encode(), _stream_of(t)))
        return o

    def group_all_reduce(self, tensors, outs=None, op="sum", scale=None, names=None):
        """All tensors of a gradient set in one call (CUDA: one fused launch per
        staging slot; CPU: pipelined, deadlock-free for any arrival order)."""
        ts = [_checked(t, "group_all_reduce") for t in tensors]
        os_ = ts if outs is None else [_checked(t, "group_all_reduce") for t in outs]
        if not ts:
            return tensors
        n = len(ts)
        ins = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
        out_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in os_])
        counts = (ctypes.c_ulonglong * n)(*[t.numel() for t in ts])
        cnames = None
        if names is not None:
            cnames = (ctypes.c_char_p * n)(*[s.encode() for s in names])
        _native.check(self._lib.stdmlc_session_group_all_reduce(
            self._h, n, ins, out_ptrs, counts, dtype_code(ts[0].dtype), op_code(op), cnames,
            1.0 if scale is None else float(scale), _stream_of(ts[0])))
        return outs if outs is not None else tensors

    def all_gather(self, tensor, out, name=""):
        t, o = _checked(tensor, "all_gather"), _checked(out, "all_gather")
        if o.numel() != t.numel() * self.size:
            raise ValueError("all_gather: out must hold size * tensor.numel() elements")
        _native.check(self._lib.stdmlc_session_all_gather(
            self._h, t.data_ptr(), o.data_ptr(), t.numel(), dtype_code(t.dtype), name.encode(),
            _stream_of(t)))
        return o

    def gather(self, tensor, out, name="", root=0):
        """Rank-major blocks on rank `root` (host tensors); `out` matters there only."""
        t, o = _checked(tensor, "gather"), _checked(out, "gather")
        _native.check(self._lib.stdmlc_session_gather_to(
            self._h, t.data_ptr(), o.data_ptr(), t.numel(), dtype_code(t.dtype), int(root),
            name.encode()))
        return o

    def reduce_scatter(self, tensor, out, op="sum", name=""):
        """`tensor` holds size blocks of out.numel() elements; `out` = block `rank`
        reduced over all ranks."""
        t, o = _checked(tensor, "reduce_scatter"), _checked(out, "reduce_scatter")
        if t.numel() != o.numel() * self.size:
            raise ValueError("reduce_scatter: tensor must hold size * out.numel() elements")
        _native.check(self._lib.stdmlc_session_reduce_scatter(
            self._h, t.data_ptr(), o.data_ptr(), o.numel(), dtype_code(t.dtype), op_code(op),
            name.encode(), _stream_of(t)))
        return o

    def all_to_all(self, tensor, out, name=""):
        """Block q of `tensor` goes to rank q; block q of `out` comes from rank q."""
        t, o = _checked(tensor, "all_to_all"), _checked(out, "all_to_all")
        if t.numel() != o.numel() or t.numel() % self.size != 0:
            raise ValueError("all_to_all: both tensors must hold size equal blocks")
        _native.check(self._lib.stdmlc_session_all_to_all(
            self._h, t.data_ptr(), o.data_ptr(), t.numel() // self.size, dtype_code(t.dtype),
            name.encode(), _stream_of(t)))
        return o

    def broadcast(self, tensor, out=None, name="", root=0):
        """From rank `root` to everyone."""
        t = _checked(tensor, "broadcast")
        o = t if out is None else _checked(out, "broadcast")
        _native.check(self._lib.stdmlc_session_broadcast_from(
            self._h, t.data_ptr(), o.data_ptr(), t.numel(), dtype_code(t.dtype), int(root),
            name.encode(), _stream_of(t)))
        return o

    def send(self, tensor, target, name=""):
        """Returns when the tensor may be reused.  CPU tensors: the TCP rendezvous
        message; CUDA tensors: NCCL send on the session's transfer stream, after the
        work the current stream holds."""
        if tensor.is_cuda:
            self.send_async(tensor, target, name).wait()
            return
        t = _checked(tensor, "send")
        _native.check(self._lib.stdmlc_session_send(
            self._h, t.data_ptr(), t.numel(), dtype_code(t.dtype), target, name.encode()))

    def recv(self, out, source, name=""):
        if out.is_cuda:
            return self.recv_async(out, source, name).wait()
        o = _checked(out, "recv")
        _native.check(self._lib.stdmlc_session_recv(
            self._h, o.data_ptr(), o.numel(), dtype_code(o.dtype), source, name.encode()))
        return o

    def send_async(self, tensor, target, name=""):
        """Start a send and return a Task (CUDA tensors: runs beside the collectives
        on a stream of its own; CPU tensors: done when this returns)."""
        t = _checked(tensor, "send_async")
        h = ctypes.c_void_p()
        _native.check(self._lib.stdmlc_session_send_async(
            self._h, t.data_ptr(), t.numel(), dtype_code(t.dtype), int(target), name.encode(),
            _stream_of(t), ctypes.byref(h)))
        task = Task(h, (t,))
        self._tasks.add(task)
        return task

    def recv_async(self, out, source, name=""):
        o = _checked(out, "recv_async")
        h = ctypes.c_void_p()
        _native.check(self._lib.stdmlc_session_recv_async(
            self._h, o.data_ptr(), o.numel(), dtype_code(o.dtype), int(source), name.encode(),
            _stream_of(o), ctypes.byref(h)))
        task = Task(h, (o,))
        self._tasks.add(task)
        return task

    def barrier(self):
        _native.check(self._lib.stdmlc_session_barrier(self._h))

    def symm_empty(self, numel, dtype=torch.float32, device=None):
        """A CUDA tensor in this session's symmetric heap (collective: every rank
        makes the same calls in the same order).  Collectives on it are zero-copy;
        a group of such tensors laid back to back is one fused in-place launch.
        The heap belongs to this membership: after Peer.resize() or recover()
        allocate again (the old tensors must not be used any more)."""
        from ..ops.device import _RawCuda
        nbytes = max(16, int(numel) * torch.empty((), dtype=dtype).element_size())
        p = ctypes.c_void_p()
        _native.check(self._lib.stdmlc_session_symm_alloc(self._h, nbytes, ctypes.byref(p)))
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        raw = torch.as_tensor(_RawCuda(p.value, nbytes, self), device=dev)
        return raw.view(dtype)[:numel]

    def symm_free(self, tensor):
        _native.check(self._lib.stdmlc_session_symm_free(self._h, ctypes.c_void_p(tensor.data_ptr())))

    @property
    def device_setup_ms(self):
        """Where the set-up of this membership's device world went (milliseconds)."""
        out = (ctypes.c_double * 4)()
        _native.check(self._lib.stdmlc_session_device_setup_ms(self._h, out))
        return {"rendezvous": out[0], "own_arena": out[1], "peer_arenas": out[2],
                "multicast": out[3]}

    def device_set_knob(self, name, value):
        """A tuning knob of the device plane (see DeviceSession.set_knob), the same value
        on every rank; e.g. ("register_min_bytes", 0): CUDA tensors are used in place
        through peer mappings of their allocations, a group of them is one launch."""
        _native.check(self._lib.stdmlc_session_device_set_knob(self._h, name.encode(), int(value)))

    def device_drop_registrations(self):
        """Collective: unmap what registered calls mapped (before freeing such tensors)."""
        _native.check(self._lib.stdmlc_session_device_drop_registrations(self._h))

    @property
    def device_launches(self):
        v = ctypes.c_ulonglong()
        _native.check(self._lib.stdmlc_session_device_launches(self._h, ctypes.byref(v)))
        return int(v.value)

    def consistent(self, data):
        """True when every rank holds the same bytes."""
        if isinstance(data, torch.Tensor):
            t = data.detach().cpu().contiguous()
            ptr, size = t.data_ptr(), t.numel() * t.element_size()
            keep = t
        else:
            keep = ctypes.create_string_buffer(bytes(data), len(data))
            ptr, size = ctypes.addressof(keep), len(data)
        same = ctypes.c_int()
        _native.check(self._lib.stdmlc_session_consistent(self._h, ptr, size, ctypes.byref(same)))
        del keep
        return bool(same.value)


def standby_wait():
    """Warm standby hand-over (launcher option -spares N): a process that the launcher
    started without an identity waits here until it is told which worker it is, and
    the identity is put into os.environ; every other process returns at once.
    Peer.from_env() calls it; call it earlier if the program reads the environment
    (a device index, say) before that.  Returns the identity as a dict."""
    lib = _lib()
    lib.stdmlc_standby_wait.restype = ctypes.c_longlong
    lib.stdmlc_standby_wait.argtypes = [ctypes.c_char_p, ctypes.c_ulonglong]
    buf = ctypes.create_string_buffer(1 << 16)
    n = lib.stdmlc_standby_wait(buf, len(buf))
    got = {}
    if n > 0:
        for line in buf.value.decode().splitlines():
            k, eq, v = line.partition("=")
            if eq and k:
                os.environ[k] = v
                got[k] = v
    return got


class Peer:
    def __init__(self, handle):
        self._h = handle
        self._lib = _lib()

    @classmethod
    def from_env(cls):
        standby_wait()
        h = ctypes.c_void_p()
        _native.check(_lib().stdmlc_peer_from_env(ctypes.byref(h)))
        return cls(h)

    @classmethod
    def from_list(cls, rank, peers, strategy="star", version=0, runners=()):
        """peers / runners: 'ip:port' strings."""
        h = ctypes.c_void_p()
        _native.check(_lib().stdmlc_peer_create(
            ctypes.byref(h), rank, ",".join(peers).encode(),
            {"ring": 1, "binary_tree": 2, "tree": 2, "clique": 3}.get(strategy.lower(), 0),
            version, ",".join(runners).encode()))
        return cls(h)

    @property
    def self_id(self):
        buf = ctypes.create_string_buffer(64)
        _native.check(self._lib.stdmlc_peer_self(self._h, buf, len(buf)))
        return buf.value.decode()

    def ping(self, target, timeout_ms=1000):
        """Round trip of one handshake with `target` ("ip:port") in microseconds,
        or None if it does not answer in time."""
        us = ctypes.c_double()
        _native.check(self._lib.stdmlc_peer_ping(self._h, target.encode(), timeout_ms,
                                                 ctypes.byref(us)))
        return us.value if us.value >= 0 else None

    def join(self):
        s = ctypes.c_void_p()
        _native.check(self._lib.stdmlc_peer_join(self._h, ctypes.byref(s)))
        return Session(s)

    def resize(self, sess, new_size=None, cluster=None):
        """Change the membership of `sess` in place.

        new_size: propose that many workers to the config server, then follow it;
        cluster: an explicit {"Runners": [...], "Workers": [...]} dict (no server);
        neither: follow the config server.  Returns (changed, detached)."""
        sess._release_tasks()  # the native session is replaced: its tasks go first
        changed, detached = ctypes.c_int(), ctypes.c_int()
        js = None if cluster is None else json.dumps(cluster).encode()
        _native.check(self._lib.stdmlc_peer_resize(
            self._h, sess._h, -1 if new_size is None else int(new_size), js,
            ctypes.byref(changed), ctypes.byref(detached)))
        return bool(changed.value), bool(detached.value)

    def recover(self, sess, ping_timeout_ms=1000):
        """After a PeerFailure: every surviving rank calls this.  `sess` becomes, in
        place, a session of the members that still answer (ranks keep their order,
        the version goes up by one).  Returns the number of members dropped.  As
        after a resize, re-synchronise progress and parameters afterwards."""
        # unfinished operations of the broken session end here (with its failure);
        # afterwards nothing refers to the native session that recover() destroys
        sess._release_tasks()
        dropped = ctypes.c_int()
        _native.check(self._lib.stdmlc_peer_recover(self._h, sess._h, int(ping_timeout_ms),
                                                    ctypes.byref(dropped)))
        return dropped.value

    def close(self):
        if self._h is not None:
            h, self._h = self._h, None
            _native.check(self._lib.stdmlc_peer_destroy(h))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def resized_cluster(cluster, new_size):
    """cluster_config::resize on a {"Runners", "Workers"} dict."""
    buf = ctypes.create_string_buffer(1 << 16)
    _native.check(_lib().stdmlc_cluster_resize_json(json.dumps(cluster).encode(), new_size, buf,
                                                    len(buf)))
    return json.loads(buf.value.decode())


def enable_trace(on=True):
    _lib().stdmlc_trace_enable(1 if on else 0)


def write_trace(path):
    """Chrome-trace JSON of the recorded events."""
    return _lib().stdmlc_trace_write(path.encode()) == 0
