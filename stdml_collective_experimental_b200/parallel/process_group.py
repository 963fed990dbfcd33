"""A torch.distributed backend on top of this package's Session, so that code
written against torch.distributed (DistributedDataParallel included) runs on
these collectives unchanged:

    import stdml_collective_experimental_b200.parallel.process_group  # registers "stdml"
    torch.distributed.init_process_group("stdml", init_method="tcp://...", rank=r, world_size=n)
    torch.distributed.all_reduce(t)        # CPU tensors: TCP path; CUDA tensors: NVLink kernels

The ranks find each other through torch's store: each publishes the address its
peer listens on, then all build the same peer list (rank order) and join one
session.  Operations are issued in program order on every rank, as
torch.distributed requires, so message names are a running counter.

The reference has no PyTorch binding; its session
(include/stdml/bits/collective/session.hpp:25-178) is what the backend drives:
all_reduce, broadcast, all_gather, reduce, send/recv, barrier; the remaining
torch collectives (reduce_scatter, gather, scatter, all_to_all) are composed from
those.  CUDA work is enqueued on the current stream and the returned Work is
complete in stream order, like NCCL's.
"""
import os
import socket

import torch
import torch.distributed as dist

from .peer import Peer

_REDUCE_OPS = {
    dist.ReduceOp.SUM: "sum", dist.ReduceOp.MIN: "min", dist.ReduceOp.MAX: "max",
    dist.ReduceOp.PRODUCT: "prod", dist.ReduceOp.BXOR: "bit_xor",
}


class _DoneWork(dist._Work):
    """Work that is finished when it is returned (host path), or ordered on the
    current CUDA stream (device path)."""

    def __init__(self, result):
        super().__init__()
        self._future = torch.futures.Future()
        self._future.set_result(result)

    def wait(self, timeout=None):
        return True

    def is_completed(self):
        return True

    def is_success(self):
        return True

    def get_future(self):
        return self._future

    def result(self):
        return self._future.value()


def _op_of(opts):
    op = getattr(opts, "reduceOp", dist.ReduceOp.SUM)
    # ReduceOp objects compare equal to their RedOpType
    for k, v in _REDUCE_OPS.items():
        if op == k:
            return v, False
    if op == dist.ReduceOp.AVG:
        return "sum", True
    raise NotImplementedError(f"stdml backend: reduce op {op} is not supported")


def _local_address(store_host):
    """The address other ranks can reach this one at."""
    if store_host in ("127.0.0.1", "localhost", "", None):
        return "127.0.0.1"
    try:
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as s:
            s.connect((store_host, 9))  # no packet is sent: picks the outgoing interface
            return s.getsockname()[0]
    except OSError:
        return "127.0.0.1"


def _free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("", 0))
        return s.getsockname()[1]


class StdmlProcessGroup(dist.ProcessGroup):
    def __init__(self, store, rank, size, timeout=None):
        super().__init__(rank, size)
        self._rank, self._size = rank, size
        ip = _local_address(os.environ.get("MASTER_ADDR", "127.0.0.1"))
        base = os.environ.get("STDML_COLLECTIVE_BASE_PORT")
        port = int(base) + rank if base else _free_port()
        store.set(f"stdml/addr/{rank}", f"{ip}:{port}")
        peers = [store.get(f"stdml/addr/{r}").decode() for r in range(size)]
        strategy = os.environ.get("KUNGFU_ALLREDUCE_STRATEGY", "STAR").lower()
        self.peer = Peer.from_list(rank, peers, strategy=strategy)
        self.sess = self.peer.join()
        self._seq = 0

    # -------------------------------------------------------------- plumbing
    def getBackendName(self):
        return "stdml"

    def _name(self, what):
        self._seq += 1
        return f"pg/{what}/{self._seq}"

    @staticmethod
    def _dense(t):
        return t if t.is_contiguous() else t.contiguous()

    def _each(self, tensors, fn):
        """Runs fn on a contiguous version of every tensor and copies back if needed."""
        for t in tensors:
            d = self._dense(t)
            fn(d)
            if d is not t:
                t.copy_(d)

    # ----------------------------------------------------------- collectives
    def allreduce(self, tensors, opts=None):
        op, average = _op_of(opts)

        def one(t):
            self.sess.all_reduce(t, op=op, name=self._name("ar"))
            if average:
                t.div_(self._size)
        self._each(tensors, one)
        return _DoneWork(tensors)

    def allreduce_coalesced(self, tensors, opts=None):
        if len({t.dtype for t in tensors}) > 1:  # a fused group has one element type
            return self.allreduce(tensors, opts)
        op, average = _op_of(opts)
        dense = [self._dense(t) for t in tensors]
        names = [self._name("arc") for _ in dense]
        self.sess.group_all_reduce(dense, op=op, names=names,
                                   scale=(1.0 / self._size) if average else None)
        for d, t in zip(dense, tensors):
            if d is not t:
                t.copy_(d)
        return _DoneWork(tensors)

    def broadcast(self, tensors, opts=None):
        root = getattr(opts, "rootRank", 0)
        self._each(tensors, lambda t: self.sess.broadcast(t, root=root, name=self._name("bc")))
        return _DoneWork(tensors)

    def reduce(self, tensors, opts=None):
        op, average = _op_of(opts)
        root = getattr(opts, "rootRank", 0)
        for t in tensors:
            src = self._dense(t)
            out = torch.empty_like(src) if self._rank == root else src  # others keep their tensor
            self.sess.reduce(src, out=out, op=op, root=root, name=self._name("rd"))
            if self._rank == root:
                t.copy_(out.div_(self._size) if average else out)
        return _DoneWork(tensors)

    def _allgather_base(self, output, input, opts=None):
        out = output if output.is_contiguous() else torch.empty_like(
            output, memory_format=torch.contiguous_format)
        self.sess.all_gather(self._dense(input).view(-1), out.view(-1), name=self._name("ag"))
        if out is not output:
            output.copy_(out)
        return _DoneWork(output)

    def allgather(self, output_tensors, input_tensors, opts=None):
        for outs, inp in zip(output_tensors, input_tensors):
            flat = torch.empty(self._size * inp.numel(), dtype=inp.dtype, device=inp.device)
            self.sess.all_gather(self._dense(inp).view(-1), flat, name=self._name("ag"))
            for r, o in enumerate(outs):
                o.copy_(flat[r * inp.numel():(r + 1) * inp.numel()].view_as(o))
        return _DoneWork(output_tensors)

    def allgather_into_tensor_coalesced(self, outputs, inputs, opts=None):
        for o, i in zip(outputs, inputs):
            self._allgather_base(o, i, opts)
        return _DoneWork(outputs)

    def _reduce_scatter_base(self, output, input, opts=None):
        op, average = _op_of(opts)
        out = output if output.is_contiguous() else torch.empty_like(
            output, memory_format=torch.contiguous_format)
        self.sess.reduce_scatter(self._dense(input).view(-1), out.view(-1), op=op,
                                 name=self._name("rs"))
        if average:
            out.div_(self._size)
        if out is not output:
            output.copy_(out)
        return _DoneWork(output)

    def reduce_scatter(self, output_tensors, input_tensors, opts=None):
        for out, ins in zip(output_tensors, input_tensors):
            self._reduce_scatter_base(out, torch.cat([self._dense(t).view(-1) for t in ins]), opts)
        return _DoneWork(output_tensors)

    def reduce_scatter_tensor_coalesced(self, outputs, inputs, opts=None):
        for o, i in zip(outputs, inputs):
            self._reduce_scatter_base(o, i, opts)
        return _DoneWork(outputs)

    def barrier(self, opts=None):
        self.sess.barrier()
        return _DoneWork(None)

    # -------------------------------------------------------- point to point
    # A rendezvous message whose destination is not posted yet is parked at the
    # receiver, so a send never waits for the matching recv: the composed
    # collectives below send everything first and receive afterwards.
    def send(self, tensors, dst, tag=0):
        for i, t in enumerate(tensors):
            self.sess.send(self._dense(t), dst, name=f"pg/p2p/{tag}/{i}")
        return _DoneWork(None)

    def recv(self, tensors, src, tag=0):
        for i, t in enumerate(tensors):
            d = t if t.is_contiguous() else torch.empty_like(t, memory_format=torch.contiguous_format)
            self.sess.recv(d, src, name=f"pg/p2p/{tag}/{i}")
            if d is not t:
                t.copy_(d)
        return _DoneWork(tensors)

    # gather, scatter and all_to_all are built from point-to-point messages in
    # which ranks may all send before any of them receives.  Host messages are
    # buffered, so that is fine there; device transfers (NCCL kernels) would wait
    # for each other for ever.  CUDA tensors of these three calls therefore travel
    # as host messages (a copy out and a copy in); they are not hot paths.
    @staticmethod
    def _wire(t):
        return t.detach().cpu().contiguous() if t.is_cuda else StdmlProcessGroup._dense(t)

    @staticmethod
    def _landing(o):
        return torch.empty(o.shape, dtype=o.dtype, device="cpu")

    def gather(self, output_tensors, input_tensors, opts=None):
        root = getattr(opts, "rootRank", 0)
        name = self._name("ga")
        for k, inp in enumerate(input_tensors):
            if self._rank != root:
                self.sess.send(self._wire(inp), root, name=f"{name}/{k}")
                continue
            for r, o in enumerate(output_tensors[k]):
                if r == root:
                    o.copy_(inp)
                else:
                    d = self._landing(o)
                    self.sess.recv(d, r, name=f"{name}/{k}")
                    o.copy_(d)
        return _DoneWork(output_tensors)

    def scatter(self, output_tensors, input_tensors, opts=None):
        root = getattr(opts, "rootRank", 0)
        name = self._name("sc")
        for k, out in enumerate(output_tensors):
            if self._rank == root:
                for r, t in enumerate(input_tensors[k]):
                    if r == root:
                        out.copy_(t)
                    else:
                        self.sess.send(self._wire(t), r, name=f"{name}/{k}")
            else:
                d = self._landing(out)
                self.sess.recv(d, root, name=f"{name}/{k}")
                out.copy_(d)
        return _DoneWork(output_tensors)

    def alltoall(self, output_tensors, input_tensors, opts=None):
        name = self._name("a2a")
        for r, t in enumerate(input_tensors):
            if r != self._rank:
                self.sess.send(self._wire(t), r, name=name)
        for r, o in enumerate(output_tensors):
            if r == self._rank:
                o.copy_(input_tensors[r])
            else:
                d = self._landing(o)
                self.sess.recv(d, r, name=name)
                o.copy_(d)
        return _DoneWork(output_tensors)

    def alltoall_base(self, output, input, output_split_sizes, input_split_sizes, opts=None):
        n = self._size
        if not input_split_sizes and not output_split_sizes and input.is_contiguous() and \
                output.is_contiguous() and input.numel() == output.numel():
            self.sess.all_to_all(input.view(-1), output.view(-1), name=self._name("a2ab"))
            return _DoneWork(output)
        ins = list(input.split(input_split_sizes if input_split_sizes else input.shape[0] // n))
        outs = list(output.split(output_split_sizes if output_split_sizes else output.shape[0] // n))
        tmp = [torch.empty_like(o, memory_format=torch.contiguous_format) for o in outs]
        self.alltoall(tmp, ins, opts)
        for o, t in zip(outs, tmp):
            o.copy_(t)
        return _DoneWork(output)

    def shutdown(self):
        if self.sess is not None:
            self.sess.close()
            self.peer.close()
            self.sess = self.peer = None

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass


def _create(store, rank, size, timeout):
    return StdmlProcessGroup(store, rank, size, timeout)


def register():
    """Makes `backend="stdml"` known to torch.distributed (idempotent)."""
    if "STDML" not in getattr(dist.Backend, "backend_list", []) and not hasattr(dist.Backend, "STDML"):
        dist.Backend.register_backend("stdml", _create, devices=["cpu", "cuda"])


register()
