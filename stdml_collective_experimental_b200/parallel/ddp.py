"""Data-parallel training on the fused device collectives.

`DataParallel` keeps every gradient of a module in ONE flat buffer inside the
symmetric heap (`.grad` tensors are views), so the gradient all-reduce is
zero-copy: each bucket is a contiguous range of that buffer and one fused kernel
launch reduces it in place over NVLink with the 1/world scale applied in
registers.  Buckets are launched from autograd hooks on a side stream as soon as
their gradients are complete, so communication overlaps the rest of backward.
Inside `no_sync()` backward only accumulates into the flat buffer; the next
backward outside it reduces the accumulated sum (gradient accumulation over
micro-batches with one all-reduce per optimizer step).

This is the PyTorch-side counterpart of the reference's `group_all_reduce`
(src/stdml/collective/session.cpp:83-97), which its framework bindings call
with one future per gradient.
"""
import contextlib

import torch

from ..ops.device import DeviceSession


class DataParallel(torch.nn.Module):
    def __init__(self, module, sess: DeviceSession, buckets=4, average=True, algo=None,
                 broadcast_parameters=True):
        super().__init__()
        if sess.vranks != 1:
            raise ValueError("DataParallel needs a real (one GPU per process) session")
        self.module = module
        self.sess = sess
        self.algo = algo
        self.scale = (1.0 / sess.world) if average else None
        params = [p for p in module.parameters() if p.requires_grad]
        if not params:
            raise ValueError("module has no trainable parameters")
        dtypes = {p.dtype for p in params}
        if len(dtypes) != 1:
            raise ValueError("DataParallel: parameters of one dtype expected, got %s" % dtypes)
        self.dtype = params[0].dtype
        # gradients become ready roughly in reverse registration order
        self.params = list(reversed(params))
        esize = params[0].element_size()
        lane = 16 // esize
        offs, total = [], 0
        for p in self.params:
            offs.append(total)
            total += -(-p.numel() // lane) * lane  # every tensor starts on a 16-byte boundary
        self.flat = sess.symm_empty(total, self.dtype)
        self.flat.zero_()
        for p, off in zip(self.params, offs):
            # same strides as the parameter (e.g. channels_last), so autograd
            # accumulates in place without a layout conversion
            dense = p.is_contiguous() or p.is_contiguous(memory_format=torch.channels_last) \
                if p.dim() == 4 else p.is_contiguous()
            if dense:
                p.grad = torch.as_strided(self.flat, p.size(), p.stride(), off)
            else:
                p.grad = self.flat[off:off + p.numel()].view_as(p)
        # contiguous buckets of about equal bytes, in readiness order
        nb = max(1, min(buckets, len(self.params)))
        target = total / nb
        self.bucket_of, self.bounds = [], []
        lo, b = 0, 0
        for i, (p, off) in enumerate(zip(self.params, offs)):
            self.bucket_of.append(b)
            end = offs[i + 1] if i + 1 < len(offs) else total
            if (end - lo >= target and b < nb - 1) or i + 1 == len(self.params):
                self.bounds.append((lo, end))
                lo, b = end, b + 1
        self.nbuckets = len(self.bounds)
        self.need = [self.bucket_of.count(k) for k in range(self.nbuckets)]
        self.comm = torch.cuda.Stream(sess.device)
        self._ready = [0] * self.nbuckets
        self._launched = 0
        self._callback_queued = False
        self._sync = True
        self._events = [torch.cuda.Event() for _ in range(self.nbuckets)]
        for i, p in enumerate(self.params):
            p.register_post_accumulate_grad_hook(self._make_hook(self.bucket_of[i]))
        if broadcast_parameters and sess.world > 1:
            self.broadcast_parameters()

    # ------------------------------------------------------------------ hooks
    def _make_hook(self, bucket):
        def hook(_param):
            if not self._sync:
                return  # accumulating: the reduction waits for a backward outside no_sync()
            if not self._callback_queued:
                self._callback_queued = True
                torch.autograd.Variable._execution_engine.queue_callback(self._finish)
            self._ready[bucket] += 1
            # launch in bucket order so that every rank issues the same sequence
            while (self._launched < self.nbuckets and
                   self._ready[self._launched] >= self.need[self._launched]):
                self._launch(self._launched)
                self._launched += 1
        return hook

    def _launch(self, k):
        lo, hi = self.bounds[k]
        ev = self._events[k]
        ev.record(torch.cuda.current_stream(self.sess.device))
        self.comm.wait_event(ev)
        self.sess.all_reduce(self.flat[lo:hi], scale=self.scale, algo=self.algo, stream=self.comm)

    def _finish(self):
        # parameters whose gradient was never produced (unused in this step)
        while self._launched < self.nbuckets:
            self._launch(self._launched)
            self._launched += 1
        torch.cuda.current_stream(self.sess.device).wait_stream(self.comm)
        self._ready = [0] * self.nbuckets
        self._launched = 0
        self._callback_queued = False

    # -------------------------------------------------------------------- API
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context add to the local gradients without
        communicating; every rank must use it for the same steps."""
        old, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = old

    def zero_grad(self, set_to_none=False):
        """Zeroes the flat gradient buffer (the views must stay in place)."""
        self.flat.zero_()

    def broadcast_parameters(self, root=0):
        """Every rank takes rank `root`'s parameters and buffers (also used after a resize)."""
        with torch.no_grad():
            for t in list(self.module.parameters()) + list(self.module.buffers()):
                if t.is_floating_point() or t.dtype in (torch.int64, torch.int32):
                    if t.is_contiguous():
                        self.sess.broadcast(t.data, root=root)
                    else:  # e.g. channels_last weights: through a dense copy and back
                        dense = t.data.contiguous()
                        self.sess.broadcast(dense, root=root)
                        t.data.copy_(dense)
        torch.cuda.current_stream(self.sess.device).synchronize()

    def close(self):
        for p in self.params:
            p.grad = None
        self.sess.symm_free(self.flat)
