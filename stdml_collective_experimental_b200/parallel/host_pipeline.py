"""All-reduce of HOST-memory gradient sets through the GPUs.

The reference reduces host buffers over TCP
(src/stdml/collective/session.cpp:64-111).  Here a pinned host buffer is cut
into chunks and each chunk flows host -> device (copy engine) -> fused
all-reduce kernel over NVLink -> host, with the three stages of different
chunks overlapped on three streams.  The device side is zero-copy: chunks land
directly in the symmetric heap and are reduced in place.
"""
import torch


class HostAllReduce:
    def __init__(self, sess, numel, dtype=torch.float32, chunks=8):
        if sess.vranks != 1:
            raise ValueError("HostAllReduce needs a real (one GPU per process) session")
        self.sess = sess
        self.numel = numel
        self.dtype = dtype
        self.flat = sess.symm_empty(numel, dtype)
        align = 4096
        per = -(-numel // chunks)
        per = -(-per // align) * align
        self.bounds = [(lo, min(lo + per, numel)) for lo in range(0, numel, per)]
        dev = sess.device
        self.h2d = torch.cuda.Stream(dev)
        self.comm = torch.cuda.Stream(dev)
        self.d2h = torch.cuda.Stream(dev)
        self.ev_in = [torch.cuda.Event() for _ in self.bounds]
        self.ev_red = [torch.cuda.Event() for _ in self.bounds]
        self.launches_per_run = len(self.bounds)

    @property
    def h2d_bytes(self):
        return self.numel * self.flat.element_size()

    d2h_bytes = h2d_bytes

    def run(self, host_in, host_out, op="sum", scale=None):
        """host_out = scale * all_reduce(host_in); both pinned, flat, `numel` long.
        Returns when host_out is complete."""
        for name, t in (("host_in", host_in), ("host_out", host_out)):
            if t.is_cuda or t.dtype != self.dtype or t.numel() != self.numel or not t.is_contiguous():
                raise ValueError(f"HostAllReduce.run: {name} must be a contiguous host tensor of "
                                 f"{self.numel} x {self.dtype}")
            if not t.is_pinned():
                raise ValueError(f"HostAllReduce.run: {name} must be pinned (a pageable buffer "
                                 "makes every copy synchronous and ends the overlap)")
        cur = torch.cuda.current_stream(self.sess.device)
        for s in (self.h2d, self.comm, self.d2h):
            s.wait_stream(cur)
        for i, (lo, hi) in enumerate(self.bounds):
            with torch.cuda.stream(self.h2d):
                self.flat[lo:hi].copy_(host_in[lo:hi], non_blocking=True)
                self.ev_in[i].record(self.h2d)
            self.comm.wait_event(self.ev_in[i])
            self.sess.all_reduce(self.flat[lo:hi], op=op, scale=scale, stream=self.comm)
            self.ev_red[i].record(self.comm)
            self.d2h.wait_event(self.ev_red[i])
            with torch.cuda.stream(self.d2h):
                host_out[lo:hi].copy_(self.flat[lo:hi], non_blocking=True)
        self.d2h.synchronize()
        return host_out

    def close(self):
        self.sess.symm_free(self.flat)
