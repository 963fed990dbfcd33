"""Data-parallel training through a `Session` (host or device tensors):

    peer = Peer.from_env(); sess = peer.join()
    broadcast_parameters(model, sess)                 # everyone starts from rank 0's weights
    opt = DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1), sess)
    loss.backward(); opt.step()                       # gradients are averaged, then applied

`step()` hands ALL gradients to one `group_all_reduce` (CUDA tensors: one fused
launch per staging slot with the 1/size scale in the kernel; CPU tensors: the
pipelined TCP path, any arrival order) -- the call the reference's framework
bindings are built around (src/stdml/collective/session.cpp:83-97).  For CUDA
models `DataParallel` (ddp.py) additionally overlaps the all-reduce with backward.
"""
import torch


def broadcast_parameters(module, sess):
    """Parameters and buffers of `module` on every rank := rank 0's."""
    with torch.no_grad():
        for i, t in enumerate(list(module.parameters()) + list(module.buffers())):
            if t.numel() == 0:
                continue
            flat = t.data.contiguous()
            sess.broadcast(flat, name=f"stdml::param:{i}")
            if flat.data_ptr() != t.data.data_ptr():
                t.data.copy_(flat)


class DistributedOptimizer:
    def __init__(self, optimizer, sess, average=True):
        self.optimizer = optimizer
        self.sess = sess
        self.average = average
        self.param_groups = optimizer.param_groups

    def _grads(self):
        out = []
        for group in self.optimizer.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    out.append(p.grad)
        return out

    def synchronize(self):
        """All-reduce (and average) every gradient, one group per dtype."""
        by_dtype = {}
        for g in self._grads():
            if not g.is_contiguous():
                raise ValueError("DistributedOptimizer: contiguous gradients expected")
            by_dtype.setdefault(g.dtype, []).append(g)
        scale = (1.0 / self.sess.size) if self.average else None
        for k, (dt, grads) in enumerate(by_dtype.items()):
            names = [f"stdml::grad:{k}:{i}" for i in range(len(grads))]
            self.sess.group_all_reduce(grads, scale=scale if dt.is_floating_point else None,
                                       names=names)

    def step(self, closure=None):
        self.synchronize()
        return self.optimizer.step(closure)

    def zero_grad(self, set_to_none=True):
        self.optimizer.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, state):
        self.optimizer.load_state_dict(state)
