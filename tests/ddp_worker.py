"""One rank of the data-parallel test: a small conv net trained for a few steps
with DataParallel must match (a) the same model trained on one process with the
concatenated batch (gradient averaging is exact up to float rounding) and (b)
stay identical across ranks."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from stdml_collective_experimental_b200 import DeviceSession  # noqa: E402
from stdml_collective_experimental_b200.parallel.ddp import DataParallel  # noqa: E402


def make_model():
    torch.manual_seed(7)
    return torch.nn.Sequential(
        torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(8, 4, 3, padding=1),
        torch.nn.ReLU(), torch.nn.AdaptiveAvgPool2d(4), torch.nn.Flatten(),
        torch.nn.Linear(64, 10))


def data(rank):
    g = torch.Generator().manual_seed(1000 + rank)
    return torch.randn(6, 3, 16, 16, generator=g), torch.randint(0, 10, (6,), generator=g)


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    sess = DeviceSession.from_env(heap_bytes=64 << 20, staging_bytes=4 << 20)
    model = make_model().to(dev)
    if rank != 0:  # broadcast_parameters must repair this
        with torch.no_grad():
            for p in model.parameters():
                p.add_(1.0)
    ddp = DataParallel(model, sess, buckets=3)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.1)
    x, y = (t.to(dev) for t in data(rank))
    for _ in range(3):
        ddp.zero_grad()
        torch.nn.functional.cross_entropy(ddp(x), y).backward()
        opt.step()
    torch.cuda.synchronize()
    sess.check()

    # reference: one process, all ranks' batches, mean of per-rank mean losses
    ref = make_model().to(dev)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    batches = [tuple(t.to(dev) for t in data(r)) for r in range(world)]
    for _ in range(3):
        ropt.zero_grad()
        loss = sum(torch.nn.functional.cross_entropy(ref(bx), by) for bx, by in batches) / world
        loss.backward()
        ropt.step()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-5), float((p - q).abs().max())
    # identical on every rank, bit for bit
    flat = torch.cat([p.detach().flatten() for p in model.parameters()])
    lo, hi = flat.clone(), flat.clone()
    sess.all_reduce(lo, op="min")
    sess.all_reduce(hi, op="max")
    torch.cuda.synchronize()
    assert torch.equal(lo, hi)

    # gradient accumulation: two micro-batches, the first without communication
    x2, y2 = (t.to(dev) for t in data(rank + 100))
    ddp.zero_grad()
    with ddp.no_sync():
        torch.nn.functional.cross_entropy(ddp(x), y).backward()
    torch.nn.functional.cross_entropy(ddp(x2), y2).backward()
    opt.step()
    torch.cuda.synchronize()
    sess.check()
    ropt.zero_grad()
    batches2 = [tuple(t.to(dev) for t in data(r + 100)) for r in range(world)]
    loss = sum(torch.nn.functional.cross_entropy(ref(bx), by) for bx, by in batches + batches2) / world
    loss.backward()
    ropt.step()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-5), float((p - q).abs().max())
    ddp.close()
    sess.close()
    print(f"OK rank {rank}", flush=True)


if __name__ == "__main__":
    main()
