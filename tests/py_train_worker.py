"""One rank of the CPU data-parallel training test."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from stdml_collective_experimental_b200.parallel import Peer  # noqa: E402
from stdml_collective_experimental_b200.parallel.optimizer import (DistributedOptimizer,  # noqa: E402
                                                                    broadcast_parameters)


def make_model(seed):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(20, 32), torch.nn.Tanh(), torch.nn.Linear(32, 5))


def batch(rank):
    g = torch.Generator().manual_seed(500 + rank)
    return torch.randn(16, 20, generator=g), torch.randint(0, 5, (16,), generator=g)


def main():
    rank, n, base = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    peer = Peer.from_list(rank, [f"127.0.0.1:{base + i}" for i in range(n)], strategy="ring")
    sess = peer.join()
    model = make_model(seed=rank)          # different everywhere ...
    broadcast_parameters(model, sess)      # ... until rank 0's weights arrive
    opt = DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.2, momentum=0.9), sess)
    x, y = batch(rank)
    for _ in range(5):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()

    ref = make_model(seed=0)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.2, momentum=0.9)
    batches = [batch(r) for r in range(n)]
    for _ in range(5):
        ropt.zero_grad()
        loss = sum(torch.nn.functional.cross_entropy(ref(bx), by) for bx, by in batches) / n
        loss.backward()
        ropt.step()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-6), float((p - q).abs().max())
    flat = torch.cat([p.detach().flatten() for p in model.parameters()])
    assert sess.consistent(flat), "ranks must hold identical weights"
    sess.close()
    peer.close()
    print(f"rank {rank} OK", flush=True)


if __name__ == "__main__":
    main()
