"""One rank of the torch.distributed backend test (spawned by test_python_api.py,
and with a fourth argument "cuda" by test_device_multigpu.py): every
torch.distributed collective through backend "stdml" on CPU (or CUDA) tensors, then
DistributedDataParallel against single-process training on the joint batch."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import stdml_collective_experimental_b200.parallel.process_group  # noqa: E402,F401  (registers "stdml")


def make_model():
    torch.manual_seed(11)
    return torch.nn.Sequential(torch.nn.Linear(12, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))


def data(rank):
    g = torch.Generator(device="cpu").manual_seed(500 + rank)
    x = torch.randn(8, 12, generator=g, device="cpu")
    y = torch.randn(8, 4, generator=g, device="cpu")
    dev = torch.get_default_device()
    return x.to(dev), y.to(dev)


def main():
    rank, n, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    if len(sys.argv) > 4 and sys.argv[4] == "cuda":
        # the same calls on CUDA tensors: one GPU per rank, every factory call below
        # then makes device tensors and the backend takes the NVLink kernels
        os.environ["STDML_COLLECTIVE_DEVICE_ID"] = str(rank)
        torch.cuda.set_device(rank)
        torch.set_default_device(torch.device("cuda", rank))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    dist.init_process_group("stdml", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=n)
    assert dist.get_backend() == "stdml" and dist.get_rank() == rank and dist.get_world_size() == n

    t = torch.arange(1000, dtype=torch.float32) + rank
    dist.all_reduce(t)
    assert torch.equal(t, torch.arange(1000, dtype=torch.float32) * n + n * (n - 1) / 2)
    t = torch.full((5,), float(rank + 1))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert torch.all(t == n)
    t = torch.full((4,), float(rank))
    dist.all_reduce(t, op=dist.ReduceOp.AVG)
    assert torch.allclose(t, torch.full((4,), (n - 1) / 2))
    t = torch.full((3, 4), float(rank)).t()  # not contiguous
    dist.all_reduce(t)
    assert torch.all(t == n * (n - 1) / 2)

    b = torch.full((7,), float(rank))
    dist.broadcast(b, src=n - 1)
    assert torch.all(b == n - 1)

    outs = [torch.empty(3, dtype=torch.int64) for _ in range(n)]
    dist.all_gather(outs, torch.full((3,), rank, dtype=torch.int64))
    assert [int(o[0]) for o in outs] == list(range(n))
    flat = torch.empty(n * 2)
    dist.all_gather_into_tensor(flat, torch.full((2,), float(rank)))
    assert flat.tolist() == [float(r) for r in range(n) for _ in range(2)]

    r = torch.full((4,), float(rank + 1))
    dist.reduce(r, dst=1)
    if rank == 1:
        assert torch.all(r == n * (n + 1) / 2)
    else:
        assert torch.all(r == rank + 1)

    rs = torch.empty(2)
    dist.reduce_scatter_tensor(rs, torch.arange(2 * n, dtype=torch.float32) + rank)
    want = torch.arange(2 * n, dtype=torch.float32) * n + n * (n - 1) / 2
    assert torch.equal(rs, want[2 * rank:2 * rank + 2])

    if rank == 0:
        dist.send(torch.tensor([42.0]), dst=n - 1, tag=3)
    elif rank == n - 1:
        got = torch.zeros(1)
        dist.recv(got, src=0, tag=3)
        assert got.item() == 42.0

    gathered = [torch.empty(2) for _ in range(n)] if rank == 0 else None
    dist.gather(torch.full((2,), float(rank)), gathered, dst=0)
    if rank == 0:
        assert [int(g[0]) for g in gathered] == list(range(n))
    piece = torch.empty(2)
    dist.scatter(piece, [torch.full((2,), float(10 + r)) for r in range(n)] if rank == 0 else None,
                 src=0)
    assert torch.all(piece == 10 + rank)
    a2a_out = [torch.empty(1) for _ in range(n)]
    dist.all_to_all(a2a_out, [torch.tensor([float(rank * 10 + r)]) for r in range(n)])
    assert [int(o.item()) for o in a2a_out] == [r * 10 + rank for r in range(n)]
    single_in = torch.arange(n * 2, dtype=torch.float32) + 100 * rank
    single_out = torch.empty(n * 2)
    dist.all_to_all_single(single_out, single_in)
    assert single_out.tolist() == [100.0 * q + 2 * rank + j for q in range(n) for j in range(2)]
    dist.barrier()

    # a sub-group is a process group of its own (its members build their own session)
    if n >= 3:
        sub = dist.new_group([0, n - 1])
        if rank in (0, n - 1):
            v = torch.tensor([float(rank + 1)])
            dist.all_reduce(v, group=sub)
            assert v.item() == 1 + n
        dist.barrier()

    # DistributedDataParallel over the backend == one process on the joint batch
    model = make_model()
    ddp = torch.nn.parallel.DistributedDataParallel(model)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.1)
    x, y = data(rank)
    for _ in range(3):
        opt.zero_grad()
        torch.nn.functional.mse_loss(ddp(x), y).backward()
        opt.step()
    ref = make_model()
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    batches = [data(r) for r in range(n)]
    for _ in range(3):
        ropt.zero_grad()
        (sum(torch.nn.functional.mse_loss(ref(bx), by) for bx, by in batches) / n).backward()
        ropt.step()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, q, rtol=1e-5, atol=1e-6), float((p - q).abs().max())

    dist.destroy_process_group()
    print(f"rank {rank} OK", flush=True)


if __name__ == "__main__":
    main()
