"""One rank of the multi-GPU device tests (launched by torchrun from
test_device_multigpu.py, one process per GPU).  Every rank regenerates all
ranks' inputs from seeds, so the expected result needs no communication."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from stdml_collective_experimental_b200 import DeviceSession  # noqa: E402
from stdml_collective_experimental_b200.utils.oracle import reduce_many  # noqa: E402


def inputs(world, n, dtype, seed, exact=False):
    g = torch.Generator().manual_seed(seed)
    outs = []
    for _ in range(world):
        if dtype.is_floating_point:
            if exact:
                x = torch.randint(-8, 9, (n,), generator=g).float()
            else:
                x = torch.rand(n, generator=g) * 2 - 1
            outs.append(x.to(dtype))
        else:
            outs.append(torch.randint(-100, 101, (n,), generator=g).to(dtype))
    return outs


def bits_equal(a, b):
    return torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    sess = DeviceSession.from_env(heap_bytes=256 << 20, staging_bytes=4 << 20,
                                  wait_timeout_ms=20000)
    assert sess.rank == rank and sess.world == world
    info = f"backend={sess.backend} nvls={sess.has_nvls}"
    algos = ["oneshot", "twoshot", "twoshot_tma"] + (["nvls", "nvls_oneshot", "nvls_hybrid"] if sess.has_nvls else [])

    # ---- all_reduce: dtype x op x size, default algorithm choice (staged path)
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int32,
                  torch.int64, torch.uint8):
        for op in ("sum", "min", "max", "prod"):
            for n in (1, 7, 33, 4099, 300_001):
                host = inputs(world, n, dtype, seed=n, exact=True)
                if op == "prod":
                    host = [(h.abs() % 2 + 1).to(dtype) for h in host]
                want = reduce_many(host, op)
                x = host[rank].cuda()
                out = torch.empty_like(x)
                sess.all_reduce(x, out=out, op=op)
                torch.cuda.synchronize()
                sess.check()
                assert bits_equal(out.cpu(), want), (dtype, op, n)
                sess.all_reduce(x, op=op)
                torch.cuda.synchronize()
                assert bits_equal(x.cpu(), want), (dtype, op, n, "in place")

    # ---- every algorithm, random floats, with scale
    for algo in algos:
        for dtype in (torch.float32, torch.bfloat16):
            for n in (5, 1000, 2_000_003):
                host = inputs(world, n, dtype, seed=7 * n)
                scale = 1.0 / world
                want = reduce_many(host, "sum", scale)
                x = host[rank].cuda()
                sess.all_reduce(x, op="sum", scale=scale, algo=algo)
                torch.cuda.synchronize()
                sess.check()
                got = x.cpu()
                if algo.startswith("nvls"):
                    tol = 1e-5 if dtype == torch.float32 else 2e-2
                    assert torch.allclose(got.float(), want.float(), rtol=tol, atol=tol), (algo, n)
                else:
                    assert bits_equal(got, want), (algo, dtype, n)

    # ---- zero-copy symmetric buffers, every owner algorithm
    for algo in [a for a in algos if a in ("twoshot", "twoshot_tma", "nvls", "nvls_hybrid")]:
        n = 1_000_003
        host = inputs(world, n, torch.float32, seed=99, exact=True)
        want = reduce_many(host, "sum")
        sym = sess.symm_empty(n, torch.float32)
        sym.copy_(host[rank])
        before = sess.launches
        sess.all_reduce(sym, algo=algo)
        torch.cuda.synchronize()
        sess.check()
        assert sess.launches == before + 1
        assert bits_equal(sym.cpu(), want), algo
        sess.symm_free(sym)

    # ---- every inner loop of the NVLS reduce and several ring geometries of the
    # bulk-copy two-shot give the same values
    n = 3_000_017
    host = inputs(world, n, torch.float32, seed=5, exact=True)
    want = reduce_many(host, "sum")
    sym = sess.symm_empty(n, torch.float32)
    cases = [("twoshot_tma", "tma_tile_vec", v) for v in (32, 256, 512)]
    cases += [("twoshot_tma", "tma_blocks", v) for v in (1, 7, 148)]
    if sess.has_nvls:
        cases += [("nvls", "nvls_variant", v) for v in (0, 1, 2, 3)]
        cases += [("nvls", "nvls_blocks", v) for v in (16, 64)]
    for algo, knob, value in cases:
        sess.set_knob(knob, value)
        sym.copy_(host[rank])
        sess.all_reduce(sym, algo=algo)
        torch.cuda.synchronize()
        sess.check()
        assert bits_equal(sym.cpu(), want), (algo, knob, value)
    for knob, value in (("tma_tile_vec", 0), ("tma_blocks", 0), ("nvls_variant", 1), ("nvls_blocks", 0)):
        sess.set_knob(knob, value)
    sess.symm_free(sym)

    # ---- fused group, f32 and bf16-wire
    sizes = [1, 7, 768, 3, 2304, 590_000, 5, 64, 1000, 1_234_567, 2, 768]
    g = torch.Generator().manual_seed(1)
    host = [[torch.rand(n, generator=g) * 2 - 1 for n in sizes] for _ in range(world)]
    scale = 1.0 / world
    for algo in algos:
        dev = [t.cuda() for t in host[rank]]
        sess.group_all_reduce(dev, scale=scale, algo=algo)
        torch.cuda.synchronize()
        sess.check()
        for i in range(len(sizes)):
            want = reduce_many([host[r][i] for r in range(world)], "sum", scale)
            if algo.startswith("nvls"):
                assert torch.allclose(dev[i].cpu(), want, rtol=1e-5, atol=1e-6), (algo, i)
            else:
                assert bits_equal(dev[i].cpu(), want), (algo, i)
    dev = [t.cuda() for t in host[rank]]
    sess.group_all_reduce(dev, scale=scale, wire_dtype=torch.bfloat16, algo="twoshot")
    torch.cuda.synchronize()
    for i in range(len(sizes)):
        want = reduce_many([host[r][i].to(torch.bfloat16) for r in range(world)], "sum",
                           scale).float()
        assert torch.equal(dev[i].cpu(), want), i

    # ---- all_gather / broadcast / reduce / barrier
    for n in (1, 10, 37, 1_000_001):
        host = inputs(world, n, torch.int32, seed=n)
        out = torch.empty(n * world, dtype=torch.int32, device="cuda")
        sess.all_gather(host[rank].cuda(), out)
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), torch.cat(host))
        for root in sorted({0, world - 1}):
            b = host[rank].cuda()
            sess.broadcast(b, root=root)
            torch.cuda.synchronize()
            assert torch.equal(b.cpu(), host[root])
            r_out = torch.full((n,), -7, dtype=torch.int32, device="cuda")
            sess.reduce(host[rank].cuda(), out=r_out, root=root)
            torch.cuda.synchronize()
            if rank == root:
                assert torch.equal(r_out.cpu(), reduce_many(host, "sum"))
            else:
                assert torch.all(r_out == -7)
    for _ in range(10):
        sess.barrier()
    torch.cuda.synchronize()
    sess.check()

    # ---- registered execution: ordinary tensors, their allocations mapped on every
    # peer, no staging (the launch count tells: one launch whatever the size)
    sess.set_knob("register_min_bytes", 0)
    for dtype in (torch.float32, torch.bfloat16, torch.int32):
        for n in (1000, 3_000_004):
            host = inputs(world, n, dtype, seed=n + 9, exact=True)
            want = reduce_many(host, "sum")
            x = host[rank].cuda()
            before = sess.launches
            sess.all_reduce(x)  # in place
            torch.cuda.synchronize()
            sess.check()
            assert sess.launches == before + 1, "registered calls are one launch"
            assert bits_equal(x.cpu(), want), ("registered in place", dtype, n)
            x = host[rank].cuda()
            y = torch.empty_like(x)
            sess.all_reduce(x, out=y, scale=0.5 if dtype.is_floating_point else None)
            torch.cuda.synchronize()
            assert bits_equal(y.cpu(), reduce_many(host, "sum", 0.5 if dtype.is_floating_point else 1.0))
            assert bits_equal(x.cpu(), host[rank]), "out of place must not touch the input"
            for root in sorted({0, world - 1}):
                r_out = torch.full((n,), 3, dtype=dtype, device="cuda")
                sess.reduce(x, out=r_out, root=root)
                torch.cuda.synchronize()
                sess.check()
                assert bits_equal(x.cpu(), host[rank])
                if rank == root:
                    assert bits_equal(r_out.cpu(), want), ("registered reduce", dtype, n, root)
                else:
                    assert torch.all(r_out == 3)
                b = host[rank].cuda()
                sess.broadcast(b, root=root)
                torch.cuda.synchronize()
                assert bits_equal(b.cpu(), host[root]), ("registered broadcast", dtype, n, root)
            if (n * x.element_size()) % 16 == 0:
                g_out = torch.empty(n * world, dtype=dtype, device="cuda")
                before = sess.launches
                sess.all_gather(x, g_out)
                torch.cuda.synchronize()
                sess.check()
                assert sess.launches == before + 1
                assert bits_equal(g_out.cpu(), torch.cat(host)), ("registered all_gather", dtype, n)
    # a set of separately allocated tensors: one launch on the tensors themselves, the
    # table of peer pointers kept between calls and rebuilt when one rank's tensors move
    sizes = [3, 1000, 7, 250_001, 64, 1_000_003, 1]
    for dtype in (torch.float32, torch.bfloat16):
        host = [[inputs(1, n, dtype, seed=100 * r + i)[0] for i, n in enumerate(sizes)]
                for r in range(world)]
        want = [reduce_many([host[r][i] for r in range(world)], "sum", 0.5)
                for i in range(len(sizes))]
        keep = []
        for step in range(5):
            # (step 4: 16-byte peer loads instead of bulk copies into shared memory)
            sess.set_knob("group_bulk_min_bytes", -1 if step == 4 else 0)
            if step < 2 or rank == step % world:  # steps 2 and 3: one rank has new tensors
                dev = [t.cuda() for t in host[rank]]
                keep.append(dev)  # (earlier sets stay allocated: peers may still map them)
            else:
                for t, h in zip(dev, host[rank]):
                    t.copy_(h)
            before = sess.launches
            sess.group_all_reduce(dev, scale=0.5)
            torch.cuda.synchronize()
            sess.check()
            assert sess.launches == before + 1, "registered group: one launch"
            for i in range(len(sizes)):
                assert bits_equal(dev[i].cpu(), want[i]), ("registered group", dtype, step, i)
        outs = [torch.full((n + 8,), 3, dtype=dtype, device="cuda") for n in sizes]
        for t, h in zip(dev, host[rank]):
            t.copy_(h)
        sess.group_all_reduce(dev, outs=[o[:n] for o, n in zip(outs, sizes)], scale=0.5)
        torch.cuda.synchronize()
        sess.check()
        for i, n in enumerate(sizes):
            assert bits_equal(outs[i][:n].cpu(), want[i]) and torch.all(outs[i][n:] == 3)
            assert bits_equal(dev[i].cpu(), host[rank][i])
    sess.set_knob("group_bulk_min_bytes", 4 << 20)
    sess.drop_registrations()
    del keep
    sess.set_knob("register_min_bytes", -1)
    x = torch.ones(1000, device="cuda")
    sess.all_reduce(x)  # staged again
    torch.cuda.synchronize()
    assert torch.all(x == world)

    # ---- the same three on symmetric buffers (zero-copy: pushed straight into the
    # destinations, through the switch where there is one), and a message of
    # several staging slots (chunks unpacked on a second stream)
    for n in (4, 1000, 1_000_004):
        host = inputs(world, n, torch.int32, seed=n + 1)
        out = sess.symm_empty(n * world, torch.int32)
        out.fill_(-1)
        before = sess.launches
        sess.all_gather(host[rank].cuda(), out)
        torch.cuda.synchronize()
        sess.check()
        assert sess.launches == before + 1 and torch.equal(out.cpu(), torch.cat(host)), n
        for use_mc in (0, 1):
            sess.set_knob("gather_mc", use_mc)
            out.fill_(-1)
            sess.all_gather(host[rank].cuda(), out)
            torch.cuda.synchronize()
            assert torch.equal(out.cpu(), torch.cat(host)), (n, use_mc)
        sess.symm_free(out)
        sym = sess.symm_empty(n, torch.int32)
        for root in sorted({0, world - 1}):
            sym.copy_(host[rank])
            sess.broadcast(sym, root=root)
            torch.cuda.synchronize()
            assert torch.equal(sym.cpu(), host[root]), (n, root)
            sym.copy_(host[rank])
            r_out = torch.full((n,), -7, dtype=torch.int32, device="cuda")
            sess.reduce(sym, out=r_out, root=root)
            torch.cuda.synchronize()
            sess.check()
            assert torch.equal(sym.cpu(), host[rank])
            if rank == root:
                assert torch.equal(r_out.cpu(), reduce_many(host, "sum"))
            else:
                assert torch.all(r_out == -7)
        fsym = sess.symm_empty(n, torch.float32)
        fhost = inputs(world, n, torch.float32, seed=n, exact=True)
        fsym.copy_(fhost[rank])
        f_out = torch.zeros(n, device="cuda")
        sess.reduce(fsym, out=f_out, root=0, scale=0.5)  # f32 sum: the switch reduces for root
        torch.cuda.synchronize()
        if rank == 0:
            assert bits_equal(f_out.cpu(), reduce_many(fhost, "sum", 0.5))
        sess.symm_free(fsym)
        sess.symm_free(sym)
    # the broadcast in rounds (the default above 8 MB from three ranks up), forced at
    # every size here
    sess.set_knob("bcast_pipelined_min_bytes", 0)
    for n in (1, 5000, 3_000_001):
        host = inputs(world, n, torch.int32, seed=n + 5)
        for root in sorted({0, world - 1}):
            b = host[rank].cuda()
            sess.broadcast(b, root=root)
            sym = sess.symm_empty(n, torch.int32)
            sym.copy_(host[rank])
            sess.broadcast(sym, root=root)
            torch.cuda.synchronize()
            sess.check()
            assert torch.equal(b.cpu(), host[root]) and torch.equal(sym.cpu(), host[root]), (n, root)
            sess.symm_free(sym)
    sess.set_knob("bcast_pipelined_min_bytes", 8 << 20)
    n = 5_000_001  # 20 MB per rank through 4 MB slots
    host = inputs(world, n, torch.int32, seed=77)
    out = torch.empty(n * world, dtype=torch.int32, device="cuda")
    sess.all_gather(host[rank].cuda(), out)
    b = host[rank].cuda()
    sess.broadcast(b, root=world - 1)
    r_int = torch.full((n,), -3, dtype=torch.int32, device="cuda")
    sess.reduce(host[rank].cuda(), out=r_int, root=world - 1)   # several slots: three-stream pipeline
    fhost = inputs(world, n, torch.float32, seed=78, exact=True)
    r_f = torch.zeros(n, device="cuda")
    sess.reduce(fhost[rank].cuda(), out=r_f, root=0)
    fsym = sess.symm_empty(n, torch.float32)                     # symmetric input, several slots
    fsym.copy_(fhost[rank])
    r_s = torch.zeros(n, device="cuda")
    sess.reduce(fsym, out=r_s, root=0, scale=0.5)
    sess.all_reduce(out[:1000])  # a staged call right after the pipelines: the slots are free
    torch.cuda.synchronize()
    sess.check()
    if rank == world - 1:
        assert torch.equal(r_int.cpu(), reduce_many(host, "sum"))
    else:
        assert torch.all(r_int == -3)
    if rank == 0:
        assert bits_equal(r_f.cpu(), reduce_many(fhost, "sum"))
        assert bits_equal(r_s.cpu(), reduce_many(fhost, "sum", 0.5))
    assert bits_equal(fsym.cpu(), fhost[rank])
    sess.symm_free(fsym)
    assert torch.equal(out[1000:].cpu(), torch.cat(host)[1000:]) and torch.equal(b.cpu(), host[world - 1])
    assert torch.equal(out[:1000].cpu(), torch.cat(host)[:1000] * world)

    # ---- ranks that reach a collective at very different times (0 - 50 ms apart, a
    # different rank late every time): the device-side waits are bounded by seconds,
    # so lateness of this order must change nothing
    import random
    import time
    rnd = random.Random(1000 + rank)
    x = torch.empty(100_000, device="cuda")
    for it in range(12):
        time.sleep(rnd.random() * 0.05)
        x.fill_(float(rank + it))
        sess.all_reduce(x)
        g_in = torch.full((1000,), float(rank), device="cuda")
        g_out = torch.empty(1000 * world, device="cuda")
        sess.all_gather(g_in, g_out)
        torch.cuda.synchronize()
        sess.check()
        assert torch.all(x == world * (world - 1) / 2 + world * it), ("skew", it)
        assert g_out[::1000].tolist() == [float(r) for r in range(world)]

    # ---- the collectives as torch custom ops
    from stdml_collective_experimental_b200.ops import torch_ops
    torch_ops.set_default_session(sess)
    t = torch.full((1000,), float(rank + 1), device="cuda")
    torch.ops.stdml_collective.all_reduce_(t, "sum", 1.0 / world)
    g = torch.ops.stdml_collective.all_gather(torch.full((3,), float(rank), device="cuda"))
    torch.cuda.synchronize()
    assert torch.allclose(t, torch.full_like(t, (world + 1) / 2))
    assert g.tolist() == [float(r) for r in range(world) for _ in range(3)]

    # ---- CUDA graph: a zero-copy all_reduce and a staged one, captured once, replayed
    sym = sess.symm_empty(4096, torch.float32)
    user = torch.empty(4096, device="cuda")
    sess.all_reduce(sym)  # warm up outside the capture
    sess.all_reduce(user)
    sess.all_reduce(user)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    cap = torch.cuda.Stream()
    with torch.cuda.stream(cap):
        with torch.cuda.graph(graph, stream=cap):
            sess.all_reduce(sym, stream=cap)
            sess.all_reduce(user, stream=cap)
            sess.all_reduce(user, stream=cap)
    for it in range(3):
        sym.fill_(rank + it)
        user.fill_(1.0)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        sess.check()
        assert torch.all(sym == world * (world - 1) / 2 + world * it), "graph replay (zero-copy)"
        assert torch.all(user == float(world * world)), "graph replay (staged)"
    sess.symm_free(sym)

    # ---- point to point on NCCL's side stream, overlapping a collective
    import torch.distributed as dist
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world > 1:
        out = torch.full((1 << 20,), float(rank), device="cuda")
        inn = torch.empty(1 << 20, device="cuda")
        if rank % 2 == 0:
            hs = sess.send(out, (rank + 1) % world)
            hr = sess.recv(inn, (rank - 1) % world)
        else:
            hr = sess.recv(inn, (rank - 1) % world)
            hs = sess.send(out, (rank + 1) % world)
        busy = torch.ones(1 << 18, device="cuda")
        sess.all_reduce(busy)
        hs.wait()
        hr.wait()
        torch.cuda.synchronize()
        assert torch.all(inn == float((rank - 1) % world)) and torch.all(busy == world)
    dist.destroy_process_group()
    sess.close()
    print(f"OK rank {rank}/{world} {info}", flush=True)


if __name__ == "__main__":
    main()
