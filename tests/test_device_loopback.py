"""Device kernels on ONE GPU: all ranks are emulated as rows of one cooperative
launch (a loopback world), results are compared bit for bit with the native
host reducer (rank-ascending order, one rounding for 16-bit floats)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from stdml_collective_experimental_b200 import DeviceSession, DeviceTimeoutError  # noqa: E402
from stdml_collective_experimental_b200.ops.device import (ALGO_ONESHOT,  # noqa: E402
                                                           ALGO_TWOSHOT, ALGO_TWOSHOT_TMA)
from stdml_collective_experimental_b200.utils.oracle import reduce_many  # noqa: E402

FLOATS = [torch.float32, torch.float64, torch.bfloat16, torch.float16]
INTS = [torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8]


def make_inputs(world, n, dtype, seed, small=False):
    g = torch.Generator().manual_seed(seed)
    outs = []
    for r in range(world):
        if dtype.is_floating_point:
            x = torch.rand(n, generator=g) * 2 - 1
            if small:
                x = x * 0.5 + 1.0  # keeps products away from 0 and inf
            outs.append(x.to(dtype))
        else:
            info = torch.iinfo(dtype)
            lo, hi = max(info.min, -100), min(info.max, 100)
            outs.append(torch.randint(lo, hi + 1, (n,), generator=g).to(dtype))
    return outs


@pytest.fixture(scope="module", params=[1, 2, 4, 8])
def sess(request):
    s = DeviceSession.loopback(request.param, heap_bytes=32 << 20, staging_bytes=1 << 20)
    yield s
    s.close()


def same(a, b):
    if a.dtype.is_floating_point:
        return torch.equal(a.view(torch.uint8), b.view(torch.uint8)) or torch.equal(a, b)
    return torch.equal(a, b)


@pytest.mark.parametrize("dtype", FLOATS + INTS)
@pytest.mark.parametrize("op", ["sum", "min", "max", "prod", "bit_xor"])
def test_all_reduce_matrix(sess, dtype, op):
    if op == "bit_xor" and dtype.is_floating_point:
        with pytest.raises(ValueError):
            x = [torch.zeros(4, dtype=dtype, device="cuda") for _ in range(sess.world)]
            sess.all_reduce(x if sess.vranks > 1 else x[0], op=op)
        return
    for n in [1, 2, 3, 5, 7, 8, 9, 15, 16, 17, 31, 33, 100, 1024, 4099]:
        host = make_inputs(sess.world, n, dtype, seed=n, small=(op == "prod"))
        want = reduce_many(host, op)
        dev = [h.cuda() for h in host]
        out = [torch.empty_like(d) for d in dev]
        arg = (dev, out) if sess.vranks > 1 else (dev[0], out[0])
        sess.all_reduce(arg[0], out=arg[1], op=op)
        torch.cuda.synchronize()
        sess.check()
        for r in range(sess.world):
            assert same(out[r].cpu(), want), (dtype, op, n, r)
            assert same(dev[r].cpu(), host[r]), "input was modified"
        # in place
        sess.all_reduce(arg[0], op=op)
        torch.cuda.synchronize()
        for r in range(sess.world):
            assert same(dev[r].cpu(), want), (dtype, op, n, r, "in place")


@pytest.mark.parametrize("algo", ["oneshot", "twoshot"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_all_reduce_large_chunked_and_scaled(sess, algo, dtype):
    # 3 MiB+ of data through 1 MiB staging slots: several launches, alternating slots
    n = (3 << 20) // torch.empty((), dtype=dtype).element_size() + 13
    host = make_inputs(sess.world, n, dtype, seed=3)
    scale = 1.0 / sess.world
    want = reduce_many(host, "sum", scale)
    dev = [h.cuda() for h in host]
    arg = dev if sess.vranks > 1 else dev[0]
    sess.all_reduce(arg, op="sum", scale=scale, algo=algo)
    torch.cuda.synchronize()
    sess.check()
    for r in range(sess.world):
        assert same(dev[r].cpu(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
def test_symmetric_zero_copy_in_place(sess, dtype):
    n = 70001
    host = make_inputs(sess.world, n, dtype, seed=11)
    want = reduce_many(host, "sum")
    sym = sess.symm_empty(n, dtype)
    syms = sym if sess.vranks > 1 else [sym]
    for r in range(sess.world):
        syms[r].copy_(host[r])
    before = sess.launches
    sess.all_reduce(sym)
    torch.cuda.synchronize()
    sess.check()
    assert sess.launches == before + 1
    for r in range(sess.world):
        assert same(syms[r].cpu(), want)
    sess.symm_free(sym)


def test_raw_algorithms_agree(sess):
    n = 50000
    host = make_inputs(sess.world, n, torch.float32, seed=5)
    want = reduce_many(host, "sum", 0.5)
    sym = sess.symm_empty(n, torch.float32)
    syms = sym if sess.vranks > 1 else [sym]
    for blocks in (1, 3, 16):
        src = [h.cuda() for h in host]
        dst = [torch.empty(n, device="cuda") for _ in host]
        a = (src, dst) if sess.vranks > 1 else (src[0], dst[0])
        sess.raw_all_reduce(sym, src=a[0], dst=a[1], algo=ALGO_ONESHOT, blocks=blocks, scale=0.5)
        torch.cuda.synchronize()
        for r in range(sess.world):
            assert same(dst[r].cpu(), want), ("oneshot", blocks)
        dst2 = [torch.empty(n, device="cuda") for _ in host]
        a = (src, dst2) if sess.vranks > 1 else (src[0], dst2[0])
        sess.raw_all_reduce(sym, src=a[0], dst=a[1], algo=ALGO_TWOSHOT, blocks=blocks, scale=0.5)
        torch.cuda.synchronize()
        for r in range(sess.world):
            assert same(dst2[r].cpu(), want), ("twoshot", blocks)
            if sess.world > 1:  # a single GPU copies straight from src to dst
                assert same(syms[r].cpu(), want), ("twoshot leaves the result in the arena",
                                                   blocks)
    sess.check()
    sess.symm_free(sym)


@pytest.mark.parametrize("dtype,op", [(torch.float32, "sum"), (torch.bfloat16, "sum"),
                                      (torch.float64, "prod"), (torch.int32, "max"),
                                      (torch.uint8, "bit_xor"), (torch.float16, "min")])
def test_bulk_copy_two_shot_matches_the_oracle(sess, dtype, op):
    """The two-shot whose owner pulls tiles with bulk async copies into a shared
    memory ring: every dtype path, grids of 1..16 CTAs per rank, tiles small enough
    that each ring slot is reused many times (both mbarrier parities), ragged
    sizes (partial last tile, partial last vector)."""
    if sess.world == 1:
        pytest.skip("a world of one has no peers to pull from")
    for tile_vec, n, blocks in [(0, 1, 1), (0, 33, 3), (64, 4099, 1), (32, 70_001, 2),
                                (128, 1_000_003, 1), (0, 1_000_003, 16), (64, 262_144, 16)]:
        sess.set_knob("tma_tile_vec", tile_vec)
        host = make_inputs(sess.world, n, dtype, seed=n + blocks, small=(op == "prod"))
        scale = 0.5 if dtype.is_floating_point else None
        want = reduce_many(host, op, 1.0 if scale is None else scale)
        sym = sess.symm_empty(n, dtype)
        src = [h.cuda() for h in host]
        dst = [torch.empty_like(x) for x in src]
        sess.raw_all_reduce(sym, src=src, dst=dst, op=op, algo=ALGO_TWOSHOT_TMA, blocks=blocks,
                            scale=scale)
        torch.cuda.synchronize()
        sess.check()
        for r in range(sess.world):
            assert same(dst[r].cpu(), want), (dtype, op, n, blocks, tile_vec, r)
            assert same(sym[r][:n].cpu(), want), "the result also stays in the symmetric buffer"
        sess.symm_free(sym)
    sess.set_knob("tma_tile_vec", 0)


def test_bulk_copy_two_shot_through_the_public_calls(sess):
    """Staged (several 1 MiB slots, pack and unpack fused) and zero-copy in place."""
    n = (3 << 20) // 4 + 13
    host = make_inputs(sess.world, n, torch.float32, seed=21)
    want = reduce_many(host, "sum", 1.0 / sess.world)
    dev = [h.cuda() for h in host]
    sess.all_reduce(dev if sess.vranks > 1 else dev[0], scale=1.0 / sess.world, algo="twoshot_tma")
    sym = sess.symm_empty(n, torch.float32)
    syms = sym if sess.vranks > 1 else [sym]
    for r in range(sess.world):
        syms[r].copy_(host[r])
    sess.all_reduce(sym, scale=1.0 / sess.world, algo="twoshot_tma")
    torch.cuda.synchronize()
    sess.check()
    for r in range(sess.world):
        assert same(dev[r].cpu(), want) and same(syms[r].cpu(), want)
    sess.symm_free(sym)


def test_f64_scale_keeps_all_its_bits(sess):
    """1/3 is not a float: f64 buffers must be scaled in double, like the host reducer."""
    n = 10_007
    host = make_inputs(sess.world, n, torch.float64, seed=9)
    want = reduce_many(host, "sum", 1.0 / 3.0)
    assert torch.allclose(want, torch.stack(host).sum(0) / 3.0, rtol=1e-15, atol=0)
    for algo in ("oneshot", "twoshot", "twoshot_tma"):
        if sess.world == 1 and algo == "twoshot_tma":
            continue
        dev = [h.cuda() for h in host]
        sess.all_reduce(dev if sess.vranks > 1 else dev[0], scale=1.0 / 3.0, algo=algo)
        torch.cuda.synchronize()
        sess.check()
        for r in range(sess.world):
            assert same(dev[r].cpu(), want), algo


def test_kernel_refuses_arguments_that_fail_its_own_checks():
    """With debug checks on, a kernel handed a misaligned offset (or one inside the
    signal pad) reports kStatusBadArgs and touches nothing; recover() clears it."""
    with DeviceSession.loopback(2, heap_bytes=8 << 20, staging_bytes=1 << 20) as s:
        for inject, algo in [(1, ALGO_TWOSHOT), (2, ALGO_TWOSHOT_TMA), (1, ALGO_ONESHOT)]:
            sym = s.symm_empty(4096, torch.float32)
            src = [torch.ones(4096, device="cuda") for _ in range(2)]
            dst = [torch.full((4096,), -7.0, device="cuda") for _ in range(2)]
            for t in sym:
                t.fill_(3.0)
            s.set_knob("debug_inject", inject)
            s.raw_all_reduce(sym, src=src, dst=dst, algo=algo, blocks=2)
            torch.cuda.synchronize()
            assert s.status()[0] == 2  # kStatusBadArgs
            with pytest.raises(ValueError):
                s.check()
            assert all(bool((d == -7.0).all()) for d in dst) and all(bool((t == 3.0).all()) for t in sym)
            s.recover()
            assert s.status()[0] == 0
            # and the same call runs normally afterwards, with the checks on
            s.set_knob("debug_checks", 1)
            s.raw_all_reduce(sym, src=src, dst=dst, algo=algo, blocks=2)
            torch.cuda.synchronize()
            s.check()
            assert bool((dst[0] == 2.0).all()) and bool((dst[1] == 2.0).all())
            s.set_knob("debug_checks", 0)
            s.symm_free(sym)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_group_all_reduce_fused(sess, dtype):
    sizes = [1, 7, 768, 3, 2304, 590_000, 5, 64, 1000, 123_457, 2, 768]
    g = torch.Generator().manual_seed(1)
    host = [[(torch.rand(n, generator=g) * 2 - 1).to(dtype) for n in sizes]
            for _ in range(sess.world)]
    scale = 1.0 / sess.world
    want = [reduce_many([host[r][i] for r in range(sess.world)], "sum", scale)
            for i in range(len(sizes))]
    dev = [[t.cuda() for t in host[r]] for r in range(sess.world)]
    before = sess.launches
    sess.group_all_reduce(dev if sess.vranks > 1 else dev[0], scale=scale)
    torch.cuda.synchronize()
    sess.check()
    launches = sess.launches - before
    total_bytes = sum((n * host[0][0].element_size() + 15) // 16 * 16 for n in sizes)
    assert launches == -(-total_bytes // sess.staging_bytes), "one launch per staging slot"
    for r in range(sess.world):
        for i in range(len(sizes)):
            assert same(dev[r][i].cpu(), want[i]), (r, i)
    # second call hits the cached descriptor table
    sess.group_all_reduce(dev if sess.vranks > 1 else dev[0])
    torch.cuda.synchronize()
    sess.check()


@pytest.mark.parametrize("bulk", [False, True])
@pytest.mark.parametrize("dtype,op,scale", [
    (torch.float32, "sum", 0.125), (torch.bfloat16, "sum", None), (torch.int32, "max", None),
    (torch.float64, "prod", 1.0 / 3.0), (torch.int8, "bit_xor", None), (torch.float16, "min", None),
])
def test_group_all_reduce_on_registered_loose_tensors(sess, dtype, op, scale, bulk):
    """Separately allocated tensors, reduced where they lie: one launch, no staging.
    `bulk`: operands come in by bulk asynchronous copies into a shared-memory ring
    (the default from 4 MB up), else by 16-byte peer loads."""
    if sess.world == 1:
        pytest.skip("needs peers")
    sess.set_knob("group_bulk_min_bytes", 0 if bulk else -1)
    sizes = [1, 7, 768, 3, 2304, 590_000, 5, 64, 1000, 123_457, 2, 768]
    host = [[make_inputs(1, n, dtype, seed=31 * r + i, small=op == "prod")[0]
             for i, n in enumerate(sizes)] for r in range(sess.world)]
    want = [reduce_many([host[r][i] for r in range(sess.world)], op, scale)
            for i in range(len(sizes))]
    sess.set_knob("register_min_bytes", 0)
    try:
        # in place, twice (the second call reuses the table of peer pointers)
        for _ in range(2):
            dev = [[t.cuda() for t in host[r]] for r in range(sess.world)]
            before = sess.launches
            sess.group_all_reduce(dev if sess.vranks > 1 else dev[0], op=op, scale=scale)
            torch.cuda.synchronize()
            sess.check()
            assert sess.launches == before + 1
            for r in range(sess.world):
                for i in range(len(sizes)):
                    assert same(dev[r][i].cpu(), want[i]), (r, i)
        # out of place: inputs stay, outputs carry the result and nothing beyond their end
        dev = [[t.cuda() for t in host[r]] for r in range(sess.world)]
        pad = 16
        outs = [[torch.full((n + pad,), 3, dtype=dtype, device="cuda") for n in sizes]
                for _ in range(sess.world)]
        views = [[o[:n] for o, n in zip(outs[r], sizes)] for r in range(sess.world)]
        before = sess.launches
        sess.group_all_reduce(dev if sess.vranks > 1 else dev[0],
                              outs=views if sess.vranks > 1 else views[0], op=op, scale=scale)
        torch.cuda.synchronize()
        sess.check()
        assert sess.launches == before + 1
        for r in range(sess.world):
            for i, n in enumerate(sizes):
                assert same(views[r][i].cpu(), want[i]), (r, i)
                assert bool((outs[r][i][n:] == 3).all()), "wrote past the end of a tensor"
                assert torch.equal(dev[r][i].cpu(), host[r][i]), "inputs must stay untouched"
        # a tensor that does not start on a 16-byte boundary sends the set the staged way
        dev = [[t.cuda() for t in host[r]] for r in range(sess.world)]
        for r in range(sess.world):
            odd = torch.empty(sizes[5] + 1, dtype=dtype, device="cuda")[1:]
            if odd.data_ptr() % 16 != 0:
                odd.copy_(host[r][5])
                dev[r][5] = odd
        before = sess.launches
        sess.group_all_reduce(dev if sess.vranks > 1 else dev[0], op=op, scale=scale)
        torch.cuda.synchronize()
        sess.check()
        assert sess.launches > before
        for r in range(sess.world):
            for i in range(len(sizes)):
                assert same(dev[r][i].cpu(), want[i]), (r, i)
    finally:
        sess.set_knob("register_min_bytes", -1)
        sess.set_knob("group_bulk_min_bytes", 4 << 20)


def test_group_all_reduce_bf16_wire_for_f32_grads(sess):
    sizes = [5, 4096, 33, 100_000]
    g = torch.Generator().manual_seed(2)
    host = [[torch.rand(n, generator=g) * 2 - 1 for n in sizes] for _ in range(sess.world)]
    scale = 1.0 / sess.world
    dev = [[t.cuda() for t in host[r]] for r in range(sess.world)]
    sess.group_all_reduce(dev if sess.vranks > 1 else dev[0], scale=scale,
                          wire_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    sess.check()
    for i in range(len(sizes)):
        want = reduce_many([host[r][i].to(torch.bfloat16) for r in range(sess.world)], "sum",
                           scale).float()
        for r in range(sess.world):
            assert torch.equal(dev[r][i].cpu(), want), (r, i)


def test_group_zero_copy_flat(sess):
    sizes = [8, 100, 4, 50_000]  # every tensor a multiple of 16 bytes: back to back
    flat = sess.symm_empty(sum(sizes), torch.float32)
    flats = flat if sess.vranks > 1 else [flat]
    g = torch.Generator().manual_seed(7)
    host = [torch.rand(sum(sizes), generator=g) for _ in range(sess.world)]
    for r in range(sess.world):
        flats[r].copy_(host[r])
    views = [list(torch.split(f, sizes)) for f in flats]
    before = sess.launches
    sess.group_all_reduce(views if sess.vranks > 1 else views[0], scale=0.25)
    torch.cuda.synchronize()
    sess.check()
    assert sess.launches == before + 1
    want = reduce_many(host, "sum", 0.25)
    for r in range(sess.world):
        assert same(flats[r].cpu(), want)
    sess.symm_free(flat)


@pytest.mark.parametrize("n", [1, 2, 10, 1000, 300_001])
def test_all_gather(sess, n):
    host = make_inputs(sess.world, n, torch.int32, seed=n)
    dev = [h.cuda() for h in host]
    out = [torch.empty(n * sess.world, dtype=torch.int32, device="cuda") for _ in dev]
    a = (dev, out) if sess.vranks > 1 else (dev[0], out[0])
    sess.all_gather(a[0], a[1])
    torch.cuda.synchronize()
    sess.check()
    want = torch.cat(host)
    for r in range(sess.world):
        assert torch.equal(out[r].cpu(), want)


def test_all_gather_odd_bytes(sess):
    n = 37  # 37 bytes per rank: unaligned destinations
    host = make_inputs(sess.world, n, torch.uint8, seed=9)
    dev = [h.cuda() for h in host]
    out = [torch.empty(n * sess.world, dtype=torch.uint8, device="cuda") for _ in dev]
    a = (dev, out) if sess.vranks > 1 else (dev[0], out[0])
    sess.all_gather(a[0], a[1])
    torch.cuda.synchronize()
    want = torch.cat(host)
    for r in range(sess.world):
        assert torch.equal(out[r].cpu(), want)


@pytest.mark.parametrize("n", [1, 17, 300_001])
def test_broadcast_and_reduce(sess, n):
    host = make_inputs(sess.world, n, torch.float32, seed=n)
    for root in sorted({0, sess.world - 1}):
        dev = [h.cuda() for h in host]
        out = [torch.empty_like(d) for d in dev]
        a = (dev, out) if sess.vranks > 1 else (dev[0], out[0])
        sess.broadcast(a[0], out=a[1], root=root)
        torch.cuda.synchronize()
        for r in range(sess.world):
            assert torch.equal(out[r].cpu(), host[root])
        red = [torch.full_like(d, -7.0) for d in dev]
        a = (dev, red) if sess.vranks > 1 else (dev[0], red[0])
        sess.reduce(a[0], out=a[1], op="sum", root=root)
        torch.cuda.synchronize()
        want = reduce_many(host, "sum")
        for r in range(sess.world):
            if r == root:
                assert same(red[r].cpu(), want)
            else:
                assert torch.all(red[r] == -7.0)
    sess.check()


@pytest.mark.parametrize("n", [4, 1000, 300_004])
def test_zero_copy_all_gather_broadcast_reduce_on_symmetric_buffers(sess, n):
    """Output (all_gather, broadcast) or input (reduce) in the symmetric heap: one
    launch, no staging; blocks are pushed straight into every rank's buffer."""
    w = sess.world
    host = make_inputs(w, n, torch.int32, seed=n + 3)
    out = sess.symm_empty(n * w, torch.int32)
    outs = out if sess.vranks > 1 else [out]
    for o in outs:
        o.fill_(-1)
    ins = [h.cuda() for h in host]
    before = sess.launches
    sess.all_gather(ins if sess.vranks > 1 else ins[0], out)
    torch.cuda.synchronize()
    sess.check()
    assert sess.launches == before + 1 or w == 1  # alone: a plain copy through the slots
    for r in range(w):
        assert torch.equal(outs[r].cpu(), torch.cat(host)), r
    # in place: every rank's block already sits in its own output
    for r in range(w):
        outs[r].fill_(-1)
        outs[r][r * n:(r + 1) * n].copy_(host[r])
    views = [outs[r][r * n:(r + 1) * n] for r in range(w)]
    sess.all_gather(views if sess.vranks > 1 else views[0], out)
    torch.cuda.synchronize()
    for r in range(w):
        assert torch.equal(outs[r].cpu(), torch.cat(host)), (r, "in place")
    sess.symm_free(out)

    for root in sorted({0, w - 1}):
        sym = sess.symm_empty(n, torch.int32)
        syms = sym if sess.vranks > 1 else [sym]
        for r in range(w):
            syms[r].copy_(host[r])
        sess.broadcast(sym, root=root)  # in place on a symmetric buffer
        torch.cuda.synchronize()
        sess.check()
        for r in range(w):
            assert torch.equal(syms[r].cpu(), host[root]), (root, r)
        # from an ordinary tensor on root into symmetric buffers everywhere
        for t in syms:
            t.fill_(-5)
        sess.broadcast(ins if sess.vranks > 1 else ins[0], out=sym, root=root)
        torch.cuda.synchronize()
        for r in range(w):
            assert torch.equal(syms[r].cpu(), host[root]), (root, r, "out of place")
        # reduce: symmetric inputs, ordinary output on root only
        for r in range(w):
            syms[r].copy_(host[r])
        res = [torch.full((n,), -7, dtype=torch.int32, device="cuda") for _ in range(w)]
        sess.reduce(sym, out=res if sess.vranks > 1 else res[0], root=root)
        torch.cuda.synchronize()
        sess.check()
        for r in range(w):
            if r == root:
                assert torch.equal(res[r].cpu(), reduce_many(host, "sum"))
            else:
                assert bool((res[r] == -7).all())
            assert torch.equal(syms[r].cpu(), host[r]), "reduce must leave its inputs alone"
        sess.symm_free(sym)


def test_broadcast_in_rounds(sess):
    """The pipelined broadcast (root sends in rounds and signals, holders forward
    while root goes on) at sizes from one vector to many rounds, staged and on
    symmetric buffers, from both ends of the rank range."""
    if sess.world < 3:
        pytest.skip("used from three ranks up")
    sess.set_knob("bcast_pipelined_min_bytes", 0)
    try:
        for n in (1, 17, 5000, 300_001, 2_000_003):
            host = make_inputs(sess.world, n, torch.float32, seed=n + 1)
            for root in sorted({0, sess.world - 1}):
                dev = [h.cuda() for h in host]
                sess.broadcast(dev, root=root)
                if n * 4 <= (4 << 20):
                    sym = sess.symm_empty(n, torch.float32)
                    for r in range(sess.world):
                        sym[r].copy_(host[r])
                    sess.broadcast(sym, root=root)
                torch.cuda.synchronize()
                sess.check()
                for r in range(sess.world):
                    assert torch.equal(dev[r].cpu(), host[root]), (n, root, r)
                    if n * 4 <= (4 << 20):
                        assert torch.equal(sym[r].cpu(), host[root]), (n, root, r, "symmetric")
                if n * 4 <= (4 << 20):
                    sess.symm_free(sym)
    finally:
        sess.set_knob("bcast_pipelined_min_bytes", 8 << 20)


@pytest.mark.parametrize("algo_knob", [0, 1 << 40])
def test_all_gather_push_and_pull_agree(sess, algo_knob):
    sess.set_knob("gather_push_min_bytes", algo_knob)  # 0: always push; huge: always pull
    try:
        for n in (3, 1000, 70_001):
            host = make_inputs(sess.world, n, torch.int16, seed=n)
            outs = [torch.empty(n * sess.world, dtype=torch.int16, device="cuda")
                    for _ in range(sess.world)]
            ins = [h.cuda() for h in host]
            sess.all_gather(ins if sess.vranks > 1 else ins[0],
                            outs if sess.vranks > 1 else outs[0])
            torch.cuda.synchronize()
            sess.check()
            for r in range(sess.world):
                assert torch.equal(outs[r].cpu(), torch.cat(host)), (n, r)
    finally:
        sess.set_knob("gather_push_min_bytes", 64 << 10)


def test_kernels_against_plain_pytorch_arithmetic(sess):
    """An oracle that shares nothing with the library: the same reductions done by
    PyTorch in float32 / float64 on the host.  all_reduce (every algorithm), the
    fused group with the 1/world scale, and the bf16 wire format for f32 tensors."""
    w = sess.world
    g = torch.Generator().manual_seed(42)
    n = 100_003
    host = [torch.rand(n, generator=g) * 2 - 1 for _ in range(w)]
    exact = torch.stack([h.double() for h in host]).sum(0)
    f32 = host[0].clone()
    for h in host[1:]:
        f32 += h  # rank-ascending float32 adds: what the peer-load kernels do
    for algo in ("oneshot", "twoshot") + (("twoshot_tma",) if w > 1 else ()):
        dev = [h.cuda() for h in host]
        sess.all_reduce(dev if sess.vranks > 1 else dev[0], algo=algo)
        torch.cuda.synchronize()
        sess.check()
        for r in range(w):
            assert torch.equal(dev[r].cpu(), f32), algo
            assert torch.allclose(dev[r].cpu().double(), exact, rtol=0, atol=w * 2.0 ** -23)
    sizes = [3, 1000, 70_001, 17]
    hosts = [[torch.rand(m, generator=g) * 2 - 1 for m in sizes] for _ in range(w)]
    dev = [[t.cuda() for t in hosts[r]] for r in range(w)]
    sess.group_all_reduce(dev if sess.vranks > 1 else dev[0], scale=1.0 / w)
    dev16 = [[t.cuda() for t in hosts[r]] for r in range(w)]
    sess.group_all_reduce(dev16 if sess.vranks > 1 else dev16[0], scale=1.0 / w,
                          wire_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    sess.check()
    for i in range(len(sizes)):
        mean = torch.stack([hosts[r][i].double() for r in range(w)]).mean(0)
        for r in range(w):
            assert torch.allclose(dev[r][i].cpu().double(), mean, rtol=0, atol=2.0 ** -22)
            # bf16 wire: every operand rounded to 8 bits of mantissa, then the mean rounded
            assert torch.allclose(dev16[r][i].cpu().double(), mean, rtol=0, atol=3 * 2.0 ** -8)


def test_barrier_and_launch_count(sess):
    before = sess.launches
    for _ in range(5):
        sess.barrier()
    torch.cuda.synchronize()
    sess.check()
    assert sess.launches == before + 5


def test_bounded_wait_reports_and_recovers():
    """A rank that never arrives: the wait runs out, the host reads a status, the
    context stays usable, and after recover() collectives work again."""
    s = DeviceSession.loopback(2, heap_bytes=1 << 20, staging_bytes=1 << 20, wait_timeout_ms=200)
    try:
        s.barrier_rows(1)  # rank 1 is not launched: nothing sets its flag
        torch.cuda.synchronize()
        code, rank, block, peer, phase, want, have = s.status()
        assert code == 1 and rank == 0 and peer == 1 and want == have + 1
        with pytest.raises(DeviceTimeoutError):
            s.all_reduce([torch.ones(4, device="cuda"), torch.ones(4, device="cuda")])
        s.recover()
        assert s.status()[0] == 0
        x = [torch.full((9,), 1.0, device="cuda"), torch.full((9,), 2.0, device="cuda")]
        s.all_reduce(x)
        torch.cuda.synchronize()
        s.check()
        assert torch.all(x[0] == 3.0) and torch.all(x[1] == 3.0)
    finally:
        s.close()


def test_profile_summary_counts_device_time(sess):
    sess.enable_profile()
    x = [torch.ones(100_000, device="cuda") for _ in range(sess.world)]
    arg = x if sess.vranks > 1 else x[0]
    for _ in range(3):
        sess.all_reduce(arg)
    out = [torch.empty(100_000 * sess.world, device="cuda") for _ in range(sess.world)]
    sess.all_gather(arg, out if sess.vranks > 1 else out[0])
    summary = sess.profile_summary()
    sess.enable_profile(False)
    assert summary["all_reduce"]["calls"] == 3 and summary["all_reduce"]["bytes"] == 3 * 400_000
    assert summary["all_reduce"]["ms"] > 0 and summary["all_gather"]["calls"] == 1
    assert sess.profile_summary() == {}


def test_cuda_graph_capture_and_replay():
    """Collectives are plain kernel launches with device-side epochs: a captured
    graph replays them (world 1: no cooperative launch inside the capture)."""
    with DeviceSession.loopback(1, heap_bytes=1 << 20, staging_bytes=1 << 20) as s:
        sym = s.symm_empty(1000, torch.float32)
        user = torch.empty(1000, device="cuda")
        s.all_reduce(sym, scale=0.5)
        s.all_reduce(user, scale=2.0)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        cap = torch.cuda.Stream()
        with torch.cuda.stream(cap):
            with torch.cuda.graph(g, stream=cap):
                s.all_reduce(sym, scale=0.5, stream=cap)
                s.all_reduce(user, scale=2.0, stream=cap)
        for it in range(3):
            sym.fill_(4.0 + it)
            user.fill_(1.0 + it)
            torch.cuda.synchronize()
            g.replay()
            torch.cuda.synchronize()
            s.check()
            assert torch.all(sym == (4.0 + it) / 2) and torch.all(user == 2.0 * (1.0 + it))


@pytest.mark.parametrize("world", [2, 4])
def test_large_staged_messages_are_pipelined_on_three_streams(world, monkeypatch):
    """Above a size threshold staged calls run pack / reduce / unpack of successive
    chunks on three streams; the result must not change."""
    monkeypatch.setenv("STDML_COLLECTIVE_PIPELINE_MIN_BYTES", str(1 << 20))
    with DeviceSession.loopback(world, heap_bytes=1 << 20, staging_bytes=1 << 20) as s:
        n = (5 << 20) // 4 + 13
        host = make_inputs(world, n, torch.float32, seed=21)
        want = reduce_many(host, "sum", 0.5)
        dev = [h.cuda() for h in host]
        out = [torch.empty_like(d) for d in dev]
        before = s.launches
        s.all_reduce(dev, out=out, scale=0.5)
        torch.cuda.synchronize()
        s.check()
        assert s.launches - before == 3 * 6 + 1, \
                "6 slot-sized chunks, three launches each, and the barrier that ends a pipeline"
        for r in range(world):
            assert same(out[r].cpu(), want) and same(dev[r].cpu(), host[r])
        # a fused group above the threshold takes the same route
        sizes = [300_000, 7, 500_000, 64, 400_000]
        g = torch.Generator().manual_seed(3)
        hosts = [[torch.rand(k, generator=g) for k in sizes] for _ in range(world)]
        devs = [[t.cuda() for t in hosts[r]] for r in range(world)]
        s.group_all_reduce(devs, scale=1.0 / world)
        s.all_reduce(dev)  # ordinary call right behind the pipeline
        torch.cuda.synchronize()
        s.check()
        for i in range(len(sizes)):
            w = reduce_many([hosts[r][i] for r in range(world)], "sum", 1.0 / world)
            for r in range(world):
                assert same(devs[r][i].cpu(), w), (r, i)
        assert same(dev[0].cpu(), reduce_many(host, "sum"))


def test_group_with_mixed_dtypes_splits_per_dtype(sess):
    g = torch.Generator().manual_seed(4)
    kinds = [torch.float32, torch.bfloat16, torch.float32, torch.int32, torch.bfloat16]
    sizes = [100, 33, 7, 64, 4096]
    host = [[(torch.rand(n, generator=g) * 8).to(dt) for n, dt in zip(sizes, kinds)]
            for _ in range(sess.world)]
    dev = [[t.cuda() for t in host[r]] for r in range(sess.world)]
    sess.group_all_reduce(dev if sess.vranks > 1 else dev[0])
    torch.cuda.synchronize()
    sess.check()
    for i in range(len(sizes)):
        want = reduce_many([host[r][i] for r in range(sess.world)], "sum")
        for r in range(sess.world):
            assert same(dev[r][i].cpu(), want), (r, i)


def test_session_async_interface_on_cuda_tensors():
    """Peer/Session (the C++ session) with device pointers: a single-rank world,
    the returned task polls a CUDA event."""
    from stdml_collective_experimental_b200.parallel import Peer
    peer = Peer.from_list(0, ["127.0.0.1:10990"])
    sess = peer.join()
    x = torch.arange(100_000, dtype=torch.float32, device="cuda")
    y = torch.empty_like(x)
    task = sess.all_reduce_async(x, out=y, name="dev")
    task.wait()
    assert torch.equal(x, y)
    sess.all_reduce(x, op="max")
    gathered = torch.empty(100_000, device="cuda")
    sess.all_gather(x, gathered)
    torch.cuda.synchronize()
    assert torch.equal(gathered, x)
    sess.close()
    peer.close()
