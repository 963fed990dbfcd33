"""One rank of the Python host-API test (spawned by test_python_api.py)."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from stdml_collective_experimental_b200.parallel import Peer, resized_cluster  # noqa: E402


def main():
    rank, n, base = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    strategy = sys.argv[4]
    peers = [f"127.0.0.1:{base + i}" for i in range(n)]
    peer = Peer.from_list(rank, peers, strategy=strategy)
    sess = peer.join()
    assert (sess.rank, sess.size, sess.version, sess.strategy) == (rank, n, 0, strategy)

    x = torch.arange(1000, dtype=torch.float32) + rank
    y = torch.empty_like(x)
    sess.all_reduce(x, out=y, name="x")
    assert torch.equal(y, torch.arange(1000, dtype=torch.float32) * n + n * (n - 1) / 2)
    h = torch.full((33,), rank + 0.5, dtype=torch.bfloat16)
    sess.all_reduce(h, op="max")
    assert torch.all(h == n - 0.5)

    grads = [torch.full((k,), float(rank + i)) for i, k in enumerate([3, 70000, 1, 512])]
    sess.group_all_reduce(grads, scale=1.0 / n, names=[f"g{i}" for i in range(4)])
    for i, g in enumerate(grads):
        assert torch.allclose(g, torch.full_like(g, (n - 1) / 2 + i))

    out = torch.empty(n * 5, dtype=torch.int64)
    sess.all_gather(torch.full((5,), rank, dtype=torch.int64), out)
    assert out.tolist() == [r for r in range(n) for _ in range(5)]
    b = torch.full((7,), float(rank))
    sess.broadcast(b)
    assert torch.all(b == 0)
    r = torch.full((4,), float(rank))
    ro = torch.full((4,), -1.0)
    sess.reduce(r, out=ro)
    assert torch.all(ro == (n * (n - 1) / 2 if rank == 0 else -1))
    # any root: reduce and gather to the last rank
    rl = torch.full((4,), -1.0)
    sess.reduce(r, out=rl, root=n - 1, name="to-last")
    assert torch.all(rl == (n * (n - 1) / 2 if rank == n - 1 else -1))
    gl = torch.full((n * 2,), -1.0)
    sess.gather(torch.full((2,), float(rank)), gl, root=n - 1, name="g-last")
    if rank == n - 1:
        assert gl.tolist() == [float(q) for q in range(n) for _ in range(2)]
    assert sess.consistent(b) and (n == 1 or not sess.consistent(torch.tensor([rank])))
    if n > 1:
        if rank == 0:
            sess.send(torch.tensor([42.0]), 1, name="p2p")
        elif rank == 1:
            assert sess.recv(torch.zeros(1), 0, name="p2p").item() == 42.0
    # reduce_scatter / all_to_all
    rs = torch.empty(3)
    sess.reduce_scatter(torch.arange(3 * n, dtype=torch.float32) + rank, rs, name="rs")
    assert torch.equal(rs, (torch.arange(3 * n, dtype=torch.float32) * n + n * (n - 1) / 2)[3 * rank:3 * rank + 3])
    a2 = torch.empty(n, dtype=torch.int64)
    sess.all_to_all(torch.arange(n, dtype=torch.int64) + 10 * rank, a2, name="a2a")
    assert a2.tolist() == [10 * q + rank for q in range(n)]
    # sub-group: all but the last rank
    if n > 2:
        sub = sess.subgroup(list(range(n - 1)), "head")
        if rank < n - 1:
            v = torch.tensor([float(rank)])
            sub.all_reduce(v, name="sub")
            assert (sub.size, sub.rank) == (n - 1, rank) and v.item() == (n - 1) * (n - 2) / 2
            sub.close()
        else:
            assert sub is None
    # async interface: two operations in flight, polled from this thread
    a, b = torch.full((300_000,), float(rank)), torch.ones(10)
    ta = sess.all_reduce_async(a, name="async:a")
    tb = sess.all_reduce_async(b, op="max", name="async:b")
    while not (ta.poll() and tb.poll()):
        pass
    assert a[0] == n * (n - 1) / 2 and a[-1] == a[0] and b[0] == 1
    sess.barrier()

    # elastic: shrink to n - 1 by explicit configuration; the last rank detaches
    if n > 2:
        # an operation that is still unfinished when the session is replaced: resize
        # must finish and free it first (its native task polls the old session), and
        # dropping the handle afterwards must touch nothing that is gone
        pending_in = torch.full((400_000,), float(rank + 1))
        pending = sess.all_reduce_async(pending_in, name="async:across-resize")
        smaller = resized_cluster(sess.cluster, n - 1)
        changed, detached = peer.resize(sess, cluster=smaller)
        assert changed
        assert pending._h is None and pending_in[0] == n * (n + 1) / 2
        del pending
        if rank == n - 1:
            assert detached
        else:
            assert not detached and sess.size == n - 1 and sess.version == 1
            assert sess.all_reduce(torch.ones(3))[0] == n - 1
    sess.close()
    peer.close()
    print(f"rank {rank} OK", flush=True)


if __name__ == "__main__":
    main()
