"""One rank of the Python failure-detection test (spawned by test_python_api.py):
rank 1 leaves after joining; the others must get PeerFailure from their next
collective, without any timeout configured, and carry on as a smaller world
after Peer.recover()."""
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from stdml_collective_experimental_b200 import PeerFailure  # noqa: E402
from stdml_collective_experimental_b200.parallel import Peer  # noqa: E402


def main():
    rank, n, base = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    peers = [f"127.0.0.1:{base + i}" for i in range(n)]
    peer = Peer.from_list(rank, peers, strategy=sys.argv[4])
    sess = peer.join()
    # conn_ping: a member answers, a free port does not
    rtt = peer.ping(peers[(rank + 1) % n], timeout_ms=5000)
    assert rtt is not None and rtt > 0
    assert peer.ping(f"127.0.0.1:{base + 97}", timeout_ms=200) is None
    x = torch.ones(1000)
    sess.all_reduce(x, name="ok")
    assert x[0] == n
    if rank == 1:
        os._exit(0)  # gone between two steps
    t0 = time.time()
    try:
        sess.all_reduce(torch.ones(100_000), name="after")
    except PeerFailure as e:
        assert time.time() - t0 < 10, "detected too late"
        why = str(e)
    else:
        raise SystemExit("all_reduce succeeded without rank 1")
    # carry on without it
    assert peer.recover(sess) == 1
    assert (sess.size, sess.version) == (n - 1, 1) and sess.rank == (0 if rank == 0 else rank - 1)
    y = torch.ones(100_000)
    sess.all_reduce(y, name="after")
    assert y[0] == n - 1 and y[-1] == n - 1
    sess.barrier()
    print(f"rank {rank} OK: {why}", flush=True)


if __name__ == "__main__":
    main()
