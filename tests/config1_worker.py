"""One rank of the acceptance case "CPU plumbing": 4 processes on TCP loopback,
ring strategy, the 161 f32 tensors of a ResNet-50 gradient set (25.56 M floats),
values N(0, 1) seeded per rank, all-reduced with sum.  Every rank regenerates all
ranks' data, so it can check each tensor twice: against a float64 sum (within
f32 rounding), and bit for bit against the order in which a ring adds.

The ring rooted at r reduces along r+1 -> r+2 -> ... -> r, so a chunk's value is
((x[r+1] + x[r+2]) + ...) + x[r]; tensors travel in chunks of at most 1 MiB
(equal parts), and a chunk's root is the sum of the squared character codes of
its name, modulo the number of ranks (the reference picks roots the same way:
src/stdml/collective/session.cpp:142-149, topology.cpp:98-126 there)."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from stdml_collective_experimental_b200.models.gradsets import gradset_sizes  # noqa: E402
from stdml_collective_experimental_b200.parallel import Peer  # noqa: E402

CHUNK_BYTES = 1 << 20


def rank_data(rank, sizes):
    g = torch.Generator().manual_seed(1000 + rank)
    return [torch.randn(n, generator=g) for n in sizes]


def ring_expected(parts, name, n):
    count = parts[0].numel()
    k = min(max(1, -(-count * 4 // CHUNK_BYTES)), count)
    out = torch.empty(count)
    q, r = divmod(count, k)
    for i in range(k):
        b = q * i + min(i, r)
        e = b + q + (1 if i < r else 0)
        root = sum(ord(c) ** 2 for c in f"part::{name}[{b}:{e}]") % n
        acc = parts[(root + 1) % n][b:e].clone()
        for step in range(2, n + 1):
            acc += parts[(root + step) % n][b:e]
        out[b:e] = acc
    return out


def main():
    rank, n, base = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    peers = [f"127.0.0.1:{base + r}" for r in range(n)]
    peer = Peer.from_list(rank, peers, strategy="ring")
    sess = peer.join()
    assert sess.strategy == "ring" and sess.size == n
    sizes = gradset_sizes("resnet50")
    assert len(sizes) == 161 and sum(sizes) == 25_557_032
    everyone = [rank_data(r, sizes) for r in range(n)]
    mine = [t.clone() for t in everyone[rank]]
    names = [f"grad:{i}" for i in range(len(sizes))]
    # the first half one call per tensor, the second half as one group
    half = len(sizes) // 2
    for i in range(half):
        sess.all_reduce(mine[i], name=names[i])
    sess.group_all_reduce(mine[half:], names=names[half:])
    worst = 0.0
    for i, got in enumerate(mine):
        parts = [everyone[r][i] for r in range(n)]
        wide = torch.stack([p.double() for p in parts]).sum(0)
        err = float((got.double() - wide).abs().max())
        worst = max(worst, err)
        assert err <= 4 * 2.0 ** -23 * float(torch.stack(parts).abs().sum(0).max()), (i, err)
        assert torch.equal(got, ring_expected(parts, names[i], n)), f"tensor {i}: not the ring's order"
    sess.close()
    peer.close()
    print(f"rank {rank} OK worst_abs_err {worst:.3e}", flush=True)


if __name__ == "__main__":
    main()
