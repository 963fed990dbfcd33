"""all_gather / broadcast / reduce sweeps against NCCL on the same CUDA buffers.

    torchrun --nproc-per-node N -m stdml_collective_experimental_b200.benchmarks.collectives_sweep \
        [--sizes 4096,65536,1048576,4194304,67108864]

Sizes are bytes per rank (all_gather: per-rank block).  Device-timed, max over
ranks.  GB/s figures: all_gather (n-1)/n * n*bytes / t; broadcast and reduce bytes / t.
Three forms of each call: ordinary tensors staged through the arena, ordinary
tensors registered (their allocations mapped on every peer, no staging), and
tensors that live in the symmetric heap (zero-copy, through the switch where
there is one).
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import DeviceSession
from .allreduce_sweep import timed


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="4096,65536,1048576,4194304,67108864")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    sizes = [int(s) for s in args.sizes.split(",")]
    sess = DeviceSession.from_env(heap_bytes=(world + 2) * max(sizes) + (64 << 20),
                                  staging_bytes=128 << 20, rank=rank, world=world, device=local)
    rows = []
    for nbytes in sizes:
        n = nbytes // 4
        iters = 100 if nbytes <= (1 << 20) else 20
        x = torch.full((n,), float(rank), device=dev)
        out = torch.empty(n * world, device=dev)
        row = {"bytes": nbytes}
        ms = timed(lambda: sess.all_gather(x, out), iters, 5, dev)
        ok = all(float(out[r * n]) == r and float(out[(r + 1) * n - 1]) == r for r in range(world))
        row["all_gather"] = {"us": ms * 1e3, "gb_s": (world - 1) * nbytes / (ms * 1e-3) / 1e9, "ok": ok}
        ms = timed(lambda: dist.all_gather_into_tensor(out, x), iters, 5, dev)
        row["nccl_all_gather"] = {"us": ms * 1e3, "gb_s": (world - 1) * nbytes / (ms * 1e-3) / 1e9}
        b = torch.full((n,), float(rank), device=dev)
        ms = timed(lambda: sess.broadcast(b, root=0), iters, 5, dev)
        row["broadcast"] = {"us": ms * 1e3, "gb_s": nbytes / (ms * 1e-3) / 1e9,
                            "ok": float(b[0]) == 0.0 and float(b[-1]) == 0.0}
        ms = timed(lambda: dist.broadcast(b, 0), iters, 5, dev)
        row["nccl_broadcast"] = {"us": ms * 1e3, "gb_s": nbytes / (ms * 1e-3) / 1e9}
        r_in = torch.ones(n, device=dev)
        r_out = torch.zeros(n, device=dev)
        ms = timed(lambda: sess.reduce(r_in, out=r_out, root=0), iters, 5, dev)
        row["reduce"] = {"us": ms * 1e3, "gb_s": nbytes / (ms * 1e-3) / 1e9,
                         "ok": rank != 0 or float(r_out[0]) == world}
        ms = timed(lambda: dist.reduce(r_in.clone(), 0), iters, 5, dev)
        row["nccl_reduce_incl_clone"] = {"us": ms * 1e3}
        # registered: the same ordinary tensors, no staging
        sess.set_knob("register_min_bytes", 4 << 20)  # below: staged, the handle exchange costs more than it saves
        out.zero_()
        ms = timed(lambda: sess.all_gather(x, out), iters, 5, dev)
        ok = all(float(out[r * n]) == r and float(out[(r + 1) * n - 1]) == r for r in range(world))
        row["all_gather_registered"] = {"us": ms * 1e3, "gb_s": (world - 1) * nbytes / (ms * 1e-3) / 1e9, "ok": ok}
        b.fill_(float(rank))
        ms = timed(lambda: sess.broadcast(b, root=0), iters, 5, dev)
        row["broadcast_registered"] = {"us": ms * 1e3, "gb_s": nbytes / (ms * 1e-3) / 1e9,
                                       "ok": float(b[0]) == 0.0 and float(b[-1]) == 0.0}
        r_out.zero_()
        ms = timed(lambda: sess.reduce(r_in, out=r_out, root=0), iters, 5, dev)
        row["reduce_registered"] = {"us": ms * 1e3, "gb_s": nbytes / (ms * 1e-3) / 1e9,
                                    "ok": rank != 0 or float(r_out[0]) == world}
        sess.set_knob("register_min_bytes", -1)
        # symmetric heap: zero-copy
        s_out = sess.symm_empty(n * world, torch.float32)
        s_out.zero_()
        ms = timed(lambda: sess.all_gather(x, s_out), iters, 5, dev)
        ok = all(float(s_out[r * n]) == r and float(s_out[(r + 1) * n - 1]) == r for r in range(world))
        row["all_gather_symmetric"] = {"us": ms * 1e3, "gb_s": (world - 1) * nbytes / (ms * 1e-3) / 1e9, "ok": ok}
        sess.set_knob("gather_mc", 1)
        ms = timed(lambda: sess.all_gather(x, s_out), iters, 5, dev)
        row["all_gather_symmetric_through_switch"] = {"us": ms * 1e3, "gb_s": (world - 1) * nbytes / (ms * 1e-3) / 1e9}
        sess.set_knob("gather_mc", 0)
        sess.symm_free(s_out)
        s_b = sess.symm_empty(n, torch.float32)
        s_b.fill_(float(rank))
        ms = timed(lambda: sess.broadcast(s_b, root=0), iters, 5, dev)
        row["broadcast_symmetric"] = {"us": ms * 1e3, "gb_s": nbytes / (ms * 1e-3) / 1e9,
                                      "ok": float(s_b[0]) == 0.0 and float(s_b[-1]) == 0.0}
        s_b.fill_(1.0)
        r_out.zero_()
        ms = timed(lambda: sess.reduce(s_b, out=r_out, root=0), iters, 5, dev)
        row["reduce_symmetric"] = {"us": ms * 1e3, "gb_s": nbytes / (ms * 1e-3) / 1e9,
                                   "ok": rank != 0 or float(r_out[0]) == world}
        sess.symm_free(s_b)
        ms = timed(lambda: sess.barrier(), 200, 10, dev)
        row["barrier_us"] = ms * 1e3
        sess.check()
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump({"world": world, "rows": rows}, f)
    dist.barrier()
    sess.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
