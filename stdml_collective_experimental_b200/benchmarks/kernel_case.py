"""A small, self-ending case of the fused all-reduce kernel on ONE GPU, sized for
profilers: `--world` ranks emulated in one cooperative launch (loopback world),
a symmetric buffer of `--mb` MiB per rank reduced in place, `--iters` launches.

    python -m stdml_collective_experimental_b200.benchmarks.kernel_case --world 4 --mb 64 --algo twoshot

Prints the device time per launch (CUDA events) and the bytes each launch must
move through HBM, so that an achieved fraction of the copy bandwidth can be
stated next to the profiler's counters.
"""
import argparse
import json

import torch

from .. import DeviceSession


def staged_group(args, sess, dtype, es):
    total = (args.mb << 20) // es
    k = args.staged_group
    # a few big tensors and many small ones, like a real gradient set
    sizes = [total // 2, total // 4] + [max(1, (total // 4) // (k - 2))] * (k - 2)
    ranks = [[torch.full((s,), float(r + 1), dtype=dtype, device="cuda") for s in sizes]
             for r in range(args.world)]
    arg = ranks if args.world > 1 else ranks[0]
    if args.registered:
        # reduced where they lie (group_peer_kernel): no pack, no unpack
        sess.set_knob("register_min_bytes", 0)
        if args.bulk_min_bytes is not None:
            sess.set_knob("group_bulk_min_bytes", args.bulk_min_bytes)
    torch.cuda.synchronize()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(args.iters + 1)]
    e[0].record()
    for i in range(args.iters):
        sess.group_all_reduce(arg, scale=1.0 / args.world,
                              algo=None if args.registered else args.algo)
        e[i + 1].record()
    torch.cuda.synchronize()
    sess.check()
    times = [e[i].elapsed_time(e[i + 1]) for i in range(args.iters)]
    nbytes = sum(sizes) * es
    # per rank: pack (read + write), reduce (read world, write world, amortised: read + write), unpack (read + write);
    # registered: the reduce alone
    hbm = (2 if args.registered else 6) * args.world * nbytes
    best = min(times[1:]) if len(times) > 1 else times[0]
    want = sum(range(1, args.world + 1)) / args.world
    assert args.iters > 1 or all(abs(float(t[-1]) - want) < 1e-3 for t in ranks[0]), "wrong result"
    print(json.dumps({"world": args.world, "tensors": k, "set_mb": nbytes / 2**20,
                      "algo": "registered" if args.registered else args.algo,
                      "ms_per_call": times, "best_ms": best, "hbm_bytes_per_call": hbm,
                      "achieved_gb_s": hbm / (best * 1e-3) / 1e9}))
    sess.close()


def other_collective(args, sess, dtype, es, n):
    w = args.world
    ins = [torch.full((n,), float(r + 1), dtype=dtype, device="cuda") for r in range(w)]
    outs = [torch.empty(n * w if args.collective == "all_gather" else n, dtype=dtype,
                        device="cuda") for _ in range(w)]
    a_in = ins if w > 1 else ins[0]
    a_out = outs if w > 1 else outs[0]
    torch.cuda.synchronize()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(args.iters + 1)]
    e[0].record()
    for i in range(args.iters):
        if args.collective == "all_gather":
            sess.all_gather(a_in, a_out)
        elif args.collective == "broadcast":
            sess.broadcast(a_in, out=a_out, root=0)
        else:
            sess.barrier()
        e[i + 1].record()
    torch.cuda.synchronize()
    sess.check()
    times = [e[i].elapsed_time(e[i + 1]) for i in range(args.iters)]
    best = min(times[1:]) if len(times) > 1 else times[0]
    nbytes = n * es
    # all_gather: pack (r+w) per rank, then every rank reads w blocks and writes w blocks
    hbm = {"all_gather": w * nbytes * (2 + 2 * w), "broadcast": nbytes * (2 + 2 * w),
           "barrier": 0}[args.collective]
    print(json.dumps({"collective": args.collective, "world": w, "mb_per_rank": args.mb,
                      "ms_per_launch": times, "best_ms": best, "hbm_bytes_per_launch": hbm,
                      "achieved_gb_s": hbm / (best * 1e-3) / 1e9 if hbm else None}))
    sess.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--mb", type=int, default=64)
    ap.add_argument("--dtype", default="f32")
    ap.add_argument("--algo", default="twoshot")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--blocks", type=int, default=0)
    ap.add_argument("--collective", default="all_reduce",
                    help="all_reduce | all_gather | broadcast | barrier")
    ap.add_argument("--staged-group", type=int, default=0,
                    help="N > 0: reduce N separately allocated tensors per rank (pack + reduce + "
                         "unpack through a descriptor table) instead of one symmetric buffer")
    ap.add_argument("--registered", action="store_true",
                    help="with --staged-group: register the tensors instead of staging them")
    ap.add_argument("--bulk-min-bytes", type=int, default=None,
                    help="with --registered: the group_bulk_min_bytes knob (-1: peer loads only)")
    args = ap.parse_args()
    dtype = {"f32": torch.float32, "bf16": torch.bfloat16}[args.dtype]
    es = 4 if args.dtype == "f32" else 2
    n = (args.mb << 20) // es
    sess = DeviceSession.loopback(args.world, heap_bytes=(args.mb << 20) + (8 << 20),
                                  staging_bytes=(args.mb + 1) << 20
                                  if (args.staged_group or args.collective != "all_reduce")
                                  else 1 << 20)
    if args.blocks:
        sess.set_tuning(max_blocks=args.blocks)
    if args.staged_group > 0:
        return staged_group(args, sess, dtype, es)
    if args.collective != "all_reduce":
        return other_collective(args, sess, dtype, es, n)
    sym = sess.symm_empty(n, dtype)
    bufs = sym if args.world > 1 else [sym]
    for r, b in enumerate(bufs):
        b.fill_(r + 1)
    torch.cuda.synchronize()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(args.iters + 1)]
    e[0].record()
    for i in range(args.iters):
        sess.all_reduce(sym, scale=1.0 / args.world, algo=args.algo)
        e[i + 1].record()
    torch.cuda.synchronize()
    sess.check()
    times = [e[i].elapsed_time(e[i + 1]) for i in range(args.iters)]
    best = min(times[1:]) if len(times) > 1 else times[0]
    # per launch: every rank's buffer is read once and written once
    hbm_bytes = 2 * args.world * n * es
    print(json.dumps({"world": args.world, "mb_per_rank": args.mb, "algo": args.algo,
                      "ms_per_launch": times, "best_ms": best,
                      "hbm_bytes_per_launch": hbm_bytes,
                      "achieved_gb_s": hbm_bytes / (best * 1e-3) / 1e9}))
    want = sum(range(1, args.world + 1)) / args.world
    assert abs(float(bufs[0][0]) - want) < 1e-3 or args.iters > 1
    sess.close()


if __name__ == "__main__":
    main()
