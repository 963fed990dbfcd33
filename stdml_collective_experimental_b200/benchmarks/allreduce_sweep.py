"""Single-buffer all_reduce sweep: bus bandwidth vs message size, this library's
kernels (every algorithm) against NCCL on the same CUDA buffers.

    torchrun --nproc-per-node N -m stdml_collective_experimental_b200.benchmarks.allreduce_sweep \
        [--dtype f32|bf16] [--min-bytes 4] [--max-bytes 1073741824] [--blocks 64,128] [--out file.json]

Timing: CUDA events around `iters` back-to-back calls after warm-up, max over
ranks; busBW = 2(n-1)/n * bytes / t.  The reference's counterpart is
benchmarks/bench_all_reduce.cpp (host memory, wall clock).
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import DeviceSession


def timed(fn, iters, warmup, dev):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="f32")
    ap.add_argument("--min-bytes", type=int, default=4)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--blocks", default="0")
    ap.add_argument("--algos", default="oneshot,twoshot,nvls,nvls_oneshot,auto")
    ap.add_argument("--out", default="")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--configs", default="",
                    help="extra columns, ';'-separated: ALGO@knob=value,knob=value (knobs of "
                         "DeviceSession.set_knob), e.g. 'nvls@nvls_variant=2,nvls_blocks=48;"
                         "twoshot_tma@tma_blocks=64'; run zero-copy on the symmetric buffer")
    args = ap.parse_args()
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    dtype = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[args.dtype]
    es = torch.empty((), dtype=dtype).element_size()
    sess = DeviceSession.from_env(heap_bytes=args.max_bytes + (64 << 20), rank=rank, world=world,
                                  device=local)
    algos = [a for a in args.algos.split(",") if sess.has_nvls or not a.startswith("nvls")]
    blocks_list = [int(b) for b in args.blocks.split(",")]
    sym = sess.symm_empty(args.max_bytes // es, dtype)
    g = torch.Generator(device="cpu").manual_seed(rank)
    sym[: min(sym.numel(), 1 << 22)].copy_((torch.rand(min(sym.numel(), 1 << 22), generator=g) * 2 - 1).to(dtype))
    plain = torch.empty(args.max_bytes // es, dtype=dtype, device=dev)
    rows = []
    nbytes = max(args.min_bytes, es)
    while nbytes <= args.max_bytes:
        n = nbytes // es
        iters = 200 if nbytes <= (1 << 20) else (40 if nbytes <= (64 << 20) else 10)
        row = {"bytes": nbytes}
        bus = lambda ms: 2 * (world - 1) / world * nbytes / (ms * 1e-3) / 1e9  # noqa: E731
        if not args.no_nccl:
            ms = timed(lambda: dist.all_reduce(plain[:n]), iters, 5, dev)
            row["nccl"] = {"us": ms * 1e3, "busbw": bus(ms)}
        for algo in algos:
            for blocks in blocks_list:
                if blocks:
                    sess.set_tuning(max_blocks=blocks)
                key = algo if not blocks else f"{algo}/b{blocks}"
                try:
                    if algo in ("oneshot", "nvls_oneshot"):
                        if nbytes > (8 << 20):
                            continue
                        # staged one-shot: user tensor in, user tensor out
                        ms = timed(lambda: sess.all_reduce(plain[:n], algo=algo), iters, 5, dev)
                    elif algo == "auto":
                        ms = timed(lambda: sess.all_reduce(plain[:n]), iters, 5, dev)
                    elif algo == "auto_registered":
                        # ordinary tensor, its allocation mapped on every peer (no staging)
                        sess.set_knob("register_min_bytes", 4 << 20)  # below: staged, the handle exchange costs more than it saves
                        try:
                            ms = timed(lambda: sess.all_reduce(plain[:n]), iters, 5, dev)
                        finally:
                            sess.set_knob("register_min_bytes", -1)
                    else:
                        ms = timed(lambda: sess.all_reduce(sym[:n], algo=algo), iters, 5, dev)
                except ValueError:
                    continue
                row[key] = {"us": ms * 1e3, "busbw": bus(ms)}
        for cfg in filter(None, args.configs.split(";")):
            algo, _, knobs = cfg.partition("@")
            if algo.startswith("nvls") and not sess.has_nvls:
                continue
            pairs = [kv.split("=") for kv in filter(None, knobs.split(","))]
            for k, v in pairs:
                sess.set_knob(k, int(v))
            try:
                ms = timed(lambda: sess.all_reduce(sym[:n], algo=algo), iters, 5, dev)
                row[cfg] = {"us": ms * 1e3, "busbw": bus(ms)}
            except ValueError:
                pass
            for k, _ in pairs:
                sess.set_knob(k, {"nvls_variant": 1}.get(k, 0))
        sess.check()
        rows.append(row)
        if rank == 0:
            cells = " ".join(f"{k}={v['busbw']:.1f}/{v['us']:.0f}us" for k, v in row.items()
                             if isinstance(v, dict))
            print(f"{nbytes:>11d} B  {cells}", flush=True)
        nbytes *= 2
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump({"world": world, "dtype": args.dtype, "nvls": sess.has_nvls, "rows": rows}, f)
    dist.barrier()
    sess.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
