"""Fused group_all_reduce of whole gradient sets against an NCCL baseline.

    torchrun --nproc-per-node N -m stdml_collective_experimental_b200.benchmarks.gradset \
        [--sets resnet50:f32,vgg16:f32,bert-base:f32,bert-large:bf16] [--iters 20]

Per set and rank count, device-timed (CUDA events, max over ranks), gradients
N(0, 1e-3) seeded per rank, averaged over the ranks:
  ours/arena   gradients live in the symmetric heap: ONE fused in-place launch
  ours/staged  gradients are ordinary CUDA tensors: pack + reduce + unpack fused,
               one launch per staging slot (descriptor table)
  ours/registered  the same ordinary tensors with register_min_bytes = 0: their
               allocations are mapped on every peer once, then ONE launch reduces
               them where they lie (no pack, no unpack)
  nccl/flat    ncclAllReduce on one flattened bucket + a separate scale kernel
  nccl/coalesced  torch's coalesced all_reduce over the tensor list + _foreach_mul_
busBW = 2(n-1)/n * set bytes / t.  The link roofline is 770 GB/s per direction
(measured peer copy); NVLS moves S(1+1/n) per direction instead of 2S(n-1)/n, so
its bus bandwidth can exceed that figure.
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import DeviceSession
from ..models.gradsets import gradset_sizes


def timed(fn, iters, warmup, dev, world):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sets", default="resnet50:f32,vgg16:f32,bert-base:f32,bert-base:bf16,bert-large:bf16")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in
                          (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sess = DeviceSession.from_env(heap_bytes=(1536 << 20), staging_bytes=(128 << 20), rank=rank,
                                  world=world, device=local)
    results = []
    for item in args.sets.split(","):
        name, dt = item.split(":")
        dtype = {"f32": torch.float32, "bf16": torch.bfloat16}[dt]
        es = 4 if dt == "f32" else 2
        sizes = gradset_sizes(name)
        lane = 16 // es
        padded = [-(-s // lane) * lane for s in sizes]
        total = sum(padded)
        set_bytes = sum(sizes) * es
        scale = 1.0 / world
        g = torch.Generator(device="cpu").manual_seed(7 + rank)
        src = (torch.randn(total, generator=g) * 1e-3).to(dtype).to(dev)

        flat = sess.symm_empty(total, dtype)
        views, off = [], 0
        for s, p in zip(sizes, padded):
            views.append(flat[off:off + s])
            off += p
        plain_flat = torch.empty(total, dtype=dtype, device=dev)
        plain = list(torch.split(plain_flat, padded))
        plain = [t[:s] for t, s in zip(plain, sizes)]
        loose = [torch.empty(s, dtype=dtype, device=dev) for s in sizes]  # separately allocated

        # correctness of both paths against NCCL once
        flat.copy_(src)
        for t, v in zip(loose, views):
            t.copy_(v)
        ref = src.clone()
        if world > 1:
            dist.all_reduce(ref)
        ref.mul_(scale)
        sess.group_all_reduce(views, scale=scale)
        sess.group_all_reduce(loose, scale=scale)
        torch.cuda.synchronize()
        sess.check()
        tol = 1e-6 if dt == "f32" else 2e-2
        mag = float(ref.float().abs().max())
        err_a = float((flat.float() - ref.float()).abs().max())
        ref_parts = list(torch.split(ref, padded))
        picks = sorted(set(list(range(min(8, len(sizes)))) + list(range(max(0, len(sizes) - 8), len(sizes)))))
        err_s = max(float((loose[i].float() - ref_parts[i][:sizes[i]].float()).abs().max())
                    for i in picks)
        ok = err_a <= tol * mag + 1e-9 and err_s <= tol * mag + 1e-9

        row = {"set": name, "dtype": dt, "tensors": len(sizes), "bytes": set_bytes, "n": world,
               "verified": bool(ok)}
        bus = lambda ms: 2 * (world - 1) / world * set_bytes / (ms * 1e-3) / 1e9  # noqa: E731
        l0 = sess.launches
        ms = timed(lambda: sess.group_all_reduce(views, scale=scale), args.iters, 3, dev, world)
        row["ours_arena"] = {"ms": ms, "busbw": bus(ms),
                             "launches_per_call": (sess.launches - l0) // (args.iters + 3)}
        l0 = sess.launches
        ms = timed(lambda: sess.group_all_reduce(loose, scale=scale), args.iters, 3, dev, world)
        row["ours_staged"] = {"ms": ms, "busbw": bus(ms),
                              "launches_per_call": (sess.launches - l0) // (args.iters + 3)}
        if dt == "f32":
            ms = timed(lambda: sess.group_all_reduce(loose, scale=scale, wire_dtype=torch.bfloat16),
                       args.iters, 3, dev, world)
            row["ours_staged_bf16_wire"] = {"ms": ms, "busbw_equiv": bus(ms)}
        if world > 1:
            sess.set_knob("register_min_bytes", 0)
            for t, v in zip(loose, ref_parts):
                t.copy_(v[:t.numel()])  # a known value again: every rank holds the mean
            sess.group_all_reduce(loose)  # sum of n equal means = n * mean
            torch.cuda.synchronize()
            sess.check()
            err_r = max(float((loose[i].float() - world * ref_parts[i][:sizes[i]].float()).abs().max())
                        for i in picks)
            row["verified"] = bool(ok and err_r <= world * tol * mag + 1e-9)
            l0 = sess.launches
            ms = timed(lambda: sess.group_all_reduce(loose, scale=scale), args.iters, 3, dev, world)
            row["ours_registered"] = {"ms": ms, "busbw": bus(ms),
                                      "launches_per_call": (sess.launches - l0) // (args.iters + 3)}
            sess.drop_registrations()
            sess.set_knob("register_min_bytes", -1)

            def nccl_flat():
                dist.all_reduce(plain_flat)
                plain_flat.mul_(scale)
            ms = timed(nccl_flat, args.iters, 3, dev, world)
            row["nccl_flat"] = {"ms": ms, "busbw": bus(ms)}

            def nccl_coalesced():
                dist.all_reduce_coalesced(loose) if hasattr(dist, "all_reduce_coalesced") else None
                torch._foreach_mul_(loose, scale)
            try:
                ms = timed(nccl_coalesced, max(3, args.iters // 4), 2, dev, world)
                row["nccl_coalesced"] = {"ms": ms, "busbw": bus(ms)}
            except Exception as e:  # not every torch build keeps this API
                row["nccl_coalesced"] = {"error": str(e)[:80]}
        results.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        sess.symm_free(flat)
        del views, plain, loose, plain_flat, src, ref
        torch.cuda.empty_cache()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump({"world": world, "nvls": sess.has_nvls, "rows": results}, f)
    if world > 1:
        dist.barrier()
    sess.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
