#!/usr/bin/env python
"""Headline benchmark: fused group_all_reduce of a BERT-base-shaped gradient set.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

One step = one all-reduce (sum, scaled by 1/N) of the whole gradient set
(199 f32 tensors, 109.5 M elements, 438 MB; every rank owns a full set: weak
scaling).  `value` = N x gradient-set bytes / step time, in GB/s, i.e. the
gradient bytes all-reduced per second summed over the job.  The timed region is
K back-to-back steps between barriers, timed with CUDA events, max over ranks.
`--impl reference` runs the reference's own bench-all-reduce binary (built
unmodified from its sources into baseline/_ref) on host memory with N
processes over TCP loopback and reports the same metric.
"""
import argparse
import json
import os
import re
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused grad-set allreduce throughput (N x set bytes / step), GB/s"


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="bert-base")
    p.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    p.add_argument("--algo", default="auto")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-extras", action="store_true",
                   help="skip the blocks beside the headline (other dtype, loopback kernel)")
    p.add_argument("--e2e-chunks", type=int, default=16)  # measured: 8 -> 10.04 ms, 16 -> 9.73, 32 -> 9.78
    p.add_argument("--strategy", default="RING", help="reference arm: RING or STAR")
    return p.parse_args()


def workload_config(workload, sizes, n, dtype):
    """The workload, in the same words for both arms; what differs between the
    implementations goes under `impl_detail`."""
    esize = 4 if dtype == "f32" else 2
    return {"model": workload, "tensors": len(sizes), "elements": sum(sizes),
            "set_bytes": esize * sum(sizes), "global_batch": None, "seq_len": None,
            "parallelism": f"dp{n}", "dtype": dtype, "op": "sum"}


def env_rank():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


# --------------------------------------------------------------------- reference
_UNITS = {"ns": 1e-6, "us": 1e-3, "ms": 1.0, "s": 1e3}


def run_reference(args):
    from stdml_collective_experimental_b200.models.gradsets import gradset_sizes, write_sizes_file
    rank, world, _ = env_rank()
    n = args.gpus
    binary = os.path.join(ROOT, "baseline", "_ref", "bin", "bench-all-reduce")

    def emit(obj):
        if rank == 0:
            print(json.dumps(obj), flush=True)

    if not os.path.exists(binary):
        emit({"impl": "reference", "unavailable":
              "baseline/_ref/bin/bench-all-reduce is missing (the reference is a CMake C++ "
              "project; pip cannot install it, its binaries are built with cmake into baseline/_ref)"})
        return 0
    if args.dtype != "f32":
        emit({"impl": "reference", "unavailable": "the reference implements no bf16/f16 reducers"})
        return 0
    if world not in (1, n):
        emit({"impl": "reference", "unavailable": f"launched with WORLD_SIZE={world}, --gpus {n}"})
        return 0
    sizes = gradset_sizes(args.workload)
    total_bytes = 4 * sum(sizes)
    base_port = 21000 + (int(os.environ.get("MASTER_PORT", "29500")) % 500) * 16
    peers = ",".join(f"127.0.0.1:{base_port + r}" for r in range(n))

    def launch(r, sizes_path):
        env = dict(os.environ)
        env.update({
            "KUNGFU_SELF_SPEC": f"127.0.0.1:{base_port + r}",
            "KUNGFU_INIT_PEERS": peers,
            "KUNGFU_INIT_RUNNERS": "127.0.0.1:38080",
            "KUNGFU_ALLREDUCE_STRATEGY": args.strategy,
            "STDML_COLLECTIVE_USE_THREAD_POOL": "1",
        })
        return subprocess.Popen([binary, sizes_path, str(args.steps), str(args.warmup)], env=env,
                                stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)

    with tempfile.TemporaryDirectory() as tmp:
        path = write_sizes_file(args.workload, os.path.join(tmp, f"{args.workload}.txt"))
        ranks = [rank] if world == n and n > 1 else list(range(n))
        procs = [launch(r, path) for r in ranks]
        outs = []
        try:
            for p in procs:
                outs.append(p.communicate(timeout=1500)[0])
        except subprocess.TimeoutExpired:
            for p in procs:
                p.kill()
            emit({"impl": "reference", "unavailable": "reference bench-all-reduce timed out"})
            return 0
    if rank != 0:
        return 0
    text = outs[0]
    m = re.search(r'took:\s*([0-9.]+)\s*(ns|us|ms|s)\s*@run_stage\("step"', text)
    if m is None or procs[0].returncode != 0:
        emit({"impl": "reference", "unavailable":
              "reference bench-all-reduce failed: " + text.strip().splitlines()[-1][:200]
              if text.strip() else "reference bench-all-reduce printed nothing"})
        return 0
    total_ms = float(m.group(1)) * _UNITS[m.group(2)]
    ms = total_ms / args.steps
    value = n * total_bytes / (ms * 1e-3) / 1e9
    final = re.search(r"FINAL RESULT:\s*\S+\s+([0-9.]+) GiB/s", text)
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": n,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "timing": "host wall clock of the reference's own benchmark loop (it has no device path)",
        "reference_metric_gib_s": float(final.group(1)) if final else None,
        # the reference reduces host buffers in place: its figure already is end to end
        # (host memory in, host memory out), with no device copies to count
        "e2e": {"value": value, "unit": "GB/s", "ms_per_step": ms, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0,
                "path": "host buffers -> TCP loopback ring -> host buffers (no GPU involved)"},
        "config": workload_config(args.workload, sizes, n, "f32"),
        "impl_detail": {"memory": "host", "transport": "tcp-loopback", "strategy": args.strategy,
                        "runtime": "rt_thread_pool", "scale": "not applied (the reference has none)"},
    })
    return 0


# -------------------------------------------------------------------------- ours
def run_ours(args):
    import torch
    import torch.distributed as dist

    from stdml_collective_experimental_b200 import DeviceSession
    from stdml_collective_experimental_b200.models.gradsets import gradset_sizes
    from stdml_collective_experimental_b200.parallel.host_pipeline import HostAllReduce
    from stdml_collective_experimental_b200.utils.clocks import ClockSampler

    rank, world, local = env_rank()
    n = args.gpus
    if world != n:
        if world == 1 and n > 1:
            # convenience: re-launch under torchrun
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                   f"--nproc-per-node={n}", "--master-addr", "127.0.0.1", "--master-port",
                   str(29500 + os.getpid() % 400)] + sys.argv
            return subprocess.call(cmd)
        raise SystemExit(f"WORLD_SIZE={world} but --gpus {n}")
    from stdml_collective_experimental_b200.utils.numa import bind_to_gpu_numa
    numa_node = bind_to_gpu_numa(local)  # before any pinned allocation
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if n > 1:
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local)  # NVML set-up stays outside the timed region

    def host_barrier():
        if n > 1:
            dist.barrier()

    def max_over_ranks(x):
        if n == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sizes = gradset_sizes(args.workload)
    scale = 1.0 / n
    algo = None if args.algo == "auto" else args.algo
    steps, warmup = args.steps, max(args.warmup, 3)

    def layout(esize):
        padded = [-(-s * esize // 16) * 16 // esize for s in sizes]
        return padded, sum(padded)

    max_total_bytes = layout(4)[1] * 4
    heap = 2 * max_total_bytes + layout(2)[1] * 2 + (96 << 20)
    sess = DeviceSession.from_env(heap_bytes=heap, rank=rank, world=n, device=local)

    def gradient_set(dtype_name, seed):
        """The set as one flat region of the symmetric heap, tensors as views of it,
        plus its pinned host twin (N(0, 1e-3), seeded per rank)."""
        dtype = torch.float32 if dtype_name == "f32" else torch.bfloat16
        esize = 4 if dtype_name == "f32" else 2
        padded, total = layout(esize)
        flat = sess.symm_empty(total, dtype)
        views, off = [], 0
        for s_, p_ in zip(sizes, padded):
            views.append(flat[off:off + s_])
            off += p_
        g = torch.Generator(device="cpu").manual_seed(seed + rank)
        host_in = torch.empty(total, dtype=dtype).pin_memory()
        host_in.copy_((torch.randn(total, generator=g) * 1e-3).to(dtype))
        flat.copy_(host_in, non_blocking=True)
        torch.cuda.synchronize()
        return dtype, esize, total, flat, views, host_in

    def check_against_nccl(flat, views, dtype):
        """Correctness of the exact call that is timed (against NCCL when N > 1,
        against the input itself when alone)."""
        check = flat.clone()
        sess.group_all_reduce(views, scale=scale, algo=algo)
        torch.cuda.synchronize()
        sess.check()
        if n > 1:
            dist.all_reduce(check)
            check.mul_(scale)
        err = float((flat.float() - check.float()).abs().max())
        ref_mag = float(check.float().abs().max())
        tol = 1e-6 if dtype == torch.float32 else 2e-2
        if not err <= tol * max(ref_mag, 1e-30) + 1e-12:
            raise SystemExit(f"rank {rank}: fused group_all_reduce mismatch: max err {err}")

    def timed_device_steps(views, with_sampler):
        def step():
            sess.group_all_reduce(views, scale=scale, algo=algo)

        if with_sampler:
            sampler.start()  # runs through the warm-up too: short regions still get samples
        for _ in range(warmup):
            step()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        torch.cuda.synchronize()
        host_barrier()
        sess.barrier()  # ranks leave the host barrier at different times: line them up on the device
        launches0 = sess.launches
        if with_sampler:
            sampler.mark_begin()
        ev[0].record()
        for i in range(steps):
            step()
            ev[i + 1].record()
        torch.cuda.synchronize()
        if with_sampler:
            sampler.mark_end()
        host_barrier()
        launches = sess.launches - launches0
        ms = max_over_ranks(ev[0].elapsed_time(ev[-1]) / steps)
        clocks = sampler.stop() if with_sampler else None
        sess.check()
        return ms, launches, clocks

    # ---- the headline: the set in the dtype asked for (f32 is what the reference can do)
    dtype, esize, total, flat, views, host_in = gradient_set(args.dtype, 1234)
    set_bytes = sum(sizes) * esize
    check_against_nccl(flat, views, dtype)
    ms, launches, clocks = timed_device_steps(views, True)
    value = n * set_bytes / (ms * 1e-3) / 1e9

    e2e = None
    if not args.no_e2e:
        host_out = torch.empty(total, dtype=dtype).pin_memory()
        pipe = HostAllReduce(sess, total, dtype, chunks=args.e2e_chunks)
        for _ in range(3):
            pipe.run(host_in, host_out, scale=scale)
        torch.cuda.synchronize()
        host_barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            pipe.run(host_in, host_out, scale=scale)
        torch.cuda.synchronize()
        dt_ms = (time.perf_counter() - t0) * 1e3 / steps
        host_barrier()
        e2e_ms = max_over_ranks(dt_ms)
        e2e = {"value": n * set_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
               "ms_per_step": e2e_ms, "h2d_bytes_per_step": pipe.h2d_bytes,
               "d2h_bytes_per_step": pipe.d2h_bytes,
               "path": "pinned host set -> H2D -> fused all-reduce in the symmetric heap -> D2H "
                       f"(HostAllReduce, {args.e2e_chunks} chunks pipelined on 3 streams)"}
        sess.check()
        pipe.close()
        del host_out

    # ---- the same set in the other float width (bf16 when the headline is f32): the
    # reference has no 16-bit reducers, so this block has no counterpart in its arm
    other = None
    other_name = "bf16" if args.dtype == "f32" else "f32"
    if not args.no_extras:
        try:
            o_dtype, o_esize, _, o_flat, o_views, _ = gradient_set(other_name, 4321)
            check_against_nccl(o_flat, o_views, o_dtype)
            o_ms, o_launches, _ = timed_device_steps(o_views, False)
            o_bytes = sum(sizes) * o_esize
            other = {"dtype": other_name, "set_bytes": o_bytes, "ms_per_step": o_ms,
                     "value": n * o_bytes / (o_ms * 1e-3) / 1e9, "unit": "GB/s",
                     "bus_bandwidth_gb_s": 2 * (n - 1) / n * o_bytes / (o_ms * 1e-3) / 1e9,
                     "gpu_launches": o_launches}
            sess.symm_free(o_flat)
        except Exception as e:  # an extra must never cost the headline
            other = {"dtype": other_name, "error": str(e)[:200]}

    bus = 2 * (n - 1) / n * set_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": n, "steps": steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "impl": "ours", "bus_bandwidth_gb_s": bus, "gpu_launches": launches, "clocks": clocks,
        "e2e": e2e, "also_" + other_name: other,
        "config": workload_config(args.workload, sizes, n, args.dtype),
        "impl_detail": {"memory": "symmetric heap (zero-copy)", "nvls": sess.has_nvls,
                        "backend": sess.backend, "numa_node": numa_node, "scale": "fused, 1/N",
                        "l2": f"inputs ({set_bytes >> 20} MB per rank) are larger than the 126 MB "
                              "L2; no flush"},
    }
    host_barrier()
    sess.close()
    if n == 1 and not args.no_extras:
        # Alone on a GPU an all-reduce is a scaled copy: no barrier, no peer.  So that
        # a one-GPU run still exercises the collective kernel itself, the same set is
        # also reduced among 8 ranks emulated on this GPU (one cooperative launch,
        # every "peer" access an HBM access).  Reported beside the headline, not in it.
        try:
            out["kernel_loopback8"] = loopback_kernel_block(args, sizes, steps, warmup)
        except Exception as e:
            out["kernel_loopback8"] = {"error": str(e)[:200]}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def loopback_kernel_block(args, sizes, steps, warmup, world=8):
    import torch

    from stdml_collective_experimental_b200 import DeviceSession
    esize = 4 if args.dtype == "f32" else 2
    dtype = torch.float32 if args.dtype == "f32" else torch.bfloat16
    padded = [-(-s * esize // 16) * 16 // esize for s in sizes]
    total = sum(padded)
    with DeviceSession.loopback(world, heap_bytes=total * esize + (32 << 20),
                                staging_bytes=1 << 20) as sess:
        flats = sess.symm_empty(total, dtype)
        for r, f in enumerate(flats):
            f.normal_(0, 1e-3, generator=torch.Generator(device="cuda").manual_seed(r))
        views = []
        for f in flats:
            off, vs = 0, []
            for s_, p_ in zip(sizes, padded):
                vs.append(f[off:off + s_])
                off += p_
            views.append(vs)
        want = torch.stack([f.double() for f in flats]).sum(0) / world
        sess.group_all_reduce(views, scale=1.0 / world)
        torch.cuda.synchronize()
        sess.check()
        err = float((flats[3].double() - want).abs().max())
        if not err <= (1e-6 if esize == 4 else 2e-2) * float(want.abs().max()) + 1e-12:
            raise RuntimeError(f"loopback all-reduce mismatch: {err}")
        del want
        for _ in range(warmup):
            sess.group_all_reduce(views, scale=1.0 / world)
        l0 = sess.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            sess.group_all_reduce(views, scale=1.0 / world)
        e1.record()
        torch.cuda.synchronize()
        sess.check()
        ms = e0.elapsed_time(e1) / steps
        hbm = 2 * world * total * esize  # every rank's set is read once and written once
        return {"ranks_emulated": world, "ms_per_step": ms, "gpu_launches": sess.launches - l0,
                "hbm_bytes_per_step": hbm, "hbm_gb_s": hbm / (ms * 1e-3) / 1e9,
                "kernel": "owner_kernel (bulk-copy two-shot), one cooperative launch per step"}


def keep_stdout_for_the_result():
    """Libraries write to file descriptor 1 on their own (NCCL prints its version there when
    NCCL_DEBUG is set in the environment).  The contract is ONE JSON line on stdout, so
    everything else that this process or its children write to fd 1 goes to stderr, and
    only print() reaches the real stdout."""
    sys.stdout.flush()
    real = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real, "w", buffering=1)


def main():
    args = parse_args()
    keep_stdout_for_the_result()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
