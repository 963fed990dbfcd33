"""Elastic workload: BERT-base-shaped gradient all-reduce + 4 MB all_gather +
broadcast from rank 0 every iteration, with the membership changing at fixed
steps; survivors keep their process, joiners are started by the runner.

    csrc/build/bin/stdml_collective_run -np 8 -w -builtin-config-port 0 \
        python -m stdml_collective_experimental_b200.benchmarks.elastic \
        --max-step 200 --schedule 50:4,100:6,150:8 [--device cuda|cpu] [--model bert-base]

Reports, on rank 0 of each membership: resize latency (agreement + commit + new
session), the cost of the first collectives on the new device world broken down
(step agreement on the host, device world + heap, first kernels, state
broadcast; and inside the device world: rendezvous, own arena, peer arenas,
multicast), and the steady-state bus bandwidth of the gradient all-reduce after
each resize (gradients live in the new membership's symmetric heap; CUDA
events).  Schedules that drop members run with STDML_COLLECTIVE_NVLS=0.  The reference's
counterpart is examples/example-elastic.cpp driven by kungfu-run.
"""
import argparse
import json
import os
import time

import torch

from ..models.gradsets import gradset_sizes
from ..parallel import Peer
from ..parallel.peer import standby_wait


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-step", type=int, default=200)
    ap.add_argument("--schedule", default="")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--model", default="bert-base")
    ap.add_argument("--state-mb", type=float, default=4.0)
    args = ap.parse_args()
    schedule = {}
    for item in filter(None, args.schedule.split(",")):
        k, v = item.split(":")
        schedule[int(k)] = int(v)

    use_cuda = args.device == "cuda"
    # a warm standby (launcher option -spares) learns here which worker, and so which GPU, it is
    standby_wait()
    if use_cuda:
        dev_id = int(os.environ.get("STDML_COLLECTIVE_DEVICE_ID", os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev_id % torch.cuda.device_count())
        dev = torch.device("cuda", dev_id % torch.cuda.device_count())
    else:
        dev = torch.device("cpu")

    peer = Peer.from_env()
    sess = peer.join()
    try:
        run(args, peer, sess, schedule, use_cuda, dev)
    finally:
        # orderly on every path (detached, finished, error): the device world is
        # torn down (barrier -> unbind -> release) before the process goes
        sess.close()
        peer.close()


def shrinks(size_now, schedule, from_step=0):
    """True if following `schedule` ({step: size}) from `size_now` ever drops members."""
    cur = size_now
    for k in sorted(schedule):
        if k < from_step:
            continue
        if schedule[k] < cur:
            return True
        cur = schedule[k]
    return False


def nvls_requested():
    return os.environ.get("STDML_COLLECTIVE_NVLS", "1") not in ("0", "off", "false")


def run(args, peer, sess, schedule, use_cuda, dev):
    me = peer.self_id
    if use_cuda and shrinks(sess.size, schedule) and nvls_requested():
        # A rank that leaves while its arena is bound to an NVLink multicast
        # object can fault the GPUs of the ranks that stay.  Runs in which the
        # membership shrinks therefore use plain peer loads (two-shot); the
        # NVLS figures belong to fixed-membership runs.
        raise SystemExit("elastic: this schedule drops members; set STDML_COLLECTIVE_NVLS=0 "
                         "(and NCCL_NVLS_ENABLE=0) for runs in which a rank leaves")
    sizes = gradset_sizes(args.model)
    set_bytes = 4 * sum(sizes)
    padded = [-(-n * 4 // 16) * 4 for n in sizes]  # tensors start on 16-byte boundaries
    state_n = int(args.state_mb * (1 << 20)) // 4
    state = torch.zeros(state_n, device=dev)
    weights = torch.zeros(1 << 20, device=dev)

    def sync():
        if use_cuda:
            torch.cuda.synchronize()

    def log(obj):
        print(json.dumps(obj), flush=True)

    def gradient_views():
        """The gradient set of this membership.  On GPUs it lives in the session's
        symmetric heap as one flat region (tensors are views of it), so that the
        group all-reduce is ONE zero-copy launch; the heap belongs to a membership,
        hence this runs again after every resize."""
        if not use_cuda:
            return None, [torch.empty(n) for n in sizes]
        flat = sess.symm_empty(sum(padded), torch.float32, dev)
        views, off = [], 0
        for n, p in zip(sizes, padded):
            views.append(flat[off:off + n])
            off += p
        return flat, views

    def timed_ms(fn):
        """Device time of fn() on GPUs (CUDA events), wall clock on CPUs."""
        if not use_cuda:
            t0 = time.perf_counter()
            fn()
            return (time.perf_counter() - t0) * 1e3
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1)

    step = 0
    synced = False
    flat, grads = None, None
    window = []  # all-reduce times since the last resize
    while step < args.max_step:
        if not synced:
            t0 = time.perf_counter()
            s = torch.tensor([step], dtype=torch.int64)
            step = int(sess.all_reduce(s, op="max").item())      # joiners catch up
            t1 = time.perf_counter()
            flat, grads = gradient_views()       # first device call: builds the device world
            sync()
            t2 = time.perf_counter()
            sess.barrier()
            if use_cuda:
                probe = grads[0][:4]
                sess.all_reduce(probe)            # first kernel of the new world
            sync()
            t3 = time.perf_counter()
            sess.broadcast(weights)                               # model state from rank 0
            sync()
            t4 = time.perf_counter()
            if sess.rank == 0:
                log({"event": "state_sync", "version": sess.version, "size": sess.size,
                     "step": step, "first_collectives_ms": (t4 - t0) * 1e3,
                     "breakdown_ms": {"step_agreement_host": (t1 - t0) * 1e3,
                                      "device_world_and_heap": (t2 - t1) * 1e3,
                                      "first_kernels": (t3 - t2) * 1e3,
                                      "state_broadcast_4MB": (t4 - t3) * 1e3},
                     "device_world_setup_ms": sess.device_setup_ms if use_cuda else None})
            synced = True
            window = []
            if step >= args.max_step:
                break
        if flat is not None:
            flat.fill_(1.0)
        else:
            for g in grads:
                g.fill_(1.0)
        sync()
        sess.barrier()
        ar_ms = timed_ms(lambda: sess.group_all_reduce(grads, scale=1.0 / sess.size))
        gathered = torch.empty(state_n * sess.size, device=dev)
        sess.all_gather(state, gathered)
        sess.broadcast(state)
        weights.add_(1.0)
        sync()
        window.append(ar_ms)
        if abs(float(grads[-1][0]) - 1.0) > 1e-6:
            raise SystemExit(f"{me}: wrong all-reduce result at step {step}")
        if step in schedule:
            old_size = sess.size
            steady = sorted(window[len(window) // 2:])
            med = steady[len(steady) // 2] if steady else None
            flat, grads = None, None  # the heap goes with the membership
            t0 = time.perf_counter()
            changed, detached = peer.resize(sess, new_size=schedule[step])
            ms = (time.perf_counter() - t0) * 1e3
            if detached:
                log({"event": "detached", "peer": me, "step": step})
                return
            if changed:
                if sess.rank == 0:
                    log({"event": "resized", "step": step, "old_size": old_size,
                         "new_size": sess.size, "version": sess.version, "resize_ms": ms,
                         "prev_allreduce_ms_median": med,
                         "prev_bus_gb_s": None if not med else
                         2 * (old_size - 1) / old_size * set_bytes / (med * 1e-3) / 1e9})
                synced = False
            else:
                flat, grads = gradient_views()
        step += 1
    if sess.rank == 0:
        steady = sorted(window[len(window) // 2:])
        med = steady[len(steady) // 2] if steady else None
        n = sess.size
        log({"event": "finished", "size": n, "version": sess.version, "steps": step,
             "allreduce_ms_median": med, "timing": "CUDA events" if use_cuda else "wall clock",
             "gradients": "symmetric heap, one fused launch" if use_cuda else "host tensors",
             "bus_gb_s": None if not med else 2 * (n - 1) / n * set_bytes / (med * 1e-3) / 1e9,
             "weights_ok": bool(abs(float(weights[0]) - args.max_step) < 1e-3)})


if __name__ == "__main__":
    main()
