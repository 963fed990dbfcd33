"""Elastic workload: BERT-base-shaped gradient all-reduce + 4 MB all_gather +
broadcast from rank 0 every iteration, with the membership changing at fixed
steps; survivors keep their process, joiners are started by the runner.

    csrc/build/bin/stdml_collective_run -np 8 -w -builtin-config-port 0 \
        python -m stdml_collective_experimental_b200.benchmarks.elastic \
        --max-step 200 --schedule 50:4,100:6,150:8 [--device cuda|cpu] [--model bert-base]

Reports, on rank 0 of each membership: resize latency (agreement + commit + new
session, and separately the first collective on the new device world, which
builds the new arenas / peer mappings / multicast object) and the steady-state
bus bandwidth of the gradient all-reduce after each resize.  The reference's
counterpart is examples/example-elastic.cpp driven by kungfu-run.
"""
import argparse
import json
import os
import time

import torch

from ..models.gradsets import gradset_sizes
from ..parallel import Peer


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
    grads = [torch.full((n,), 1.0, device=dev) for n in sizes]
    state_n = int(args.state_mb * (1 << 20)) // 4
    state = torch.zeros(state_n, device=dev)
    weights = torch.zeros(1 << 20, device=dev)

    def sync():
        if use_cuda:
            torch.cuda.synchronize()

    def log(obj):
        print(json.dumps(obj), flush=True)

    step = 0
    synced = False
    window = []  # step times since the last resize
    while step < args.max_step:
        if not synced:
            t0 = time.perf_counter()
            s = torch.tensor([step], dtype=torch.int64)
            step = int(sess.all_reduce(s, op="max").item())      # joiners catch up
            sess.broadcast(weights)                               # model state from rank 0
            sync()
            first_ms = (time.perf_counter() - t0) * 1e3
            if sess.rank == 0:
                log({"event": "state_sync", "version": sess.version, "size": sess.size,
                     "step": step, "first_collectives_ms": first_ms})
            synced = True
            window = []
            if step >= args.max_step:
                break
        for g in grads:
            g.fill_(1.0)
        sync()
        sess.barrier()
        t0 = time.perf_counter()
        sess.group_all_reduce(grads, scale=1.0 / sess.size)
        sync()
        ar_ms = (time.perf_counter() - t0) * 1e3
        gathered = torch.empty(state_n * sess.size, device=dev)
        sess.all_gather(state, gathered)
        sess.broadcast(state)
        weights.add_(grads[0][0].item() if False else 1.0)
        sync()
        window.append(ar_ms)
        if abs(float(grads[-1][0]) - 1.0) > 1e-6:
            raise SystemExit(f"{me}: wrong all-reduce result at step {step}")
        if step in schedule:
            t0 = time.perf_counter()
            changed, detached = peer.resize(sess, new_size=schedule[step])
            ms = (time.perf_counter() - t0) * 1e3
            if detached:
                log({"event": "detached", "peer": me, "step": step})
                return
            if changed:
                if sess.rank == 0:
                    steady = sorted(window[len(window) // 2:])
                    med = steady[len(steady) // 2] if steady else None
                    log({"event": "resized", "step": step, "new_size": sess.size,
                         "version": sess.version, "resize_ms": ms,
                         "prev_allreduce_ms_median": med})
                synced = False
        step += 1
    if sess.rank == 0:
        steady = sorted(window[len(window) // 2:])
        med = steady[len(steady) // 2] if steady else None
        n = sess.size
        log({"event": "finished", "size": n, "version": sess.version, "steps": step,
             "allreduce_ms_median": med,
             "bus_gb_s": None if not med else 2 * (n - 1) / n * set_bytes / (med * 1e-3) / 1e9,
             "weights_ok": bool(abs(float(weights[0]) - args.max_step) < 1e-3)})


if __name__ == "__main__":
    main()
