"""Host-memory (TCP loopback) benchmark suite: this library's C++ benchmarks next
to the reference's own binaries on the same machine, same workloads, same
metric ("GiB/s" = 4 (np-1) bytes / s / 2^30, rank 0, mean over steps).

    python -m stdml_collective_experimental_b200.benchmarks.host_suite [--np 4] [--out table.md]

Plays the role of the reference's scripts/bench/1.sh and scripts/bench/group.sh.
The reference binaries are looked up in baseline/_ref/bin (built from the
unmodified reference sources with cmake); rows are skipped when they are absent.
"""
import argparse
import os
import re
import subprocess
import tempfile

from .. import _native
from ..models.gradsets import GRADSETS, SWEEP, write_sizes_file

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
OURS = os.path.join(_native.CSRC, "build", "bin")
REF = os.path.join(ROOT, "baseline", "_ref", "bin")


def run_ours(prog, np_, strategy, workload, steps, warmup, env=None, timeout=600):
    e = dict(os.environ, **(env or {}))
    cmd = [os.path.join(OURS, "stdml_collective_run"), "-q", "-np", str(np_), "-strategy", strategy,
           os.path.join(OURS, prog), workload, str(steps), str(warmup)]
    try:
        out = subprocess.run(cmd, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                             text=True, timeout=timeout).stdout
    except subprocess.TimeoutExpired:
        return "hang"
    m = re.search(r"FINAL RESULT: \S+ ([0-9.]+) GiB/s", out)
    return float(m.group(1)) if m else "fail"


def run_ref(prog, np_, strategy, workload, steps, warmup, env=None, timeout=120):
    binary = os.path.join(REF, prog)
    if not os.path.exists(binary):
        return None
    peers = ",".join(f"127.0.0.1:{11000 + r}" for r in range(np_))
    procs = []
    for r in range(np_):
        e = dict(os.environ, KUNGFU_SELF_SPEC=f"127.0.0.1:{11000 + r}", KUNGFU_INIT_PEERS=peers,
                 KUNGFU_INIT_RUNNERS="127.0.0.1:38080", KUNGFU_ALLREDUCE_STRATEGY=strategy,
                 **(env or {}))
        procs.append(subprocess.Popen([binary, workload, str(steps), str(warmup)], env=e,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    hang = False
    for p in procs:
        try:
            outs.append(p.communicate(timeout=timeout)[0])
        except subprocess.TimeoutExpired:
            hang = True
            break
    if hang:
        for p in procs:
            p.kill()
            p.wait()
        return "hang"
    m = re.search(r"FINAL RESULT: \S+\s+([0-9.]+) GiB/s", outs[0])
    return float(m.group(1)) if m else "fail"


def fmt(x):
    if x is None:
        return "n/a"
    return f"{x:.3f}" if isinstance(x, float) else str(x)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--np", type=int, default=4)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--workloads", default="1024x100,16384x100,102400x100,262144x10,resnet50,vgg16")
    ap.add_argument("--out", default="")
    ap.add_argument("--strategies", default="RING,STAR",
                    help="comma list of RING, STAR, BINARY_TREE, CLIQUE (the reference knows the first two)")
    args = ap.parse_args()
    # "sweep" stands for the reference's AxB list (testdata/test-set-1.txt there)
    args.workloads = ",".join(",".join(SWEEP) if w == "sweep" else w
                              for w in args.workloads.split(","))
    _native.build()
    lines = ["| workload | strategy | ours all_reduce (threads) | ours all_reduce (pool) | "
             "ours group_all_reduce | ref all_reduce (threads) | ref all_reduce (pool) | "
             "ref group_all_reduce |", "|---|---|---|---|---|---|---|---|"]
    pool = {"STDML_COLLECTIVE_USE_THREAD_POOL": "1"}
    with tempfile.TemporaryDirectory() as tmp:
        for w in args.workloads.split(","):
            path = write_sizes_file(w, os.path.join(tmp, w + ".txt")) if w in GRADSETS else w
            for strategy in args.strategies.split(","):
                a = (args.np, strategy, path, args.steps, args.warmup)
                row = [run_ours("bench_all_reduce", *a), run_ours("bench_all_reduce", *a, env=pool),
                       run_ours("bench_group_all_reduce", *a)]
                if strategy in ("RING", "STAR"):
                    row += [run_ref("bench-all-reduce", *a), run_ref("bench-all-reduce", *a, env=pool),
                            run_ref("bench-group-all-reduce", *a, timeout=60)]
                else:
                    row += [None, None, None]
                line = f"| {w} | {strategy} | " + " | ".join(fmt(x) for x in row) + " |"
                print(line, flush=True)
                lines.append(line)
    if args.out:
        with open(args.out, "w") as f:
            f.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    main()
