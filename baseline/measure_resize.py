#!/usr/bin/env python
"""Resize latency of the reference implementation and of this library, measured
by ONE driver source (baseline/resize_driver.cpp) that uses only the public API
the two share: peer::from_env, join_elastic, all_reduce, peer::resize(sess,
config_provider).

    python baseline/measure_resize.py [--impl reference --reference <its source tree> | --impl ours] [--schedule 8,4,6,8]

The reference's elastic launcher needs a Go toolchain, which is not available
offline, but its peer::resize(sess, config_provider) overload is plain C++.  This
script copies the reference sources to a scratch directory, builds its library
with cmake, compiles baseline/ref_resize_driver.cpp against it, and then plays
a membership schedule on CPU ranks over TCP loopback: it rewrites the
configuration file, starts joiners with the reference's environment contract
(its OpenMPI variables: ports 10000 + rank, no runners, star graph), and
collects the latencies that rank 0 prints.  Output: one JSON line."""
import argparse
import json
import os
import re
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def build_ours(out_bin):
    root = os.path.dirname(HERE)
    csrc = os.path.join(root, "stdml_collective_experimental_b200", "csrc")
    libdir = os.path.join(root, "stdml_collective_experimental_b200")
    os.makedirs(os.path.dirname(out_bin), exist_ok=True)
    subprocess.run(["g++", "-std=c++20", "-O2", "-pthread", "-I", os.path.join(csrc, "include"),
                    os.path.join(HERE, "resize_driver.cpp"), "-o", out_bin, "-L", libdir,
                    "-lstdml_collective_b200", f"-Wl,-rpath,{libdir}", "-lpthread"], check=True)


def build(reference, out_bin):
    scratch = tempfile.mkdtemp(prefix="ref_resize_")
    src = os.path.join(scratch, "src")
    shutil.copytree(reference, src)
    bdir = os.path.join(src, "build")
    os.makedirs(bdir)
    subprocess.run(["cmake", "..", "-DCMAKE_BUILD_TYPE=Release", "-DBUILD_TESTS=OFF",
                    "-DBUILD_BENCHMARKS=OFF", "-DBUILD_EXAMPLES=OFF"], cwd=bdir, check=True,
                   stdout=subprocess.DEVNULL)
    subprocess.run(["make", "-j8"], cwd=bdir, check=True, stdout=subprocess.DEVNULL)
    libs = [os.path.join(dp, f) for dp, _, fs in os.walk(bdir) for f in fs
            if f.endswith(".a") or (f.endswith(".so") and "stdml" in f)]
    if not libs:
        raise SystemExit("the reference build produced no library")
    os.makedirs(os.path.dirname(out_bin), exist_ok=True)
    subprocess.run(["g++", "-std=c++17", "-O2", "-pthread", "-I", os.path.join(src, "include"),
                    os.path.join(HERE, "resize_driver.cpp"), "-o", out_bin] + libs +
                   ["-lpthread"], check=True)
    shutil.rmtree(scratch, ignore_errors=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--schedule", default="8,4,6,8")
    ap.add_argument("--reference", default=os.environ.get("STDML_REFERENCE_SRC", ""),
                    help="source tree of the reference implementation (or $STDML_REFERENCE_SRC)")
    ap.add_argument("--impl", default="reference", choices=["reference", "ours"])
    args = ap.parse_args()
    sizes = [int(x) for x in args.schedule.split(",")]
    if args.impl == "ours":
        binary = os.path.join(HERE, "_ref", "bin", "ours-resize-driver")
        build_ours(binary)
    else:
        binary = os.path.join(HERE, "_ref", "bin", "ref-resize-driver")
        if not os.path.exists(binary):
            if not os.path.isdir(args.reference):
                print(json.dumps({"impl": "reference",
                                  "unavailable": "reference sources not found at " + args.reference}))
                return 0
            build(args.reference, binary)
    top = max(sizes)
    # The OpenMPI variables give a membership without runners (ports 10000 + rank,
    # star graph): with no runner to notify, committing a new configuration is
    # purely local, which is what lets the resize run without the Go launcher.
    addr = [f"127.0.0.1:{10000 + i}" for i in range(top)]
    tmp = tempfile.mkdtemp(prefix="ref_resize_run_")
    cfg = os.path.join(tmp, "cluster.txt")

    def write_cfg(n):
        with open(cfg + ".new", "w") as f:
            f.write(",".join(addr[:n]) + "\n")
        os.replace(cfg + ".new", cfg)

    def start(i, n, version):
        env = dict(os.environ, REF_RESIZE_CONFIG=cfg)
        for k in ("KUNGFU_SELF_SPEC", "KUNGFU_INIT_PEERS", "RANK", "WORLD_SIZE",
                  "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_RANK"):
            env.pop(k, None)
        if args.impl == "reference":
            env.update(OMPI_COMM_WORLD_SIZE=str(n), OMPI_COMM_WORLD_RANK=str(i))
        else:
            # this library's message names carry the cluster version, so a joiner has
            # to be told which membership it joins (the reference's names do not)
            env.update(KUNGFU_SELF_SPEC=addr[i], KUNGFU_INIT_PEERS=",".join(addr[:n]),
                       KUNGFU_INIT_RUNNERS="", KUNGFU_INIT_CLUSTER_VERSION=str(version),
                       KUNGFU_ALLREDUCE_STRATEGY="STAR")
        return subprocess.Popen([binary, "400"], env=env, stdout=subprocess.PIPE,
                                stderr=subprocess.DEVNULL, text=True)

    write_cfg(sizes[0])
    procs = {i: start(i, sizes[0], 0) for i in range(sizes[0])}
    time.sleep(1.0)
    cur = sizes[0]
    for version, n in enumerate(sizes[1:], start=1):
        write_cfg(n)
        for i in range(cur, n):  # joiners know the new membership from the start
            procs[i] = start(i, n, version)
        time.sleep(2.5)
        cur = n
    time.sleep(1.0)
    text = ""
    deadline = time.time() + 60
    for i, p in procs.items():
        try:
            out, _ = p.communicate(timeout=max(1, deadline - time.time()))
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        text += out
    shutil.rmtree(tmp, ignore_errors=True)
    events = [{"from": int(a), "to": int(b), "ms": float(ms)}
              for a, b, ms in re.findall(r"resized (\d+) -> (\d+) ([0-9.]+) ms", text)]
    print(json.dumps({"impl": args.impl, "what": "peer::resize(sess, config_provider) on CPU ranks "
                      "over TCP loopback, file-backed configuration, joiners started by this script",
                      "schedule": sizes, "strategy": "STAR", "resizes": events,
                      "finished": "finished size" in text}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
