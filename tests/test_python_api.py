"""Python host API over the native runtime: ranks are real processes on TCP loopback."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def collect(procs, timeout):
    """Outputs of all processes; none of them is left behind if one hangs."""
    try:
        return [p.communicate(timeout=timeout)[0] for p in procs]
    except subprocess.TimeoutExpired:
        for p in procs:
            if p.poll() is None:
                p.kill()
        raise



@pytest.mark.parametrize("n,strategy,base", [(1, "star", 12100), (3, "star", 12110),
                                             (4, "ring", 12120), (3, "clique", 12130)])
def test_python_peer_session(n, strategy, base, native_lib):
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "py_rank_worker.py"), str(r),
                               str(n), str(base), strategy], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(n)]
    outs = collect(procs, 300)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} OK" in o, o[-2000:]


def test_ranks_with_different_transports_meet(native_lib):
    """Ranks 0 and 2 take the default (UNIX socket + shared-memory ring for same-host peers,
    TCP when that does not answer), rank 1 speaks and listens on TCP only, rank 3 insists on
    plain UNIX sockets: every pair still connects, in both directions."""
    n, base = 4, 12180
    modes = {1: "tcp", 3: "unix"}
    procs = []
    for r in range(n):
        env = dict(os.environ)
        env.pop("STDML_COLLECTIVE_TRANSPORT", None)
        if r in modes:
            env["STDML_COLLECTIVE_TRANSPORT"] = modes[r]
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "py_rank_worker.py"),
                                       str(r), str(n), str(base), "ring"], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = collect(procs, 300)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} OK" in o, o[-2000:]


def test_resnet50_gradient_set_over_a_ring_of_four(native_lib):
    """The "CPU plumbing" acceptance case, as specified: 4 processes, ring, the 161
    f32 tensors of ResNet-50, N(0, 1) values seeded per rank, against a host sum."""
    n, base = 4, 12170
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "config1_worker.py"), str(r),
                               str(n), str(base)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(n)]
    outs = collect(procs, 600)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} OK" in o, o[-2000:]


@pytest.mark.parametrize("strategy,base", [("star", 12140), ("ring", 12150)])
def test_python_peer_failure_is_an_exception(strategy, base, native_lib):
    n = 3
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "py_fail_worker.py"), str(r),
                               str(n), str(base), strategy], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(n)]
    outs = collect(procs, 300)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o[-2000:]
        if r != 1:
            assert f"rank {r} OK" in o, o[-2000:]


def test_python_elastic_state_under_the_runner(native_lib):
    from stdml_collective_experimental_b200 import _native
    _native.build()
    runner = os.path.join(_native.CSRC, "build", "bin", "stdml_collective_run")
    cmd = [runner, "-q", "-np", "2", "-w", "-builtin-config-port", "0", "-runner-port", "38282",
           "-port-range", "10500", sys.executable, os.path.join(HERE, "py_elastic_worker.py"),
           "8", "2:3", "5:2"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stdout[-3000:]
    assert res.stdout.count("weight 36.0 OK") == 2 and res.stdout.count("detached") == 1


def test_python_elastic_growth_takes_warm_standbys(native_lib):
    """-spares 2: the launcher keeps two copies of the worker program warm (run up to
    Peer.from_env()); a growth hands them their identities instead of starting processes,
    and standbys that were never needed end quietly with the job."""
    from stdml_collective_experimental_b200 import _native
    runner = os.path.join(_native.CSRC, "build", "bin", "stdml_collective_run")
    cmd = [runner, "-np", "2", "-w", "-spares", "2", "-builtin-config-port", "0", "-runner-port",
           "38286", "-port-range", "10560", sys.executable,
           os.path.join(HERE, "py_elastic_worker.py"), "30", "--report", "--step-ms=250",
           "16:4", "24:3"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         timeout=600)
    out = res.stdout
    assert res.returncode == 0, out[-3000:]
    assert out.count("becomes worker") == 2, out[-3000:]        # both joiners were standbys
    assert out.count("started worker") == 2, out[-3000:]        # only the first two were started cold
    assert out.count("weight 465.0 OK") == 3 and out.count("detached") == 1, out[-3000:]
    took = [float(line.split("took")[1].split()[0]) for line in out.splitlines()
            if line.startswith("resize 2 -> 4")]
    assert len(took) == 1
    print("growth with warm standbys took", took[0], "ms")


def test_python_elastic_growth_survives_dead_standbys(native_lib):
    """Standbys that ended during their warm-up are skipped: the joiners are started cold."""
    from stdml_collective_experimental_b200 import _native
    runner = os.path.join(_native.CSRC, "build", "bin", "stdml_collective_run")
    cmd = [runner, "-np", "2", "-w", "-spares", "1", "-builtin-config-port", "0", "-runner-port",
           "38288", "-port-range", "10580", sys.executable,
           os.path.join(HERE, "py_elastic_worker.py"), "12", "--standby-dies", "--step-ms=100",
           "6:3"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         timeout=600)
    out = res.stdout
    assert res.returncode == 0, out[-3000:]
    assert out.count("becomes worker") == 0 and out.count("started worker") == 3, out[-3000:]
    assert out.count("weight 78.0 OK") == 3, out[-3000:]


def test_python_elastic_state_recovers_from_a_crash(native_lib):
    from stdml_collective_experimental_b200 import _native
    runner = os.path.join(_native.CSRC, "build", "bin", "stdml_collective_run")
    cmd = [runner, "-q", "-np", "3", "-w", "-builtin-config-port", "0", "-runner-port", "38284",
           "-port-range", "10540", sys.executable, os.path.join(HERE, "py_elastic_worker.py"),
           "8", "--die=10541:3"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         timeout=600)
    assert res.returncode == 1, res.stdout[-3000:]  # the runner counts the crashed worker
    assert res.stdout.count("weight 36.0 OK") == 2 and res.stdout.count("lost 1 member(s)") == 2


@pytest.mark.parametrize("strategy,port", [("STAR", 29871), ("RING", 29873)])
def test_torch_distributed_backend_and_ddp(strategy, port, native_lib):
    n = 3
    env = dict(os.environ, KUNGFU_ALLREDUCE_STRATEGY=strategy)
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "pg_worker.py"), str(r), str(n),
                               str(port)], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(n)]
    outs = collect(procs, 300)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} OK" in o, o[-2000:]


def test_distributed_optimizer_matches_single_process_training(native_lib):
    n, base = 3, 12200
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "py_train_worker.py"), str(r),
                               str(n), str(base)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(n)]
    outs = collect(procs, 300)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} OK" in o, o[-2000:]


def test_resize_latency_harness_on_this_library(native_lib):
    """The driver that times peer::resize(sess, config_provider) for both
    implementations, compiled against this library: shrink 4 -> 2, grow 2 -> 3."""
    import json
    root = os.path.dirname(HERE)
    res = subprocess.run([sys.executable, os.path.join(root, "baseline", "measure_resize.py"),
                          "--impl", "ours", "--schedule", "4,2,3"], stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["finished"] and [(e["from"], e["to"]) for e in line["resizes"]] == [(4, 2), (2, 3)]
    assert all(e["ms"] < 2000 for e in line["resizes"])
