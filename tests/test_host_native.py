"""CPU tests of the native host runtime: builds the C++ test programs and runs
them (ranks are real processes on TCP loopback, forked by the programs)."""
import os
import shutil
import subprocess

import pytest

from stdml_collective_experimental_b200 import _native

BIN = os.path.join(_native.CSRC, "build", "bin")


def collect(procs, timeout):
    """Outputs of all processes; none of them is left behind if one hangs."""
    try:
        return [p.communicate(timeout=timeout)[0] for p in procs]
    except subprocess.TimeoutExpired:
        for p in procs:
            if p.poll() is None:
                p.kill()
        raise



@pytest.fixture(scope="module", autouse=True)
def built():
    _native.build()


def run(prog, *args, env=None, timeout=600, want_rc=0):
    e = dict(os.environ)
    for k in ("KUNGFU_SELF_SPEC", "OMPI_COMM_WORLD_SIZE", "RANK", "WORLD_SIZE"):
        e.pop(k, None)
    e.update(env or {})
    res = subprocess.run([os.path.join(BIN, prog), *map(str, args)], env=e, timeout=timeout,
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == want_rc, res.stdout[-3000:]
    return res.stdout


def test_unit():
    assert "test-unit: OK" in run("test_unit")


@pytest.mark.parametrize("np_", [1, 2, 3, 4])
def test_collectives_star(np_):
    assert f"np={np_}: OK" in run("test_collectives", np_)


@pytest.mark.parametrize("env", [
    {"KUNGFU_ALLREDUCE_STRATEGY": "RING"},
    {"KUNGFU_ALLREDUCE_STRATEGY": "RING", "STDML_COLLECTIVE_USE_THREAD_POOL": "1"},
    {"KUNGFU_ALLREDUCE_STRATEGY": "RING", "STDML_COLLECTIVE_USE_ASYNC": "1"},
    {"STDML_COLLECTIVE_USE_ASYNC": "1"},
    {"STDML_COLLECTIVE_USE_THREAD_POOL": "1"},
    {"KUNGFU_ALLREDUCE_STRATEGY": "RING", "STDML_COLLECTIVE_TRANSPORT": "unix"},
    {"STDML_COLLECTIVE_TRANSPORT": "unix", "STDML_COLLECTIVE_USE_ASYNC": "1"},
    {"KUNGFU_ALLREDUCE_STRATEGY": "RING", "STDML_COLLECTIVE_TRANSPORT": "shm"},
    {"STDML_COLLECTIVE_TRANSPORT": "shm", "STDML_COLLECTIVE_USE_ASYNC": "1"},
    # a ring far smaller than the 1 MB chunks: every body goes through in pieces
    {"KUNGFU_ALLREDUCE_STRATEGY": "RING", "STDML_COLLECTIVE_TRANSPORT": "shm",
     "STDML_COLLECTIVE_SHM_RING_MB": "1"},
], ids=["ring", "ring-pool", "ring-async", "star-async", "star-pool", "ring-unix-sockets",
        "star-async-unix-sockets", "ring-shm", "star-async-shm", "ring-shm-small-ring"])
def test_collectives_strategies_and_runtimes(env):
    assert "np=4: OK" in run("test_collectives", 4, env=env)


def test_collectives_eight_ranks_ring():
    assert "np=8: OK" in run("test_collectives", 8, env={"KUNGFU_ALLREDUCE_STRATEGY": "RING"})


def launch(np_, prog, *args, flags=(), timeout=300):
    return run("stdml_collective_run", "-q", "-np", np_, *flags, os.path.join(BIN, prog), *args,
               timeout=timeout)


def test_examples_under_the_launcher():
    assert "sum: 6 10 14" in launch(4, "example_1")
    assert launch(3, "example_collective").count("OK") == 3
    assert "came back as 103" in launch(4, "example_send_recv")
    assert launch(2, "example_mpi").count("OK") == 2
    assert run("example_fork", 3).count("total 6") == 3
    lines = run("example_task").split()
    assert sorted(lines) == ["11", "12", "21", "22"]
    assert lines.index("11") < lines.index("12") and lines.index("21") < lines.index("22")
    assert run("example_rchan").count("hello") == 3
    out = run("example_recover", 4, 2, 3)
    assert "example-recover: OK" in out and out.count("done: 3 members, version 1") == 3


def test_mpi_env_launch_path():
    # OMPI_COMM_WORLD_* is a launch path of its own (star, ports 10000 + rank)
    procs = []
    for r in range(2):
        e = dict(os.environ, OMPI_COMM_WORLD_SIZE="2", OMPI_COMM_WORLD_RANK=str(r))
        e.pop("KUNGFU_SELF_SPEC", None)
        procs.append(subprocess.Popen([os.path.join(BIN, "example_mpi")], env=e,
                                      stdout=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs) and all("OK" in o for o in outs)


def test_benchmarks_run_and_verify():
    out = launch(4, "bench_all_reduce", "1024x20", 2, 1, flags=("-strategy", "RING"))
    assert "FINAL RESULT: 1024x20" in out and "RING" in out
    # 300 tensors in rank-rotated order with late futures: must not deadlock
    out = launch(4, "bench_group_all_reduce", "512x300", 2, 1, flags=("-strategy", "RING"))
    assert "verified" in out
    assert "GiB/s" in launch(2, "bench_mpi_all_reduce", 10, 256, 2)


def test_elastic_resize_schedule_with_state_broadcast():
    # 4 -> 2 -> 3 -> 4 workers; survivors keep running, joiners get step and state
    out = run("stdml_collective_run", "-np", 4, "-w", "-builtin-config-port", 0,
              os.path.join(BIN, "example_elastic"), "--max-step=12", "3:2", "6:3", "9:4",
              timeout=300)
    assert out.count("weight 78.0 (want 78.0) OK") == 4
    assert out.count("detached after step 3") == 2
    for v in (1, 2, 3):
        assert f"[runner] version {v}" in out


def test_elastic_job_over_two_emulated_hosts():
    # two "hosts" (loopback aliases), one runner each, same command line except -self:
    # 4 -> 2 workers empties the second host (its runner stays), 3 and 4 grow back onto it
    common = ["-H", "127.0.0.2:2,127.0.0.3:2", "-np", "4", "-w", "-builtin-config-port", "38393",
              "-port-range", "10820", "-runner-port", "38392"]
    prog = [os.path.join(BIN, "example_elastic"), "--max-step=12", "3:2", "6:3", "9:4"]
    e = dict(os.environ)
    for k in ("KUNGFU_SELF_SPEC", "OMPI_COMM_WORLD_SIZE", "RANK", "WORLD_SIZE"):
        e.pop(k, None)
    procs = [subprocess.Popen([os.path.join(BIN, "stdml_collective_run"), *common, "-self", ip,
                               *prog], env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True) for ip in ("127.0.0.2", "127.0.0.3")]
    outs = collect(procs, 300)
    assert all(p.returncode == 0 for p in procs), outs
    assert outs[0].count("weight 78.0 (want 78.0) OK") == 2, outs[0]
    assert outs[1].count("weight 78.0 (want 78.0) OK") == 2, outs[1]
    assert outs[1].count("detached after step 3") == 2
    assert "[runner] started worker 127.0.0.3:10820" in outs[1]  # grown back, same port range


def test_two_level_all_reduce_over_uneven_emulated_hosts():
    # 3 ranks on one "host", 2 on the other: reduce inside each host, all-reduce
    # among the two leaders, broadcast inside each host
    common = ["-q", "-H", "127.0.0.2:3,127.0.0.3:2", "-np", "5", "-port-range", "10840",
              "-runner-port", "38394", "-env", "STDML_COLLECTIVE_HIERARCHICAL=1"]
    e = dict(os.environ)
    for k in ("KUNGFU_SELF_SPEC", "OMPI_COMM_WORLD_SIZE", "RANK", "WORLD_SIZE"):
        e.pop(k, None)
    procs = [subprocess.Popen([os.path.join(BIN, "stdml_collective_run"), *common, "-self", ip,
                               os.path.join(BIN, "test_two_level")], env=e,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for ip in ("127.0.0.2", "127.0.0.3")]
    outs = collect(procs, 300)
    assert all(p.returncode == 0 for p in procs), outs
    assert outs[0].count("/5: OK") == 3 and outs[1].count("/5: OK") == 2, outs


def test_launcher_stops_its_workers_when_it_is_told_to_stop():
    import signal
    import time
    p = subprocess.Popen([os.path.join(BIN, "stdml_collective_run"), "-np", "3", "-port-range",
                          "10860", "-runner-port", "38396", "sleep", "300"],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    kids = []
    for _ in range(100):  # wait for the three workers
        out = subprocess.run(["pgrep", "-P", str(p.pid)], stdout=subprocess.PIPE, text=True).stdout
        kids = [int(x) for x in out.split()]
        if len(kids) == 3:
            break
        time.sleep(0.05)
    assert len(kids) == 3
    p.send_signal(signal.SIGTERM)
    out = p.communicate(timeout=30)[0]
    assert p.returncode == 1 and "stopping 3 workers" in out, out
    for k in kids:  # reaped: no such process any more
        with pytest.raises(ProcessLookupError):
            os.kill(k, 0)


def test_elastic_state_follows_config_server():
    out = run("stdml_collective_run", "-q", "-np", 2, "-w", "-builtin-config-port", 0,
              os.path.join(BIN, "example_elastic_state"), "--max-step=9", "2:4", "5:3",
              timeout=300)
    assert out.count("weight 45.0 (want 45.0) OK") == 3 and out.count("detached") == 1


def test_elastic_growth_from_warm_standbys_cxx_workers():
    # -spares 2: the joiners of both growth steps are standbys that waited in
    # peer::from_env(); nothing but the first two workers is started cold, and the
    # standbys that were never used end with the job
    out = run("stdml_collective_run", "-np", 2, "-w", "-spares", 2, "-builtin-config-port", 0,
              "-runner-port", 38387, "-port-range", 10640, os.path.join(BIN, "example_elastic"),
              "--max-step=12", "3:2", "6:3", "9:4", timeout=300)
    assert out.count("becomes worker") == 2 and out.count("started worker") == 2, out
    assert out.count("weight 78.0 (want 78.0) OK") == 4, out


def test_elastic_state_survives_a_crash_and_grows_back():
    # the worker on port 10601 dies at step 3; the others recover (version 1, two
    # members), rank 0 asks for three again at step 6 and the runner starts a
    # replacement, which receives progress and state.  The runner reports the
    # crashed worker in its exit status.
    out = run("stdml_collective_run", "-np", 3, "-w", "-builtin-config-port", 0, "-runner-port", 38385,
              "-port-range", 10600, os.path.join(BIN, "example_elastic_state"), "--max-step=9",
              "--die=10601:3", "6:3", timeout=300, want_rc=1)
    assert out.count("weight 45.0 (want 45.0) OK") == 3, out
    assert out.count("lost 127.0.0.1:10601, carrying on with 2 members") == 2
    assert "[runner] version 1 : 3 -> 2 workers" in out and "[runner] version 2 : 2 -> 3 workers" in out


def test_failure_detection_with_the_tree_strategy():
    # chunks of one tensor use trees with different roots, so a rank may wait for a
    # peer that has never sent it anything: the established-session ping covers that
    assert "np=5: OK" in run("test_shutdown", 5, env={"KUNGFU_ALLREDUCE_STRATEGY": "BINARY_TREE"})


def test_failure_detection_with_the_clique_strategy():
    # a star per rank: every rank is a root for some chunks and a leaf for the others
    assert "np=4: OK" in run("test_shutdown", 4, env={"KUNGFU_ALLREDUCE_STRATEGY": "CLIQUE"})


def test_shutdown_and_host_side_failure_detection():
    # clean teardown after 100 collectives; a rank that leaves between steps and a rank
    # that never joins both end in exceptions on the others, not in a hang
    assert "test-shutdown np=3: OK" in run("test_shutdown", 3)


def test_local_rendezvous_mesh_descriptor_passing_and_timeouts():
    # the side channel of the device world set-up (UNIX sockets, SCM_RIGHTS) needs no GPU
    assert "test-rendezvous: OK" in run("test_rendezvous", 4)


def test_public_headers_compile_as_cxx17():
    run("test_cxx17")


@pytest.mark.parametrize("np_,strategy", [(16, "STAR"), (16, "RING"), (7, "RING"),
                                          (4, "BINARY_TREE"), (7, "BINARY_TREE"),
                                          (16, "BINARY_TREE"), (4, "CLIQUE"), (7, "CLIQUE")])
def test_collectives_many_ranks(np_, strategy):
    # the reference's CI sweeps np = 1..16 (t:37-57 there)
    assert f"np={np_}: OK" in run("test_collectives", np_,
                                  env={"KUNGFU_ALLREDUCE_STRATEGY": strategy})


def test_host_runtime_under_address_and_thread_sanitizers():
    """The host runtime rebuilt with -fsanitize=address / thread must run the unit
    and integration programs without a report (compute-sanitizer's job for the
    device code is done by exhaustive small cases against the CPU oracle)."""
    if not os.path.exists("/usr/lib/gcc/x86_64-linux-gnu/13/libasan.so"):
        pytest.skip("sanitizer runtimes not installed")
    for san, opts in (("address", {"ASAN_OPTIONS": "detect_leaks=1:protect_shadow_gap=0"}),
                      ("thread", {"TSAN_OPTIONS": "report_thread_leaks=0"})):
        res = subprocess.run(["make", "-C", _native.CSRC, "-j8", "sanitize", f"SAN={san}"],
                             stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        assert res.returncode == 0, res.stdout[-3000:]
        sdir = os.path.join(_native.CSRC, "build", f"san-{san}", "bin")
        for prog, args, extra in (("test_unit", [], {}), ("test_collectives", ["3"], {}),
                                  ("test_shutdown", ["3"], {}), ("test_rendezvous", ["3"], {}),
                                  ("test_collectives", ["3"], {"STDML_COLLECTIVE_TRANSPORT": "shm"}),
                                  ("test_shutdown", ["3"], {"STDML_COLLECTIVE_TRANSPORT": "shm"})):
            e = dict(os.environ, **opts, **extra)
            for k in ("KUNGFU_SELF_SPEC", "OMPI_COMM_WORLD_SIZE", "RANK", "WORLD_SIZE"):
                e.pop(k, None)
            out = subprocess.run([os.path.join(sdir, prog), *args], env=e, stdout=subprocess.PIPE,
                                 stderr=subprocess.STDOUT, text=True, timeout=900)
            assert out.returncode == 0, (san, prog, out.stdout[-3000:])
            assert "Sanitizer" not in out.stdout, (san, prog, out.stdout[-3000:])
        shutil.rmtree(os.path.join(_native.CSRC, "build", f"san-{san}"), ignore_errors=True)


def test_elastic_agreement_with_stale_and_failing_config_providers():
    assert "test-elastic: OK" in run("test_elastic")


def test_standalone_config_server_get_put():
    import json
    import time
    import urllib.request
    srv = subprocess.Popen([os.path.join(BIN, "stdml_collective_config_server"), "-port", "19191",
                            "-ttl", "20"], stdout=subprocess.PIPE, text=True)
    try:
        assert "config server on" in srv.stdout.readline()
        url = "http://127.0.0.1:19191/config"
        assert json.loads(urllib.request.urlopen(url, timeout=5).read()) == {"Runners": [],
                                                                             "Workers": []}
        good = {"Runners": [{"IPv4": 2130706433, "Port": 38080}],
                "Workers": [{"IPv4": 2130706433, "Port": 10000}]}
        req = urllib.request.Request(url, data=json.dumps(good).encode(), method="PUT")
        assert json.loads(urllib.request.urlopen(req, timeout=5).read()) == good
        assert json.loads(urllib.request.urlopen(url, timeout=5).read()) == good
        bad = urllib.request.Request(url, data=b"{nope", method="PUT")
        with pytest.raises(urllib.error.HTTPError):
            urllib.request.urlopen(bad, timeout=5)
        time.sleep(0.05)
    finally:
        srv.terminate()
        srv.wait(timeout=10)


def test_kernel_index_arithmetic_on_the_cpu():
    # span partition and descriptor-table search of the device kernels, compiled for the host
    assert "test-partition: OK" in run("test_partition_cuda")
