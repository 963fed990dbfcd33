"""Real multi-GPU runs of the device collectives: one process per GPU under
torchrun, peer memory mapped through the VMM/IPC manager, NVLS when the box
has it.  Skipped on boxes with a single GPU (the loopback tests cover the
kernels there)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


# These tests are about the device plane.  Their host control plane runs over TCP loopback,
# the transport they were validated with on GPU boxes; the transport that the host path
# picks by itself is covered by the CPU tests.
CONTROL_PLANE = {"STDML_COLLECTIVE_TRANSPORT": os.environ.get("STDML_COLLECTIVE_TRANSPORT", "tcp")}


def run_world(n, port, extra_env=None, timeout=600, worker="multigpu_worker.py"):
    env = dict(os.environ, **CONTROL_PLANE)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, worker)]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         timeout=timeout)
    if res.returncode != 0 or res.stdout.count("OK rank") != n:
        # the workers' own tracebacks come long before the launcher's epilogue
        lines = res.stdout.splitlines()
        first = next((i for i, line in enumerate(lines) if "Traceback" in line), max(0, len(lines) - 60))
        raise AssertionError("\n".join(lines[first:first + 60]) + "\n...\n" + res.stdout[-1500:])
    return res.stdout


@pytest.mark.parametrize("n", [2, 4, 8])
def test_multigpu_world(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    out = run_world(n, 29610 + n)
    print(out[-600:])


def test_multigpu_ipc_backend_without_nvls():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_world(2, 29631, {"STDML_COLLECTIVE_SYMM": "ipc", "STDML_COLLECTIVE_NVLS": "0"})


def test_data_parallel_matches_single_process_training():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_world(2, 29641, worker="ddp_worker.py")


def test_torch_distributed_backend_on_cuda_tensors():
    """Backend "stdml" of torch.distributed with CUDA tensors on two GPUs: the
    collectives run on this library's kernels, DistributedDataParallel trains."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    n, port = 2, 29881
    env = dict(os.environ, STDML_COLLECTIVE_BASE_PORT="10900", **CONTROL_PLANE)
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "pg_worker.py"), str(r), str(n),
                               str(port), "cuda"], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(n)]
    try:
        outs = [p.communicate(timeout=300)[0] for p in procs]
    except subprocess.TimeoutExpired:
        for p in procs:
            if p.poll() is None:
                p.kill()
        raise
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} OK" in o, o[-3000:]


def test_elastic_resize_on_gpus():
    """2 -> 1 -> 2 workers with CUDA tensors through Peer/Session: every membership
    gets a fresh device world (arenas, mappings, multicast); the survivor keeps
    its process; the joiner catches up (step by max, state by broadcast)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    root = os.path.dirname(HERE)
    runner = os.path.join(root, "stdml_collective_experimental_b200", "csrc", "build", "bin",
                          "stdml_collective_run")
    if not os.path.exists(runner):
        from stdml_collective_experimental_b200 import _native
        _native.build()
    # a rank leaves between steps: no multicast binding may be live then, neither
    # NCCL's nor the library's own
    env = dict(os.environ, PYTHONPATH=root, NCCL_NVLS_ENABLE="0", STDML_COLLECTIVE_NVLS="0",
               **CONTROL_PLANE)
    cmd = [runner, "-q", "-np", "2", "-w", "-builtin-config-port", "0", "-runner-port", "38181",
           "-port-range", "10300", sys.executable, "-m",
           "stdml_collective_experimental_b200.benchmarks.elastic", "--model", "resnet50",
           "--max-step", "12", "--schedule", "3:1,7:2", "--state-mb", "1"]
    res = subprocess.run(cmd, env=env, cwd=root, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                         text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-4000:]
    assert '"event": "detached"' in res.stdout
    assert res.stdout.count('"event": "resized"') == 2
    assert '"weights_ok": true' in res.stdout and '"size": 2, "version": 2' in res.stdout
