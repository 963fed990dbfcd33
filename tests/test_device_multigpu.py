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


def run_world(n, port, extra_env=None, timeout=600, worker="multigpu_worker.py"):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, worker)]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         timeout=timeout)
    assert res.returncode == 0, res.stdout[-4000:]
    assert res.stdout.count("OK rank") == n, res.stdout[-4000:]
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
