"""CPU tests of the native host runtime: builds the C++ test programs and runs
them (ranks are real processes on TCP loopback, forked by the programs)."""
import os
import subprocess

import pytest

from stdml_collective_experimental_b200 import _native

BIN = os.path.join(_native.CSRC, "build", "bin")


@pytest.fixture(scope="module", autouse=True)
def built():
    _native.build()


def run(prog, *args, env=None, timeout=600):
    e = dict(os.environ)
    for k in ("KUNGFU_SELF_SPEC", "OMPI_COMM_WORLD_SIZE", "RANK", "WORLD_SIZE"):
        e.pop(k, None)
    e.update(env or {})
    res = subprocess.run([os.path.join(BIN, prog), *map(str, args)], env=e, timeout=timeout,
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout[-3000:]
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
], ids=["ring", "ring-pool", "ring-async", "star-async", "star-pool"])
def test_collectives_strategies_and_runtimes(env):
    assert "np=4: OK" in run("test_collectives", 4, env=env)


def test_collectives_eight_ranks_ring():
    assert "np=8: OK" in run("test_collectives", 8, env={"KUNGFU_ALLREDUCE_STRATEGY": "RING"})
