"""Python host API over the native runtime: ranks are real processes on TCP loopback."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("n,strategy,base", [(1, "star", 12100), (3, "star", 12110),
                                             (4, "ring", 12120)])
def test_python_peer_session(n, strategy, base, native_lib):
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "py_rank_worker.py"), str(r),
                               str(n), str(base), strategy], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(n)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} OK" in o, o[-2000:]
