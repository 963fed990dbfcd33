"""`python -m stdml_collective_experimental_b200.run -np 4 [-w ...] prog [args...]`

Front door of the native launcher (csrc/apps/stdml_collective_run.cpp): builds
it on first use and replaces this process with it.  Same flags as the binary:
-np N, -strategy STAR|RING, -w, -builtin-config-port P, -config-server URL,
-logdir DIR, -q, -runner-port P, -port-range P, -env K=V.  The reference is
started with KungFu's `kungfu-run` (scripts/bin/stdml-collective-run:15-53 there).
"""
import os
import sys

from . import _native


def runner_path():
    path = os.path.join(_native.CSRC, "build", "bin", "stdml_collective_run")
    if not os.path.exists(path):
        _native.build()
    return path


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    path = runner_path()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ)
    env["PYTHONPATH"] = root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    os.execve(path, [path] + argv, env)


if __name__ == "__main__":
    main()
