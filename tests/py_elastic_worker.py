"""A worker of the Python ElasticState test (started by the native runner)."""
import os
import sys

if "--standby-dies" in sys.argv and os.environ.get("STDML_COLLECTIVE_STANDBY_FD"):
    sys.exit(0)  # a standby that does not survive its warm-up (gone long before the job grows)

import torch  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from stdml_collective_experimental_b200 import PeerFailure  # noqa: E402
from stdml_collective_experimental_b200.parallel.elastic import ElasticState  # noqa: E402
from stdml_collective_experimental_b200.parallel.peer import resized_cluster  # noqa: E402
import json  # noqa: E402
import time  # noqa: E402
import urllib.request  # noqa: E402


def propose(sess, new_size):
    body = json.dumps(resized_cluster(sess.cluster, new_size)).encode()
    req = urllib.request.Request(os.environ["KUNGFU_CONFIG_SERVER"], data=body, method="PUT")
    urllib.request.urlopen(req, timeout=5).read()


def main():
    max_step = int(sys.argv[1])
    args = sys.argv[2:]
    die = [a[len("--die="):].split(":") for a in args if a.startswith("--die=")]
    die_port, die_step = (int(die[0][0]), int(die[0][1])) if die else (-1, -1)
    schedule = dict(tuple(map(int, a.split(":"))) for a in args if not a.startswith("--"))
    step_ms = [int(a[len("--step-ms="):]) for a in args if a.startswith("--step-ms=")]
    report = "--report" in args
    weights = torch.zeros(256)
    state = ElasticState(max_progress=max_step)
    state.on_resize(lambda s: s.broadcast(weights, name="state", root=state.state_root))
    my_port = int(state.peer.self_id.split(":")[1])
    while not state.should_stop():
        try:
            step = int(state)
            if step == die_step and my_port == die_port:
                os._exit(3)  # an unplanned loss
            g = torch.full((256,), float(step + 1))
            state.sess.all_reduce(g, name="grad")
            weights += g / state.sess.size
            if state.sess.rank == 0 and step in schedule:
                propose(state.sess, schedule[step])
            if step_ms:
                time.sleep(step_ms[0] * 1e-3)  # stands for the compute of a step
            before = state.sess.size
            state.advance()
            if report and not state.detached and state.sess.size != before and state.sess.rank == 0:
                print(f"resize {before} -> {state.sess.size} took {state.last_resize_ms:.0f} ms",
                      flush=True)
        except PeerFailure:
            print(f"lost {state.recover()} member(s)", flush=True)
    if state.detached:
        print("detached", flush=True)
        return
    want = max_step * (max_step + 1) / 2
    ok = float(weights[0]) == want
    print(f"finished rank {state.sess.rank}/{state.sess.size} weight {float(weights[0])} "
          f"{'OK' if ok else 'WRONG'}", flush=True)
    state.close()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
