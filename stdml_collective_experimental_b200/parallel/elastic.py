"""ElasticState for Python training loops: progress that survives membership
changes, the counterpart of the reference's C++ `elastic_state`
(include/stdml/bits/collective/elastic_state.hpp:8-38):

    state = ElasticState(max_progress=1000)
    state.on_resize(lambda sess: sess.broadcast(weights, root=state.state_root))
    while not state.should_stop():
        train_step(state.sess)
        state.advance()                                     # checks for a resize

`advance()` asks the config server (KUNGFU_CONFIG_SERVER) after every step; when
the membership changed, survivors get a new session in place, the progress
counter becomes the maximum over the new members and the resize hook runs
(joiners run it at their first use of the state).  A removed rank sees
`should_stop()` become true.  An unplanned loss surfaces as `PeerFailure`;
`state.recover()` then rebuilds the session from the members that still answer.
"""
import time

import torch

from .peer import Peer


class ElasticState:
    def __init__(self, max_progress=None, peer=None, get_cluster=None):
        """get_cluster: optional callable returning the wanted {"Runners", "Workers"}
        dict (or None for "no change"); default: follow the config server."""
        self.peer = Peer.from_env() if peer is None else peer
        self.sess = self.peer.join()
        self.max_progress = max_progress
        self.progress = 0
        self.detached = False
        self.last_resize_ms = None  # duration of the last advance() that changed the membership
        self._synced = False
        self._needs_state = self.sess.version > 0  # joined a running job
        self._hook = None
        self._get_cluster = get_cluster
        self.state_root = 0  # the rank whose state the resize hook should broadcast

    def on_resize(self, fn):
        self._hook = fn

    def _sync(self):
        if not self._synced:
            mine = torch.tensor([self.progress], dtype=torch.int64)
            t = mine.clone()
            self.progress = int(self.sess.all_reduce(t, op="max", name="stdml::progress").item())
            self._synced = True
            if self._needs_state:
                self._needs_state = False
                # the lowest rank that is as far as anyone holds the state to copy: rank 0
                # after a planned resize, possibly another one after a loss (the step in
                # flight may have finished on some members only)
                everyone = torch.empty(self.sess.size, dtype=torch.int64)
                self.sess.all_gather(mine, everyone, name="stdml::progress")
                self.state_root = int((everyone == self.progress).nonzero()[0].item())
                if self._hook is not None:
                    self._hook(self.sess)

    def __int__(self):
        self._sync()
        return self.progress

    def advance(self):
        self._sync()
        self.progress += 1
        t0 = time.perf_counter()
        if self._get_cluster is not None:
            wanted = self._get_cluster()
            if wanted is None:
                wanted = self.sess.cluster
            changed, detached = self.peer.resize(self.sess, cluster=wanted)
        else:
            changed, detached = self.peer.resize(self.sess)
        if detached:
            self.detached = True
        elif changed:
            self._synced = False
            self._needs_state = True
            self._sync()
            # what the members that stay pay for a change of membership: agreement, the new
            # session (which waits for every joiner to arrive) and the state hand-over
            self.last_resize_ms = (time.perf_counter() - t0) * 1e3

    def recover(self):
        """After a PeerFailure in the loop body (or in advance()): carry on with the
        members that still answer.  Progress becomes the maximum over them and the
        resize hook runs, as after a planned resize.  Returns how many were dropped."""
        dropped = self.peer.recover(self.sess)
        self._synced = False
        self._needs_state = True
        self._sync()
        return dropped

    def should_stop(self):
        if self.detached:
            return True
        self._sync()
        return self.max_progress is not None and self.progress >= self.max_progress

    def close(self):
        self.sess.close()
        self.peer.close()
