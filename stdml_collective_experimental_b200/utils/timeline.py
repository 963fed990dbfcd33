"""Turn the trace lines that a traced rank prints at exit into data.

With STDML_COLLECTIVE_ENABLE_TRACE=1 every rank prints one line per recorded
scope, starting with two back-ticks:

    `` <name> <thread> <t0 s> <t1 s> <ms>ms <payload bytes> <GB/s>GB/s

(the reference prints the same shape, src/stdml/collective/stat.cpp:27-58, and
post-processes it with scripts/vis/timeline.sh).  `parse_log` reads those lines
from a rank's log, `to_chrome_trace` merges several ranks into one Chrome /
Perfetto trace, `summary` aggregates per scope name.
"""
import json
import re

_LINE = re.compile(r"^`` (\S+) (\d+) ([0-9.]+) ([0-9.]+) ([0-9.]+)ms (\d+) ([0-9.]+)GB/s")


def parse_log(text):
    events = []
    for line in text.splitlines():
        m = _LINE.match(line)
        if m:
            events.append({"name": m.group(1), "thread": int(m.group(2)), "t0": float(m.group(3)),
                           "t1": float(m.group(4)), "bytes": int(m.group(6))})
    return events


def to_chrome_trace(per_rank_events):
    """per_rank_events: {rank: [event, ...]} -> Chrome trace dict."""
    out = []
    for rank, events in per_rank_events.items():
        for e in events:
            out.append({"name": e["name"], "ph": "X", "pid": rank, "tid": e["thread"],
                        "ts": e["t0"] * 1e6, "dur": (e["t1"] - e["t0"]) * 1e6,
                        "args": {"bytes": e["bytes"]}})
    return {"traceEvents": out}


def summary(events):
    agg = {}
    for e in events:
        d = agg.setdefault(e["name"], {"calls": 0, "seconds": 0.0, "bytes": 0})
        d["calls"] += 1
        d["seconds"] += e["t1"] - e["t0"]
        d["bytes"] += e["bytes"]
    for d in agg.values():
        d["gb_s"] = d["bytes"] / d["seconds"] / 1e9 if d["seconds"] > 0 else 0.0
    return agg


def write_chrome_trace(per_rank_events, path):
    with open(path, "w") as f:
        json.dump(to_chrome_trace(per_rank_events), f)
