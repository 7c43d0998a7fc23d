"""Per-launch timeline in Chrome's Trace Event format.

Takes the place of the reference's tracing hook: with TRACING=1 in the environment a computation
records a timeline of what it ran (ngraph/util/trace_events.py:21-60: TraceEventTracker, events
{ph: 'X', cat, name, pid, tid, ts, dur, args} serialised as {"traceEvents": [...]};
ngraph/transformers/base.py:108-111, 138: Computation.__call__ -> generate_profile).  Here every
step of the step list is bracketed by a pair of CUDA events on the launching stream; after the
call's one synchronisation the pairs become 'X' events with device timestamps in microseconds
(pid = device, tid = 0 for the compute stream).  While tracing, a computation launches step by
step even if it was captured as a CUDA graph -- a replayed graph has no per-kernel boundaries to
put events on -- so traced timings include launch gaps that the graph replay does not have.
"""
import json
import os


def is_tracing_enabled():
    return os.environ.get("TRACING") == "1"


class TraceEventTracker(object):
    """Collects events; `serialize_to_file` writes <name>.json (load it in chrome://tracing)."""

    def __init__(self, tracker_name):
        self.name = tracker_name
        self.events = []

    def add_operation(self, category, name, pid, tid, timestamp, duration, args):
        self.events.append({"ph": "X", "cat": category, "name": name, "pid": pid, "tid": tid,
                            "ts": timestamp, "dur": duration, "args": args})

    def serialize(self):
        return json.dumps({"traceEvents": self.events}, separators=(",", ":"))

    def serialize_to_file(self, path=None):
        path = path or (self.name + ".json")
        with open(path, "w") as out:
            out.write(self.serialize())
        return path


def step_name(step):
    """A readable name for a step of the executor's list."""
    if step.kind == "ew":
        ops = [getattr(m, "opname", None) or getattr(m, "redop", None) or type(m).__name__
               for m in step.group.members]
        return "b2_ew_main[" + ",".join(ops[:8]) + ("..." if len(ops) > 8 else "") + "]"
    op = getattr(step, "op", None)
    return "%s:%s" % (step.kind, getattr(op, "name", "") or step.kind)
