"""Turn a profiler log into a timeline: a Chrome / Perfetto trace (JSON) and a text summary per source.

    python -m tnn_b200.utils.profile_timeline logs/profiler.log --trace logs/profiler_trace.json

Reads the lines the profiler writes - ``Event: <name>, Source: <src>, Type: COMPUTE|COMMUNICATION|OTHER, Start: <ms> ms,
End: <ms> ms, Duration: <ms> ms`` - which is also the format of the reference's coordinator log, parsed there by
``visualizers/visualize_profiler.py:8`` with the same regular expression; that script draws a matplotlib figure, this
one writes the trace-event format that ``chrome://tracing`` and Perfetto open (one process per source, one thread per
event type), which needs no plotting library.
"""
from __future__ import annotations

import argparse
import json
import re
from typing import Dict, List, Tuple

LINE = re.compile(r"(?:Event:\s+(?P<name>.*?),\s+)?Source:\s+(?P<src>[\w.\-:]+),\s+Type:\s+(?P<type>\w+),\s+Start:\s+(?P<start>[-\d.]+)\s+ms,"
                  r"\s+End:\s+(?P<end>[-\d.]+)\s+ms")


def parse_log(path: str) -> Dict[str, Dict[str, List[Tuple[str, float, float]]]]:
    """``{source: {type: [(name, start_ms, duration_ms), ...]}}``"""
    out: Dict[str, Dict[str, List[Tuple[str, float, float]]]] = {}
    with open(path) as f:
        for line in f:
            m = LINE.search(line)
            if not m:
                continue
            start, end = float(m["start"]), float(m["end"])
            out.setdefault(m["src"], {}).setdefault(m["type"], []).append((m["name"] or m["type"], start, end - start))
    return out


def to_trace(events) -> dict:
    trace = []
    for pid, (src, by_type) in enumerate(sorted(events.items())):
        trace.append({"ph": "M", "pid": pid, "name": "process_name", "args": {"name": src}})
        for tid, (typ, evs) in enumerate(sorted(by_type.items())):
            trace.append({"ph": "M", "pid": pid, "tid": tid, "name": "thread_name", "args": {"name": typ}})
            for name, start, dur in evs:
                trace.append({"ph": "X", "pid": pid, "tid": tid, "name": name, "cat": typ, "ts": start * 1e3, "dur": max(dur, 0.0) * 1e3})
    return {"traceEvents": trace, "displayTimeUnit": "ms"}


def summary(events) -> str:
    lines = []
    for src, by_type in sorted(events.items()):
        t0 = min(s for evs in by_type.values() for _, s, _ in evs)
        t1 = max(s + d for evs in by_type.values() for _, s, d in evs)
        parts = [f"{typ} {sum(d for _, _, d in evs):.3f} ms in {len(evs)} events" for typ, evs in sorted(by_type.items())]
        lines.append(f"{src}: span {t1 - t0:.3f} ms; " + "; ".join(parts))
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("log")
    ap.add_argument("--trace", default="", help="write a Chrome / Perfetto trace-event JSON file here")
    a = ap.parse_args(argv)
    ev = parse_log(a.log)
    if not ev:
        print("no profiler events found")
        return 1
    print(summary(ev))
    if a.trace:
        with open(a.trace, "w") as f:
            json.dump(to_trace(ev), f)
        print(f"trace -> {a.trace}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
