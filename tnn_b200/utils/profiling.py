"""Per-layer timing of forward and backward passes, recorded into the C++ event profiler.

The reference declares ``EventType::COMPUTE`` and the ``print_layer_profiling`` option but instruments only its
communicator (include/profiling/profiler.hpp:135-160, include/distributed/tcp_communicator.hpp:325-349,
configs/example_config.jsonc:10-11). Here every executor segment of the graph (a layer, or a fused chain of layers)
is bracketed by CUDA events on the launching stream - device time, not host time - or by ``perf_counter`` on CPU;
the spans become ``COMPUTE`` events of :class:`H.Profiler`, which keeps the reference's merge-with-clock-offset and
its ``Event: ..., Source: ..., Type: ..., Start: ... ms, End: ... ms, Duration: ... ms`` log line, so the
reference's timeline visualiser reads our ``profiler.log`` too.

``profiler_type``: ``NORMAL`` keeps the spans of the last step, ``CUMULATIVE`` adds them up over steps.
Profiling serialises nothing by itself, but it cannot be combined with CUDA-graph replay (events inside a captured
graph carry no timing): the trainer leaves the graph off while a profiler is attached.
"""
from __future__ import annotations

import contextlib
import os
import time
from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch

from ..host import H

COMPUTE, COMMUNICATION, OTHER = 0, 1, 2


class LayerProfiler:
    def __init__(self, device: torch.device, source: str = "rank0", cumulative: bool = False, nvtx: Optional[bool] = None):
        self.device, self.source, self.cumulative = device, source, cumulative
        self.cuda = device.type == "cuda"
        # NVTX ranges ("layer:phase") around every span, so that a timeline tool shows the same names as the event
        # log; on by default on a GPU, TNNB_NVTX=0 turns them off
        self.nvtx = (self.cuda and os.environ.get("TNNB_NVTX", "1") != "0") if nvtx is None else (bool(nvtx) and self.cuda)
        self._pending: List[Tuple[str, str, object, object]] = []
        self.totals: "OrderedDict[Tuple[str, str], List[float]]" = OrderedDict()  # (name, phase) -> [ms, calls]
        self.profiler = H.Profiler()
        self.profiler.start()
        self._t0_ns = time.time_ns()
        self._base = None
        if self.cuda:
            self._base = torch.cuda.Event(enable_timing=True)
            self._base.record()

    @contextlib.contextmanager
    def span(self, name: str, phase: str):
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if self.nvtx:
                torch.cuda.nvtx.range_push(f"{name}:{phase}")
            a.record()
            try:
                yield
            finally:
                b.record()
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
            self._pending.append((name, phase, a, b))
        else:
            t0 = time.perf_counter_ns()
            yield
            t1 = time.perf_counter_ns()
            self._pending.append((name, phase, t0, t1))

    def begin_step(self) -> None:
        if not self.cumulative:
            self.totals.clear()
            self.profiler.clear()

    def end_step(self) -> None:
        """Resolve the spans of the step (one synchronisation) into events and totals."""
        if self.cuda:
            torch.cuda.synchronize(self.device)
        for name, phase, a, b in self._pending:
            if self.cuda:
                start_ns = self._t0_ns + int(self._base.elapsed_time(a) * 1e6)
                dur_ms = a.elapsed_time(b)
                end_ns = start_ns + int(dur_ms * 1e6)
            else:
                start_ns, end_ns = self._t0_ns + (a - self._cpu0()), self._t0_ns + (b - self._cpu0())
                dur_ms = (b - a) / 1e6
            self.profiler.add_event(COMPUTE, start_ns, end_ns, f"{name}:{phase}", self.source)
            t = self.totals.setdefault((name, phase), [0.0, 0])
            t[0] += dur_ms
            t[1] += 1
        self._pending.clear()

    def _cpu0(self) -> int:
        if not hasattr(self, "_cpu_base"):
            self._cpu_base = time.perf_counter_ns() - (time.time_ns() - self._t0_ns)
        return self._cpu_base

    # ------------------------------------------------------------------ reports
    def table(self, top: Optional[int] = None) -> str:
        rows: Dict[str, List[float]] = OrderedDict()
        for (name, phase), (ms, calls) in self.totals.items():
            r = rows.setdefault(name, [0.0, 0.0, 0])
            r[0 if phase == "forward" else 1] += ms
            r[2] = max(r[2], calls)
        items = sorted(rows.items(), key=lambda kv: -(kv[1][0] + kv[1][1]))
        total = sum(v[0] + v[1] for _, v in items) or 1.0
        lines = [f"{'layer':<56} {'fwd ms':>9} {'bwd ms':>9} {'share':>7} {'calls':>6}"]
        for name, (f, b, c) in items[:top]:
            lines.append(f"{name[:56]:<56} {f:9.3f} {b:9.3f} {100 * (f + b) / total:6.1f}% {c:6d}")
        lines.append(f"{'total':<56} {sum(v[0] for _, v in items):9.3f} {sum(v[1] for _, v in items):9.3f}")
        return "\n".join(lines)

    def write_log(self, path: str) -> str:
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self.profiler.sort()
        with open(path, "w") as f:
            for line in self.profiler.log_lines():
                f.write(line + "\n")
        return path


def merge_across_ranks(lp: LayerProfiler, group=None) -> Optional[H.Profiler]:
    """Gather every rank's events on rank 0 and merge them with the clock-offset shift of the reference
    (include/distributed/coordinator.hpp:450-511). Returns the merged profiler on rank 0, None elsewhere."""
    import torch.distributed as dist

    if not dist.is_initialized():
        return lp.profiler
    payload = {"start": lp.profiler.start_time(), "events": lp.profiler.events()}
    allp = [None] * dist.get_world_size(group)
    dist.all_gather_object(allp, payload, group=group)
    if dist.get_rank(group) != 0:
        return None
    merged = H.Profiler()
    merged.set_start_time(allp[0]["start"])
    for p in allp:
        other = H.Profiler()
        other.set_start_time(p["start"])
        for (s, e, t, name, src) in p["events"]:
            other.add_event(t, s, e, name, src)
        merged.merge(other)
    merged.sort()
    return merged
