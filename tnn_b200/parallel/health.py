"""Failure detection for multi-rank jobs: heartbeats, a watchdog, host-side fault injection, recovery helpers.

The reference only has bounded ``join(type, n, timeout)`` waits on its coordinator that warn and carry on, and
declares ``HEALTH_CHECK`` / ``JOB_FAILURE`` / ``BARRIER_SYNC`` commands without implementing them
(include/distributed/coordinator.hpp:110-112,145-178, include/distributed/command_type.hpp:45-64,
include/distributed/worker.hpp:192-195); a lost worker blocks training for ever
(coordinator.hpp:201-204). Here:

* every rank publishes a heartbeat (counter, wall time, last finished step) in a ``torch.distributed`` store
  from a background thread; a :class:`Watchdog` on every rank reads its peers' heartbeats and reports ranks
  whose heartbeat is older than ``timeout`` *before* the next collective or fused kernel is launched, so
  nothing is left waiting on a peer that is gone;
* a step watchdog reports a step that runs longer than ``step_timeout`` (a stalled peer, a wedged loader);
* the device side never waits without a bound: every cross-rank wait in the fused kernels gives up after
  about two seconds and records a status code that :func:`check_device_status` turns into
  :class:`KernelTimeout` after the step (the CUDA context stays usable);
* faults are injected on the host only (:class:`FaultPlan`): a rank raises, exits between steps, stalls,
  stops its heartbeat, or a checkpoint file is corrupted. Nothing here makes a GPU fault, trap or hang;
* recovery is a restart of the surviving world size from the newest snapshot
  (:func:`find_latest_snapshot`, ``Trainer.load_snapshot``), which restores weights, optimizer state and step.
"""
from __future__ import annotations

import glob
import json
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence


class RankFailure(RuntimeError):
    """One or more peers stopped sending heartbeats."""

    def __init__(self, dead: Sequence[int], ages: Dict[int, float]):
        self.dead, self.ages = list(dead), dict(ages)
        super().__init__("no heartbeat from rank(s) " + ", ".join(f"{r} ({self.ages.get(r, float('inf')):.1f} s)" for r in self.dead))


class StepTimeout(RuntimeError):
    """A training step ran longer than the watchdog allows."""


class KernelTimeout(RuntimeError):
    """A bounded device-side wait expired (status word of the kernel library)."""


class InjectedFault(RuntimeError):
    """Raised by :class:`FaultPlan` in the rank and step it was asked to fail."""


# ----------------------------------------------------------------------------- heartbeats
class Heartbeat:
    """Publishes ``hb/<rank>`` = ``{"n": counter, "t": time, "step": last finished step}`` every ``interval`` s."""

    def __init__(self, store, rank: int, interval: float = 0.5, clock: Callable[[], float] = time.time):
        self.store, self.rank, self.interval, self.clock = store, int(rank), float(interval), clock
        self.step = -1
        self._n = 0
        self._stop = threading.Event()
        self._muted = threading.Event()  # fault injection: keep running but publish nothing
        self._thread: Optional[threading.Thread] = None

    def beat(self) -> None:
        if self._muted.is_set():
            return
        self._n += 1
        self.store.set(f"hb/{self.rank}", json.dumps({"n": self._n, "t": self.clock(), "step": self.step}))

    def start(self) -> "Heartbeat":
        self.beat()
        self._thread = threading.Thread(target=self._run, name=f"tnnb-heartbeat-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self.beat()
            except Exception:  # the store went away with the job
                return

    def mute(self, flag: bool = True) -> None:
        (self._muted.set if flag else self._muted.clear)()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)


class Watchdog:
    """Reads the peers' heartbeats. ``check()`` raises :class:`RankFailure` for peers silent for ``timeout`` s;
    ``step_begin()`` / ``step_end()`` bracket a step for the step watchdog."""

    def __init__(self, store, rank: int, world: int, timeout: float = 5.0, step_timeout: Optional[float] = None,
                 clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout, self.step_timeout, self.clock = float(timeout), step_timeout, clock
        self._born = clock()
        self._step_t0: Optional[float] = None
        self._last_seen: Dict[int, dict] = {}

    def _read(self, r: int) -> Optional[dict]:
        try:
            if hasattr(self.store, "check") and not self.store.check([f"hb/{r}"]):
                return None
            return json.loads(self.store.get(f"hb/{r}").decode())
        except Exception:
            return None

    def ages(self) -> Dict[int, float]:
        now = self.clock()
        out = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            hb = self._read(r)
            if hb is not None:
                self._last_seen[r] = hb
            seen = self._last_seen.get(r)
            out[r] = (now - seen["t"]) if seen else (now - self._born)
        return out

    def dead_ranks(self) -> List[int]:
        return sorted(r for r, a in self.ages().items() if a > self.timeout)

    def check(self) -> None:
        ages = self.ages()
        dead = sorted(r for r, a in ages.items() if a > self.timeout)
        if dead:
            raise RankFailure(dead, ages)
        if self.step_timeout is not None and self._step_t0 is not None and self.clock() - self._step_t0 > self.step_timeout:
            raise StepTimeout(f"step running for {self.clock() - self._step_t0:.1f} s (limit {self.step_timeout} s)")

    def peer_steps(self) -> Dict[int, int]:
        self.ages()
        return {r: hb.get("step", -1) for r, hb in self._last_seen.items()}

    def step_begin(self) -> None:
        self._step_t0 = self.clock()

    def step_end(self) -> None:
        self._step_t0 = None


# ----------------------------------------------------------------------------- device status
def check_device_status(device=None) -> None:
    """Turn a recorded bounded-wait expiry of the kernel library into :class:`KernelTimeout`."""
    from ..ops import _lib

    try:
        _lib.check_status(device) if device is not None else _lib.check_status()
    except RuntimeError as e:
        if "timeout" in str(e):
            raise KernelTimeout(str(e)) from None
        raise


# ----------------------------------------------------------------------------- fault injection (host only)
@dataclass
class FaultPlan:
    """What to break, where and when. ``kind``: ``raise`` (exception inside the step), ``exit`` (the process leaves
    between steps), ``stall`` (sleep ``seconds`` before the step), ``mute`` (stop publishing heartbeats)."""
    kind: str = "none"
    rank: int = -1
    step: int = -1
    seconds: float = 0.0
    fired: bool = field(default=False, compare=False)

    @classmethod
    def from_env(cls, var: str = "TNNB_FAULT") -> "FaultPlan":
        """``TNNB_FAULT="exit:rank=2:step=3"`` or ``"stall:rank=1:step=2:seconds=4"``."""
        spec = os.environ.get(var, "")
        if not spec:
            return cls()
        parts = spec.split(":")
        kw = dict(p.split("=", 1) for p in parts[1:])
        return cls(kind=parts[0], rank=int(kw.get("rank", -1)), step=int(kw.get("step", -1)), seconds=float(kw.get("seconds", 0)))

    def maybe_fire(self, rank: int, step: int, heartbeat: Optional[Heartbeat] = None) -> None:
        if self.fired or self.kind == "none" or rank != self.rank or step != self.step:
            return
        self.fired = True
        if self.kind == "raise":
            raise InjectedFault(f"injected failure in rank {rank} at step {step}")
        if self.kind == "exit":
            if heartbeat is not None:
                heartbeat.stop()
            os._exit(17)
        if self.kind == "stall":
            time.sleep(self.seconds)
        if self.kind == "mute" and heartbeat is not None:
            heartbeat.mute(True)


def corrupt_file(path: str, offset: int = 64, nbytes: int = 16) -> None:
    """Flip ``nbytes`` bytes of a checkpoint file in place (for checkpoint-integrity tests)."""
    with open(path, "r+b") as f:
        f.seek(offset)
        chunk = bytearray(f.read(nbytes))
        for i in range(len(chunk)):
            chunk[i] ^= 0xFF
        f.seek(offset)
        f.write(bytes(chunk))


# ----------------------------------------------------------------------------- guarded stepping and recovery
class GuardedRunner:
    """Wraps a trainer's ``train_step`` with the checks above::

        runner = GuardedRunner(trainer, store, rank, world, timeout=5.0)
        loss = runner.step(data, labels)      # raises RankFailure / StepTimeout / KernelTimeout / InjectedFault
        runner.close()
    """

    def __init__(self, trainer, store, rank: int, world: int, timeout: float = 5.0, interval: float = 0.5,
                 step_timeout: Optional[float] = None, plan: Optional[FaultPlan] = None, check_device: bool = False):
        self.trainer, self.rank, self.world = trainer, rank, world
        self.heartbeat = Heartbeat(store, rank, interval).start()
        self.watchdog = Watchdog(store, rank, world, timeout, step_timeout)
        self.plan = plan or FaultPlan.from_env()
        self.check_device = check_device
        self.steps_done = 0

    def step(self, data, labels):
        self.plan.maybe_fire(self.rank, self.steps_done, self.heartbeat)
        self.watchdog.check()  # learn about a lost peer on the host, before launching anything that waits for it
        self.watchdog.step_begin()
        try:
            loss = self.trainer.train_step(data, labels)
        except (InjectedFault, RankFailure):
            raise
        except RuntimeError as e:
            # A collective that ended with an error (closed connection, process-group timeout): a peer that left
            # a moment ago still has a fresh heartbeat, so give it `timeout` seconds to go stale and name it.
            dead = self._wait_for_dead()
            if dead:
                raise RankFailure(dead, self.watchdog.ages()) from e
            raise
        finally:
            self.watchdog.step_end()
        if self.check_device:
            check_device_status()
        self.steps_done += 1
        self.heartbeat.step = self.steps_done - 1
        return loss

    def _wait_for_dead(self) -> List[int]:
        deadline = time.time() + self.watchdog.timeout + 2 * self.heartbeat.interval + 0.5
        while time.time() < deadline:
            dead = self.watchdog.dead_ranks()
            if dead:
                return dead
            time.sleep(self.heartbeat.interval)
        return []

    def close(self) -> None:
        self.heartbeat.stop()


def find_latest_snapshot(directory: str, pattern: str = "*.tnng") -> Optional[str]:
    """Newest readable snapshot in ``directory`` (by modification time), skipping files that do not parse."""
    from ..io import tnng

    for path in sorted(glob.glob(os.path.join(directory, pattern)), key=os.path.getmtime, reverse=True):
        try:
            tnng.read_file(path)
            return path
        except Exception:
            continue
    return None
