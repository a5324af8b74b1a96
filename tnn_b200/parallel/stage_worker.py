"""The coordinator / worker protocol of the reference, spoken in its own wire format.

The reference trains a pipeline by exchanging archiver-encoded messages between a coordinator process and one
worker process per stage over TCP or RoCE (include/distributed/coordinator.hpp:84-260,
include/distributed/worker.hpp:145-307, include/distributed/command_type.hpp:20-86). On one NVSwitch box the
production path here is SPMD (``parallel/pp.py``: 1F1B over NCCL point-to-point, no coordinator process); this module
keeps the *protocol* alive on top of the same C++ wire library, so that captured messages and ``StageConfig`` blobs
stay meaningful and a stage can be driven by any transport that moves byte strings:

* :class:`StageWorker` holds one stage graph, its optimizer and scheduler and turns each incoming message into the
  reference's reply: ``CONFIG_TRANSFER -> CONFIG_RECEIVED``, ``TRAIN_MODE / EVAL_MODE -> MODE_CHANGED``,
  ``FORWARD_JOB -> FORWARD_JOB`` to the next stage, ``BACKWARD_JOB -> BACKWARD_JOB`` to the previous stage or
  ``BACKWARD_COMPLETE`` to the coordinator at stage 0, ``UPDATE_PARAMETERS -> PARAMETERS_UPDATED``,
  ``SAVE_TO_FILE`` (``ERROR_REPORT`` on failure), ``PRINT_LR -> LR_PRINTED``, ``START_PROFILING``,
  ``REPORT_PROFILING -> PROFILING_REPORTED`` (profiler payload), ``PRINT_PROFILING -> PROFILING_PRINTED``,
  ``CLEAR_PROFILING -> PROFILING_CLEARED``, ``PRINT_LOGS -> LOGS_PRINTED``, ``HANDSHAKE`` / ``HANDSHAKE_ACK`` (ignored),
  ``SHUTDOWN``. ``SEND_PARAMS -> PARAMS_TRANSFER``, ``LOAD_PARAMS -> PARAMS_LOADED`` and
  ``STATUS_REQUEST -> STATUS_RESPONSE``, whose bodies the reference leaves empty or throwing, are implemented. Commands
  the reference declares without a handler (``HEALTH_CHECK``, ``BARRIER_SYNC``, ...) answer ``ERROR_REPORT``.
* :class:`LocalCoordinator` is the coordinator's side: it partitions a graph, configures the workers, splits a
  batch into micro-batches, computes loss and dL/dlogits (scaled by ``1 / micro-batches``,
  coordinator.hpp:225) and drives forward / backward / update - delivering messages through a ``send`` callable
  (in-process by default, like the reference's in-process communicator, include/distributed/communicator.hpp:51-62).
"""
from __future__ import annotations

import json
import time
from collections import deque
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

import torch

from ..host import H
from ..io import tnng
from ..nn.graph import Graph, partition_graph
from ..nn.loss import create_loss
from ..nn.optim import create_optimizer
from ..nn.schedulers import create_scheduler

NONE, JOB, STRING, BOOL, PROFILER, STAGE_CONFIG = range(6)
COORDINATOR = "coordinator"


def _cmd(name: str) -> int:
    return H.command_code(name)


def job_message(command: str, pid: int, tensors: Dict[str, torch.Tensor]) -> bytes:
    return H.serialize_message({"command": _cmd(command), "kind": JOB,
                                "job": {"pid": int(pid), "tensors": [(k, tnng.tensor_to_record(v)) for k, v in tensors.items()]}})


def simple_message(command: str, text: Optional[str] = None, flag: Optional[bool] = None) -> bytes:
    m = {"command": _cmd(command), "kind": NONE}
    if text is not None:
        m.update(kind=STRING, text=text)
    elif flag is not None:
        m.update(kind=BOOL, flag=bool(flag))
    return H.serialize_message(m)


def stage_config_message(stage: Graph, optimizer_cfg: dict, scheduler_cfg: dict, next_stage: str, prev_stage: str,
                         coordinator: str = "coordinator") -> bytes:
    return H.serialize_message({"command": _cmd("CONFIG_TRANSFER"), "kind": STAGE_CONFIG, "stage": {
        "graph_state": tnng.serialize(stage.state()), "input_uids": [n.uid() for n in stage.input_nodes],
        "output_uids": [n.uid() for n in stage.output_nodes], "optimizer_config": json.dumps(optimizer_cfg),
        "scheduler_config": json.dumps(scheduler_cfg), "next_stage": next_stage, "prev_stage": prev_stage,
        "coordinator": coordinator}})


class StageWorker:
    """One pipeline stage behind the message protocol. ``handle(bytes)`` returns ``[(destination, bytes), ...]``
    where destination is an endpoint name (``"coordinator"``, the next or the previous stage)."""

    def __init__(self, name: str, device: str = "cpu"):
        self.name, self.device = name, device
        self.graph: Optional[Graph] = None
        self.optimizer = self.scheduler = None
        self.next_stage = self.prev_stage = ""
        self.profiler = H.Profiler()
        self.profiling = False
        self.alive = True

    # ------------------------------------------------------------------ dispatch
    def handle(self, data: bytes) -> List[Tuple[str, bytes]]:
        t0 = time.time_ns()
        msg = H.parse_message(data)
        name = msg["command_name"]
        try:
            fn = getattr(self, "_on_" + name.lower(), None)
            out = fn(msg) if fn is not None else [(COORDINATOR, simple_message("ERROR_REPORT", text=f"{self.name}: {name} is not implemented"))]
        except Exception as e:  # the reference reports configuration / save failures as ERROR_REPORT (worker.hpp:254-258,309-319)
            out = [(COORDINATOR, simple_message("ERROR_REPORT", text=f"{self.name}: {name} failed: {type(e).__name__}: {e}"))]
        if self.profiling:
            self.profiler.add_event(0, t0, time.time_ns(), name, self.name)
        return out

    # ------------------------------------------------------------------ handlers
    def _on_config_transfer(self, msg):
        st = msg["stage"]
        self.graph = Graph.from_state(tnng.parse(bytes(st["graph_state"])), device=self.device)
        self.graph.input_requires_grad = bool(st["prev_stage"])
        self.optimizer = create_optimizer(json.loads(st["optimizer_config"] or "{}")).attach(self.graph)
        self.scheduler = create_scheduler(json.loads(st["scheduler_config"] or "{}"), self.optimizer)
        self.next_stage, self.prev_stage = st["next_stage"], st["prev_stage"]
        if sorted(n.uid() for n in self.graph.input_nodes) != sorted(st["input_uids"]):
            raise ValueError("stage inputs do not match the graph state")
        return [(COORDINATOR, simple_message("CONFIG_RECEIVED", flag=True))]

    def _on_train_mode(self, msg):
        self.graph.set_training(True)
        return [(COORDINATOR, simple_message("MODE_CHANGED"))]

    def _on_eval_mode(self, msg):
        self.graph.set_training(False)
        return [(COORDINATOR, simple_message("MODE_CHANGED"))]

    def _bundle(self, msg) -> Dict[str, torch.Tensor]:
        return {k: tnng.record_to_tensor(rec).to(self.device) for k, rec in msg["job"]["tensors"]}

    def _on_forward_job(self, msg):
        pid = msg["job"]["pid"]
        out = self.graph.forward(self._bundle(msg), pid)
        return [(self.next_stage or COORDINATOR, job_message("FORWARD_JOB", pid, out))]

    def _on_backward_job(self, msg):
        pid = msg["job"]["pid"]
        gin = self.graph.backward(self._bundle(msg), pid)
        if self.prev_stage:
            return [(self.prev_stage, job_message("BACKWARD_JOB", pid, gin))]
        return [(COORDINATOR, job_message("BACKWARD_COMPLETE", pid, {}))]

    def _on_update_parameters(self, msg):
        self.scheduler.step()
        self.optimizer.update()
        self.graph.zero_grads()
        return [(COORDINATOR, simple_message("PARAMETERS_UPDATED"))]

    def _on_save_to_file(self, msg):
        self.graph.save_state(msg["text"])
        return []

    def _on_print_lr(self, msg):
        return [(COORDINATOR, simple_message("LR_PRINTED", text=f"{self.name}: lr {self.optimizer.get_learning_rate():.8g}"))]

    def _on_start_profiling(self, msg):
        self.profiler.clear()
        self.profiler.start()
        self.profiling = True
        return [(COORDINATOR, simple_message("PROFILING_STARTED"))]

    def _on_report_profiling(self, msg):
        return [(COORDINATOR, H.serialize_message({"command": _cmd("PROFILING_REPORTED"), "kind": PROFILER,
                                                    "profiler": {"start_time": self.profiler.start_time(),
                                                                 "events": self.profiler.events()}}))]

    def _on_clear_profiling(self, msg):
        self.profiler.clear()
        return [(COORDINATOR, simple_message("PROFILING_CLEARED"))]

    def _on_print_profiling(self, msg):
        for line in self.profiler.log_lines():
            print(line, flush=True)
        return [(COORDINATOR, simple_message("PROFILING_PRINTED"))]

    def _on_print_logs(self, msg):
        return [(COORDINATOR, simple_message("LOGS_PRINTED"))]

    def _on_handshake(self, msg):
        return []

    _on_handshake_ack = _on_handshake

    def _on_error_report(self, msg):
        print(f"{self.name} received error: {msg.get('text', '')}", flush=True)
        return []

    # The reference declares the next three commands and leaves their bodies empty or throwing
    # (worker.hpp:192-195,246-261); here they work, so that a coordinator can read a stage's weights back, push new
    # ones (a restart from another run's snapshot without touching the worker's disk) and ask what a worker holds.
    def _param_items(self):
        for layer in self.graph.layers():
            for i, t in enumerate(layer.params):
                yield f"{layer.name}:{i}", t

    def _on_send_params(self, msg):
        # master precision, like a checkpoint
        return [(COORDINATOR, job_message("PARAMS_TRANSFER", 0, {k: self.graph._master_view(t) for k, t in self._param_items()}))]

    def _on_load_params(self, msg):
        mine = dict(self._param_items())
        got = self._bundle(msg)
        unknown = sorted(set(got) - set(mine))
        if unknown:
            raise KeyError(f"no such parameters on this stage: {unknown[:4]}")
        for k, t in got.items():
            if tuple(t.shape) != tuple(mine[k].shape):
                raise ValueError(f"{k}: shape {tuple(t.shape)} does not match {tuple(mine[k].shape)}")
        with torch.no_grad():
            for k, t in got.items():
                self.graph._load_param(mine[k], t)  # into the fp32 master where the stage keeps one
            self.graph.sync_params_from_master()
        return [(COORDINATOR, simple_message("PARAMS_LOADED", flag=True))]

    def _on_status_request(self, msg):
        st = {"name": self.name, "configured": self.graph is not None, "next_stage": self.next_stage, "prev_stage": self.prev_stage}
        if self.graph is not None:
            st.update(training=bool(self.graph.training), layers=len(self.graph.layers()),
                      parameters=int(sum(t.numel() for _, t in self._param_items())),
                      learning_rate=float(self.optimizer.get_learning_rate()), profiled_events=len(self.profiler))
        return [(COORDINATOR, simple_message("STATUS_RESPONSE", text=json.dumps(st)))]

    def _on_shutdown(self, msg):
        self.alive = False
        return []


class LocalCoordinator:
    """Drives stage workers through the protocol. The default transport is an in-process queue that calls the
    destination worker's ``handle``; with ``transport`` (an object with ``name``, ``send(endpoint, bytes)`` and
    ``recv(timeout_s) -> (endpoint, bytes) | None``, see ``parallel/tcp_transport.py``) and ``endpoints`` (one per
    stage, in pipeline order) the same coordinator drives worker processes on other hosts."""

    reply_timeout_s = 60.0  # the reference's join() waits 60 s for the replies of a broadcast (coordinator.hpp:541-568)

    def __init__(self, graph: Graph, ratios: Sequence[float], optimizer_cfg: dict, scheduler_cfg: Optional[dict] = None,
                 loss_cfg: Optional[dict] = None, microbatches: int = 2, device: str = "cpu",
                 workers: Optional[Dict[str, StageWorker]] = None, transport=None, endpoints: Optional[Sequence[str]] = None):
        self.micro = max(1, int(microbatches))
        self.loss = create_loss(loss_cfg or {"type": "logsoftmax_crossentropy"})
        if not graph.compiled:
            graph.compile(device="cpu", seed=0)  # initial values of the whole model, as a single-process run would draw them
        # stage graphs share the layer objects (and so the parameter values) of `graph`; only their state is shipped
        stages = partition_graph(graph, ratios)
        self.transport = transport
        if transport is not None:
            if endpoints is None or len(endpoints) != len(stages):
                raise ValueError(f"{len(stages)} stages need {len(stages)} worker endpoints")
            self.names = list(endpoints)
            self.workers = {}
        else:
            self.names = [f"stage{i}" for i in range(len(stages))]
            self.workers = workers or {n: StageWorker(n, device) for n in self.names}
        self.inbox: Deque[dict] = deque()
        self.queue: Deque[Tuple[str, bytes]] = deque()
        self.in_uid = stages[0].input_nodes[0].uid()
        self.out_uid = stages[-1].output_nodes[0].uid()
        for i, (n, s) in enumerate(zip(self.names, stages)):
            nxt = self.names[i + 1] if i + 1 < len(stages) else ""
            prv = self.names[i - 1] if i > 0 else ""
            self.post(n, stage_config_message(s, optimizer_cfg, scheduler_cfg or {"type": "no_op"}, nxt, prv,
                                              transport.name if transport is not None else COORDINATOR))
        replies = self.run(len(stages))
        bad = [r for r in replies if r["command_name"] != "CONFIG_RECEIVED" or not r.get("flag")]
        if bad or len(replies) != len(stages):
            raise RuntimeError(f"stage configuration failed: {bad}")

    # ------------------------------------------------------------------ transport
    def post(self, dst: str, data: bytes) -> None:
        if self.transport is not None:
            self.transport.send(dst, data)
        else:
            self.queue.append((dst, data))

    def run(self, expect: int = 0) -> List[dict]:
        """In process: deliver queued messages until none is left; returns what reached the coordinator. Over a
        transport: wait for ``expect`` messages addressed to the coordinator."""
        got = []
        if self.transport is not None:
            deadline = time.monotonic() + self.reply_timeout_s
            lost_fn = getattr(self.transport, "lost", None)
            while len(got) < expect:
                # wait in short slices so that a worker whose connection dropped is noticed at once instead of after
                # the whole reply timeout (the reference's coordinator blocks for ever on a lost worker)
                item = self.transport.recv(min(0.5, max(0.0, deadline - time.monotonic())))
                if item is None:
                    gone = lost_fn(self.names) if lost_fn is not None else []
                    if gone:
                        raise ConnectionError(f"lost the connection to {gone} while waiting for {expect - len(got)} replies")
                    if time.monotonic() >= deadline:
                        raise TimeoutError(f"{len(got)} of {expect} replies arrived within {self.reply_timeout_s:.0f} s")
                    continue
                m = H.parse_message(item[1])
                if m["command_name"] == "ERROR_REPORT":
                    raise RuntimeError(m.get("text", "worker error"))
                got.append(m)
            return got
        while self.queue:
            dst, data = self.queue.popleft()
            if dst == COORDINATOR:
                got.append(H.parse_message(data))
                continue
            for d2, m2 in self.workers[dst].handle(data):
                self.queue.append((d2, m2))
        for m in got:
            if m["command_name"] == "ERROR_REPORT":
                raise RuntimeError(m.get("text", "worker error"))
        return got

    def broadcast(self, command: str, expect: Optional[str] = None, **kw) -> List[dict]:
        for n in self.names:
            self.post(n, simple_message(command, **kw))
        got = self.run(len(self.names) if expect is not None else 0)
        if expect is not None and sorted(m["command_name"] for m in got) != [expect] * len(self.names):
            raise RuntimeError(f"{command}: expected {len(self.names)} x {expect}, got {[m['command_name'] for m in got]}")
        return got

    # ------------------------------------------------------------------ training
    def train_batch(self, data: torch.Tensor, labels: torch.Tensor) -> float:
        """All forward jobs go to stage 0 first (coordinator.hpp:193-195), the last stage returns the logits, the
        coordinator computes the loss and dL/dlogits scaled by 1 / micro-batches, then the update."""
        mb_data, mb_labels = data.chunk(self.micro), labels.chunk(self.micro)
        for pid, d in enumerate(mb_data):
            self.post(self.names[0], job_message("FORWARD_JOB", pid, {self.in_uid: d}))
        outs = {m["job"]["pid"]: m for m in self.run(len(mb_data)) if m["command_name"] == "FORWARD_JOB"}
        total = 0.0
        for pid, lab in enumerate(mb_labels):
            logits = dict(outs[pid]["job"]["tensors"])[self.out_uid]
            loss, grad = self.loss.compute(tnng.record_to_tensor(logits), lab, 1.0 / len(mb_data), True)
            total += float(loss) / len(mb_data)
            self.post(self.names[-1], job_message("BACKWARD_JOB", pid, {self.out_uid: grad}))
        done = [m for m in self.run(len(mb_data)) if m["command_name"] == "BACKWARD_COMPLETE"]
        if len(done) != len(mb_data):
            raise RuntimeError("not every micro-batch completed its backward pass")
        self.broadcast("UPDATE_PARAMETERS", expect="PARAMETERS_UPDATED")
        return total

    def val_batch(self, data: torch.Tensor, labels: torch.Tensor) -> Tuple[float, int]:
        """Forward-only pass of one batch through the stages, micro-batch by micro-batch; returns the mean loss and
        the number of correct arg-max predictions (reference: coordinator async_val_batch / sync_val_batch,
        distributed/train.hpp:153-199). The workers must be in evaluation mode (:meth:`evaluate` switches them)."""
        mb_data, mb_labels = data.chunk(self.micro), labels.chunk(self.micro)
        for pid, d in enumerate(mb_data):
            self.post(self.names[0], job_message("FORWARD_JOB", pid, {self.in_uid: d}))
        outs = {m["job"]["pid"]: m for m in self.run(len(mb_data)) if m["command_name"] == "FORWARD_JOB"}
        total, correct = 0.0, 0
        for pid, lab in enumerate(mb_labels):
            logits = tnng.record_to_tensor(dict(outs[pid]["job"]["tensors"])[self.out_uid])
            loss, _ = self.loss.compute(logits, lab, 1.0, False)
            total += float(loss) / len(mb_data)
            c = self.loss.corrects()
            correct += int(c) if c is not None else 0
        return total, correct

    def evaluate(self, loader, max_batches: Optional[int] = None) -> Dict[str, float]:
        """Validation over a loader: EVAL_MODE on every stage, forward-only batches, TRAIN_MODE again."""
        self.broadcast("EVAL_MODE", expect="MODE_CHANGED")
        tot, corr, rows, n = 0.0, 0, 0, 0
        try:
            for data, labels in loader:
                l, c = self.val_batch(data, labels)
                tot, corr, rows, n = tot + l, corr + c, rows + labels.numel(), n + 1
                if max_batches and n >= max_batches:
                    break
        finally:
            self.broadcast("TRAIN_MODE", expect="MODE_CHANGED")
        mean = tot / max(1, n)
        return {"loss": mean, "accuracy_pct": 100.0 * corr / max(1, rows), "batches": n}

    def merged_profile(self) -> H.Profiler:
        merged = H.Profiler()
        first = True
        for n in self.names:
            self.post(n, simple_message("REPORT_PROFILING"))
        for m in self.run(len(self.names)):
            p = H.Profiler()
            p.set_start_time(m["profiler"]["start_time"])
            for (s, e, t, name, src) in m["profiler"]["events"]:
                p.add_event(t, s, e, name, src)
            if first:
                merged.set_start_time(p.start_time())
                first = False
            merged.merge(p)
        merged.sort()
        return merged

    def shutdown(self) -> None:
        for n in self.names:
            self.post(n, simple_message("SHUTDOWN"))
        self.run()
