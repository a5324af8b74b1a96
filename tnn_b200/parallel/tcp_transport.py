"""Coordinator / worker pipeline training between hosts over TCP.

The reference's only distributed mode is a coordinator process that drives one worker process per pipeline stage over
TCP (examples/tcp_coordinator.cpp:27-128, examples/tcp_worker.cpp:39-141, include/distributed/tcp_communicator.hpp).
Inside one NVSwitch box this framework trains SPMD over NCCL and peer memory (``parallel/pp.py``); this module is the
path between boxes, or to a host without GPUs: the same protocol and wire format, carried by the C++
``TcpCommunicator`` (``csrc/host/tcp_comm.*``: several sockets per peer, 4 MiB packets, reassembly in any order,
reader / writer threads that run while the interpreter computes).

* :class:`TcpTransport` wraps one communicator: ``name`` (``"ip:port"``), ``send`` (connects on first use), ``recv``.
* :class:`TcpStageServer` is a worker process: it listens, receives its stage with ``CONFIG_TRANSFER`` and then
  serves jobs until ``SHUTDOWN``. Results go to the next / previous stage's endpoint directly, not through the
  coordinator.
* :func:`tcp_coordinator` builds a :class:`~tnn_b200.parallel.stage_worker.LocalCoordinator` that talks to such
  servers.
"""
from __future__ import annotations

import time
from typing import Optional, Sequence, Tuple

from ..host import H
from .stage_worker import COORDINATOR, LocalCoordinator, StageWorker, simple_message


def split_endpoint(endpoint: str) -> Tuple[str, int]:
    host, _, port = endpoint.rpartition(":")
    if not host or not port.isdigit():
        raise ValueError(f"endpoint must look like host:port, got {endpoint!r}")
    return host, int(port)


class TcpTransport:
    """One listening endpoint. ``sockets_per_endpoint`` and ``max_packet_size`` are the reference's
    ``skts_per_endpoint`` (default 4) and ``max_packet_size`` (4 MiB)."""

    def __init__(self, host: str = "127.0.0.1", port: int = 0, sockets_per_endpoint: int = 4, max_packet_size: int = 4 << 20):
        self.comm = H.TcpCommunicator(host, port, sockets_per_endpoint, max_packet_size)
        self.comm.start()
        self.name = self.comm.endpoint()

    def send(self, endpoint: str, data: bytes, connect_timeout_s: float = 30.0) -> None:
        if not self.comm.connected(endpoint):
            host, port = split_endpoint(endpoint)
            self.comm.connect(host, port, connect_timeout_s)
        self.comm.send(endpoint, data)

    def recv(self, timeout_s: float = -1.0):
        return self.comm.recv(timeout_s)

    def lost(self, endpoints: Sequence[str]):
        """Those of ``endpoints`` this side had a connection to, all of whose sockets have since closed (the peer
        exited or the network dropped; reference: handle_channel_error, tcp_communicator.hpp:359-393)."""
        known = set(self.comm.peers())
        return [e for e in endpoints if e in known and not self.comm.connected(e)]

    def flush(self, timeout_s: float = 30.0) -> None:
        self.comm.flush(timeout_s)

    def stats(self) -> dict:
        return self.comm.stats()

    def close(self) -> None:
        self.comm.flush(5.0)
        self.comm.stop()


class TcpStageServer:
    """A stage worker behind a TCP endpoint (the reference's ``tcp_worker <port>``). The coordinator is whoever
    sends ``CONFIG_TRANSFER``; the neighbours' endpoints arrive inside that message."""

    def __init__(self, host: str = "127.0.0.1", port: int = 0, device: str = "cpu", sockets_per_endpoint: int = 4,
                 max_packet_size: int = 4 << 20, log_path: str = ""):
        self.transport = TcpTransport(host, port, sockets_per_endpoint, max_packet_size)
        self.name = self.transport.name
        self.worker = StageWorker(self.name, device)
        self.coordinator: Optional[str] = None
        # per-event log of this worker: step (number of updates so far), command, handling time, device memory in use
        # (the reference's worker CSV: step,event_type,time_ms,mem - include/nn/csv_logger.hpp:76-99)
        self.log = None
        if log_path:
            from ..utils.csv_logger import WorkerCsvLogger
            self.log = WorkerCsvLogger(log_path)
        self._updates = 0

    def serve(self, idle_timeout_s: float = -1.0) -> int:
        """Handles messages until ``SHUTDOWN`` (or until nothing arrived for ``idle_timeout_s``); returns how many."""
        n = 0
        config_transfer = H.command_code("CONFIG_TRANSFER")
        try:
            while self.worker.alive:
                if idle_timeout_s >= 0:
                    item = self.transport.recv(idle_timeout_s)
                    if item is None:
                        break
                else:  # wait for ever, but not for a coordinator whose connection is gone
                    item = self.transport.recv(1.0)
                    if item is None:
                        if self.coordinator is not None and self.transport.lost([self.coordinator]):
                            print(f"{self.name}: the coordinator {self.coordinator} is gone, stopping", flush=True)
                            break
                        continue
                sender, data = item
                if int.from_bytes(data[:2], "little") == config_transfer:  # a message opens with its u16 command
                    self.coordinator = sender
                t0 = time.perf_counter()
                replies = self.worker.handle(data)
                if self.log is not None:
                    cmd = H.command_name(int.from_bytes(data[:2], "little"))
                    self._updates += cmd == "UPDATE_PARAMETERS"
                    mem = 0
                    if self.worker.device != "cpu":
                        import torch
                        mem = int(torch.cuda.memory_allocated())
                    self.log.log(self._updates, cmd, round((time.perf_counter() - t0) * 1e3, 3), mem)
                for dst, reply in replies:
                    target = self.coordinator if dst == COORDINATOR else dst
                    if target is None:
                        raise RuntimeError("a reply for the coordinator before any CONFIG_TRANSFER named one")
                    try:
                        self.transport.send(target, reply)
                    except RuntimeError as e:
                        if target == self.coordinator:
                            raise  # nobody left to report to
                        # a neighbour is gone: tell the coordinator instead of dying silently (the reference drops
                        # the channel and keeps waiting, tcp_communicator.hpp:359-393)
                        self.transport.send(self.coordinator, simple_message(
                            "ERROR_REPORT", text=f"{self.name}: cannot deliver to {target}: {e}"))
                n += 1
        finally:
            self.transport.close()
            if self.log is not None:
                self.log.close()
        return n


def tcp_coordinator(graph, ratios: Sequence[float], endpoints: Sequence[str], optimizer_cfg: dict,
                    scheduler_cfg: Optional[dict] = None, loss_cfg: Optional[dict] = None, microbatches: int = 2,
                    host: str = "127.0.0.1", port: int = 0, sockets_per_endpoint: int = 4,
                    max_packet_size: int = 4 << 20) -> LocalCoordinator:
    """Partitions ``graph`` by ``ratios`` and deploys stage ``i`` to the worker listening at ``endpoints[i]``."""
    t = TcpTransport(host, port, sockets_per_endpoint, max_packet_size)
    try:
        return LocalCoordinator(graph, ratios, optimizer_cfg, scheduler_cfg, loss_cfg, microbatches, transport=t,
                                endpoints=[_canonical(e) for e in endpoints])
    except Exception:
        t.close()
        raise


def _canonical(endpoint: str) -> str:
    """Endpoints are named by numeric address, as the accepting side sees them."""
    import socket

    host, port = split_endpoint(endpoint)
    return f"{socket.gethostbyname(host)}:{port}"


def ping_pong(transport: TcpTransport, peer: str, message_bytes: int, seconds: float) -> dict:
    """Bandwidth of round trips of one ``message_bytes`` message with an echoing peer (the reference's
    benchmarks/tcp_communicator_benchmark.cpp:132-223 sends 128 MiB tensors for 10 s and prints MB/s)."""
    # The loop runs inside the C++ communicator (one buffer sent again and again, the echoes received into the
    # reassembly buffer and dropped), so the figure is the communicator's, not the interpreter's.
    if not transport.comm.connected(peer):
        host, port = split_endpoint(peer)
        transport.comm.connect(host, port, 30.0)
    n, dt = transport.comm.ping_pong(peer, int(message_bytes), float(seconds))
    return {"round_trips": int(n), "seconds": dt, "mb_per_s_each_way": n * message_bytes / dt / 1e6}


def echo_until_shutdown(transport: TcpTransport) -> int:
    """The peer of :func:`ping_pong`: sends every message back; a 6-byte ``SHUTDOWN`` message ends it."""
    return int(transport.comm.echo(simple_message("SHUTDOWN")))


def main(argv=None) -> int:
    """``python -m tnn_b200.parallel.tcp_transport worker [--host H] [--port P] [--device D]`` runs one stage worker
    (the reference's ``tcp_worker``); ``echo`` runs the peer of the ping-pong benchmark. Either prints
    ``listening <ip:port>`` first, so that a launcher can read the endpoint when the port was chosen by the system."""
    import argparse

    ap = argparse.ArgumentParser(prog="tnn_b200.parallel.tcp_transport")
    ap.add_argument("role", choices=["worker", "echo"])
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--sockets", type=int, default=4)
    ap.add_argument("--max-packet", type=int, default=4 << 20)
    ap.add_argument("--idle-timeout", type=float, default=-1.0, help="worker: give up after this many idle seconds")
    ap.add_argument("--log", default="", help="worker: CSV file for its per-message log (step,event_type,time_ms,mem)")
    a = ap.parse_args(argv)
    if a.role == "worker":
        srv = TcpStageServer(a.host, a.port, a.device, a.sockets, a.max_packet, a.log)
        print("listening", srv.name, flush=True)
        n = srv.serve(a.idle_timeout)
        print(f"{srv.name}: handled {n} messages", flush=True)
    else:
        t = TcpTransport(a.host, a.port, a.sockets, a.max_packet)
        print("listening", t.name, flush=True)
        n = echo_until_shutdown(t)
        t.close()
        print(f"{t.name}: echoed {n} messages", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
