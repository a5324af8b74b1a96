"""TCP transport of the coordinator / worker protocol: the C++ communicator over loopback, then two worker
processes trained by a coordinator in this process against the unpartitioned graph."""
import os
import subprocess
import sys

import pytest
import torch

from tnn_b200.host import H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _spawn(role, *extra):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), OMP_NUM_THREADS="2")
    p = subprocess.Popen([sys.executable, "-m", "tnn_b200.parallel.tcp_transport", role, *extra], stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True, env=env, cwd=ROOT)
    line = p.stdout.readline().split()
    assert line[:1] == ["listening"], line
    return p, line[1]


def test_communicator_loopback_large_and_small_messages():
    a, b = H.TcpCommunicator("127.0.0.1", 0, 3, 64 << 10), H.TcpCommunicator("127.0.0.1", 0, 3, 64 << 10)
    a.start()
    pb = b.start()
    try:
        peer = a.connect("127.0.0.1", pb)
        assert peer == b.endpoint() and a.connected(peer) and not a.connected("127.0.0.1:1")
        big = os.urandom(5 * (64 << 10) + 13)  # 6 packets over 3 sockets, the last one short
        for m in (big, b"", b"x" * (64 << 10), b"tail"):
            a.send(peer, m)
        got = [b.recv(20.0) for _ in range(4)]
        assert all(g is not None and g[0] == a.endpoint() for g in got)  # named by the handshake, not by the socket's port
        assert sorted(g[1] for g in got) == sorted([big, b"", b"x" * (64 << 10), b"tail"])
        b.send(a.endpoint(), b"reply over the accepted sockets")
        assert a.recv(20.0) == (b.endpoint(), b"reply over the accepted sockets")
        assert b.recv(0.05) is None
        st = a.stats()
        assert st["messages_sent"] == 4 and st["bytes_sent"] == len(big) + (64 << 10) + 4 + 9 * H.PACKET_HEADER_SIZE
        with pytest.raises(RuntimeError, match="no connection"):
            a.send("127.0.0.1:1", b"nobody")
    finally:
        a.stop()
        b.stop()
    assert a.recv(0.01) is None  # a stopped communicator returns at once


def test_communicator_destroyed_with_packets_queued():
    import gc

    a, b = H.TcpCommunicator("127.0.0.1", 0, 2, 1 << 20), H.TcpCommunicator("127.0.0.1", 0, 2, 1 << 20)
    a.start()
    peer = a.connect("127.0.0.1", b.start())
    for _ in range(6):
        a.send(peer, bytes(8 << 20))  # the packets point into these bytes objects until they are written
    del a  # no stop(): the destructor joins the threads and releases what is still queued
    gc.collect()
    b.stop()


def test_aggregator_reserve_commit_matches_feed():
    msg = os.urandom(1000)
    pk = H.slice_message(msg, 7, 300)
    agg = H.Aggregator()
    out = [agg.feed(p) for p in (pk[2], pk[0], pk[0], pk[3], pk[1])]  # any order, one repeated
    assert out[:-1] == [None] * 4 and out[-1] == (7, msg) and agg.pending() == 0


def test_pipeline_over_tcp_matches_single_process(tmp_path):
    from tnn_b200.models import zoo
    from tnn_b200.nn.graph import Graph
    from tnn_b200.nn.loss import CrossEntropyLoss
    from tnn_b200.nn.optim import SGD
    from tnn_b200.parallel.stage_worker import simple_message
    from tnn_b200.parallel.tcp_transport import tcp_coordinator

    logs = [str(tmp_path / f"worker{i}.csv") for i in range(2)]
    procs = [_spawn("worker", "--idle-timeout", "120", "--log", logs[i]) for i in range(2)]
    co = None
    try:
        mk = lambda: zoo.gpt2(32, 1, 2, "t", seq_len=16, vocab=29, drop=0.0)
        ref = mk().compile(device="cpu", seed=0)
        opt = SGD(learning_rate=0.1, momentum=0.9).attach(ref)
        # 32 KiB packets: every activation message (2 x 16 x 32 fp32 + framing) and the stage states are cut up
        co = tcp_coordinator(mk(), [1.0, 1.0], [e for _, e in procs], {"type": "sgd", "learning_rate": 0.1, "momentum": 0.9},
                             microbatches=2, max_packet_size=32 << 10)
        co.reply_timeout_s = 120.0
        co.broadcast("TRAIN_MODE", expect="MODE_CHANGED")
        gen = torch.Generator().manual_seed(1)
        loss_fn = CrossEntropyLoss()
        for _ in range(3):
            seq = torch.randint(0, 29, (4, 17), generator=gen)
            d, l = seq[:, :-1].contiguous(), seq[:, 1:].contiguous()
            got = co.train_batch(d, l)
            total = 0.0
            for dm, lm in zip(d.chunk(2), l.chunk(2)):
                out = ref.forward({"input": dm})["output"]
                loss, grad = loss_fn.compute(out, lm, 0.5, True)
                ref.backward({"output": grad})
                total += float(loss) / 2
            opt.update()
            ref.zero_grads()
            assert abs(got - total) < 1e-4, (got, total)
        files = [str(tmp_path / f"stage{i}.tnng") for i in range(2)]
        for name, f in zip(co.names, files):
            co.post(name, simple_message("SAVE_TO_FILE", text=f))
        lrs = [m["text"] for m in co.broadcast("PRINT_LR", expect="LR_PRINTED")]  # answered after the save: same socket order per worker
        assert len(lrs) == 2 and all("lr 0.1" in t for t in lrs)
        ref_layers = {l.name: l for l in ref.layers()}
        n = 0
        for f in files:
            for l in Graph.load_state(f).layers():
                for a, b in zip(l.params, ref_layers[l.name].params):
                    assert torch.allclose(a, b, atol=1e-5), l.name
                    n += 1
        assert n > 10
        co.shutdown()
        co.transport.close()
        co = None
        for p, _ in procs:
            assert p.wait(timeout=60) == 0, p.stdout.read()
        for f in logs:  # the worker's own event log: header, then one row per handled message
            rows = open(f).read().strip().split("\n")
            assert rows[0] == "step,event_type,time_ms,mem"
            kinds = [r.split(",")[1] for r in rows[1:]]
            assert kinds[0] == "CONFIG_TRANSFER" and kinds.count("FORWARD_JOB") == 6 and kinds.count("UPDATE_PARAMETERS") == 3
            assert rows[-1].split(",")[0] == "3" and kinds[-1] == "SHUTDOWN"
    finally:
        if co is not None:
            co.transport.close()
        for p, _ in procs:
            if p.poll() is None:
                p.kill()


def test_coordinator_notices_a_dead_worker():
    """Failure detection on the host: a worker process is killed between steps; the coordinator's next step ends
    with ConnectionError within seconds instead of waiting out the reply timeout."""
    import time

    from tnn_b200.models import zoo
    from tnn_b200.parallel.tcp_transport import tcp_coordinator

    procs = [_spawn("worker", "--idle-timeout", "60") for _ in range(2)]
    co = None
    try:
        co = tcp_coordinator(zoo.gpt2(32, 1, 2, "t", seq_len=16, vocab=29, drop=0.0), [1.0, 1.0], [e for _, e in procs],
                             {"type": "sgd", "learning_rate": 0.1}, microbatches=2)
        co.reply_timeout_s = 60.0
        co.broadcast("TRAIN_MODE", expect="MODE_CHANGED")
        seq = torch.randint(0, 29, (4, 17), generator=torch.Generator().manual_seed(1))
        co.train_batch(seq[:, :-1].contiguous(), seq[:, 1:].contiguous())
        procs[1][0].kill()
        procs[1][0].wait(timeout=30)
        t0 = time.monotonic()
        with pytest.raises((ConnectionError, RuntimeError), match="lost the connection|cannot deliver"):
            co.train_batch(seq[:, :-1].contiguous(), seq[:, 1:].contiguous())
        assert time.monotonic() - t0 < 20.0
        assert procs[0][0].poll() is None  # the surviving worker reported the failure and is still serving
    finally:
        if co is not None:
            co.transport.close()
        for p, _ in procs:
            if p.poll() is None:
                p.kill()


def test_workers_stop_when_the_coordinator_disappears():
    """No SHUTDOWN is ever sent: the coordinator's sockets just close; workers that wait without an idle limit
    notice it and exit instead of serving nobody for ever."""
    from tnn_b200.models import zoo
    from tnn_b200.parallel.tcp_transport import tcp_coordinator

    procs = [_spawn("worker") for _ in range(2)]
    try:
        co = tcp_coordinator(zoo.gpt2(32, 1, 2, "t", seq_len=16, vocab=29, drop=0.0), [1.0, 1.0], [e for _, e in procs],
                             {"type": "sgd", "learning_rate": 0.1}, microbatches=2)
        co.broadcast("TRAIN_MODE", expect="MODE_CHANGED")
        co.transport.close()
        for p, _ in procs:
            assert p.wait(timeout=30) == 0
            assert "coordinator" in p.stdout.read()
    finally:
        for p, _ in procs:
            if p.poll() is None:
                p.kill()
