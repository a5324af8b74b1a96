"""Failure detection on the host: heartbeats, watchdog, fault plan, checkpoint corruption, and a 3-process gloo job in
which one rank leaves between steps. No GPU is involved and nothing is made to hang: every wait has a timeout."""
import json
import os
import socket
import subprocess
import sys
import time

import pytest
import torch
import torch.distributed as dist

from tnn_b200.parallel import health

HERE = os.path.dirname(os.path.abspath(__file__))


def test_watchdog_reports_silent_rank_with_fake_clock():
    store = dist.HashStore()
    now = [100.0]
    clock = lambda: now[0]
    hb = [health.Heartbeat(store, r, clock=clock) for r in range(3)]
    for h in hb:
        h.beat()
    wd = health.Watchdog(store, 0, 3, timeout=2.0, clock=clock)
    wd.check()
    now[0] += 1.5
    hb[1].beat()  # rank 1 keeps beating, rank 2 went silent
    now[0] += 1.0
    assert wd.dead_ranks() == [2]
    with pytest.raises(health.RankFailure) as e:
        wd.check()
    assert e.value.dead == [2] and e.value.ages[2] > 2.0
    hb[2].beat()  # it comes back (e.g. a paused process resumed)
    wd.check()


def test_muted_heartbeat_and_step_watchdog():
    store = dist.HashStore()
    now = [0.0]
    clock = lambda: now[0]
    h = health.Heartbeat(store, 1, clock=clock)
    h.beat()
    h.mute(True)
    now[0] += 10
    h.beat()  # dropped
    wd = health.Watchdog(store, 0, 2, timeout=5.0, step_timeout=3.0, clock=clock)
    assert wd.dead_ranks() == [1]
    h.mute(False)
    h.beat()
    wd.step_begin()
    now[0] += 4
    with pytest.raises(health.StepTimeout):
        wd.check()
    wd.step_end()
    wd.check()


def test_fault_plan_parsing_and_firing(monkeypatch):
    monkeypatch.setenv("TNNB_FAULT", "raise:rank=1:step=2")
    plan = health.FaultPlan.from_env()
    assert (plan.kind, plan.rank, plan.step) == ("raise", 1, 2)
    plan.maybe_fire(0, 2)
    plan.maybe_fire(1, 1)
    with pytest.raises(health.InjectedFault):
        plan.maybe_fire(1, 2)
    plan.maybe_fire(1, 2)  # fires once
    t0 = time.time()
    health.FaultPlan("stall", 0, 0, seconds=0.2).maybe_fire(0, 0)
    assert time.time() - t0 >= 0.19


def test_corrupt_checkpoint_is_rejected_and_previous_one_found(tmp_path):
    from tnn_b200.models import zoo
    from tnn_b200.nn.graph import Graph

    g = zoo.gpt2(32, 1, 1, "t", seq_len=16, vocab=31, drop=0.0).compile(device="cpu", seed=0)
    a, b = str(tmp_path / "a.tnng"), str(tmp_path / "b.tnng")
    g.save_state(a)
    time.sleep(0.05)
    g.save_state(b)
    os.utime(b, (time.time() + 5, time.time() + 5))
    assert health.find_latest_snapshot(str(tmp_path)) == b
    health.corrupt_file(b, offset=0, nbytes=8)  # destroys the magic / version
    with pytest.raises(Exception):
        Graph.load_state(b, device="cpu")
    assert health.find_latest_snapshot(str(tmp_path)) == a
    # truncation must fail cleanly too
    with open(a, "rb") as f:
        data = f.read()
    with open(b, "wb") as f:
        f.write(data[: len(data) // 2])
    with pytest.raises(Exception):
        Graph.load_state(b, device="cpu")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_lost_rank_is_detected_and_job_resumes_from_snapshot(tmp_path):
    world = 3
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE=str(world), HEALTH_PORT=str(_free_port()),
               TNNB_FAULT="exit:rank=2:step=3")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "_health_worker.py"), str(tmp_path)], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=120)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0])
            pytest.fail("worker did not finish: " + outs[-1][-1500:])
    assert procs[2].returncode == 17, outs[2][-1500:]          # the injected exit
    for r in (0, 1):
        assert procs[r].returncode == 0, outs[r][-1500:]
        res = json.load(open(tmp_path / f"result_{r}.json"))
        assert res["detected"] == [2], res                      # learnt on the host, no hung collective
        assert 3 <= res["steps"] < 8
    # recovery: a new single-process job restarts from the snapshot rank 0 wrote after step 2
    from tnn_b200.models import zoo
    from tnn_b200.trainer import Trainer
    from tnn_b200.utils.config import TrainingConfig

    snap = health.find_latest_snapshot(str(tmp_path))
    assert snap and snap.endswith("ckpt_step2.tnng")
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(32, 1, 1, "t", seq_len=16, vocab=31, drop=0.0))
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 2, "device_type": "CPU",
                                    "optimizer": {"type": "sgd", "learning_rate": 0.05}})
    t = Trainer(cfg, log=False)
    t.load_snapshot(snap)
    seq = torch.randint(0, 31, (2, 17))
    loss = t.train_step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous())
    assert torch.isfinite(loss)
