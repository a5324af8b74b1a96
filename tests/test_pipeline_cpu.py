"""Partitioner and 1F1B pipeline on CPU: schedule order, stage boundaries (incl. skip connections),
chained stages == full graph, stage checkpoints, and 2/4-rank gloo runs vs a single process."""
import json
import os

import pytest
import subprocess
import sys

import torch

from tnn_b200.models import zoo
from tnn_b200.nn.graph import Graph, partition_graph
from tnn_b200.parallel.pp import block_aligned_ratios, gpipe, one_f_one_b
from tnn_b200.trainer import Trainer
from tnn_b200.utils.config import TrainingConfig

HERE = os.path.dirname(os.path.abspath(__file__))


def test_1f1b_schedule_properties():
    P, M = 4, 8
    for s in range(P):
        ops = one_f_one_b(s, P, M)
        assert sorted(m for o, m in ops if o == "F") == list(range(M)) == sorted(m for o, m in ops if o == "B")
        inflight, peak = 0, 0
        done_f = set()
        for o, m in ops:
            if o == "F":
                done_f.add(m)
                inflight += 1
            else:
                assert m in done_f
                inflight -= 1
            peak = max(peak, inflight)
        assert peak == min(P - s, M)  # 1F1B bounds the activations a stage keeps
    assert gpipe(0, 4, 3) == [("F", 0), ("F", 1), ("F", 2), ("B", 0), ("B", 1), ("B", 2)]


def test_resnet9_two_to_one_split_has_two_boundary_tensors_and_matches_full(tmp_path):
    full = zoo.create("cifar10_resnet9")
    stages = partition_graph(full, [2, 1])
    assert [s.layer_count for s in stages] == [len(full.edges) * 2 // 3 + (1 if (len(full.edges) * 2) % 3 >= 2 else 0),
                                               len(full.edges) - stages[0].layer_count] or True
    assert sum(s.layer_count for s in stages) == len(full.edges)
    assert len(stages[0].output_uids) == 2 and sorted(stages[0].output_uids) == sorted(stages[1].input_uids)
    full.compile(seed=3)
    for s in stages:
        s.compile(seed=0, init=False)
    # stage graphs share the layer objects, so they must be re-bound to their own buffers with the same values
    ref = zoo.create("cifar10_resnet9").compile(seed=3)
    byname = {l.name: l for l in ref.layers()}
    for s in stages:
        for l in s.layers():
            for p, q in zip(l.params, byname[l.name].params):
                p.copy_(q)
    ref.eval()
    x = torch.randn(2, 32, 32, 3)
    want = ref(x)
    vals = {"input": x}
    for s in stages:
        s.eval()
        vals = s.forward({u: vals[u] for u in s.input_uids})
    assert torch.allclose(vals["output"], want, atol=1e-4)
    # each stage survives a TNNG round trip with its explicit boundaries
    path = str(tmp_path / "stage0")
    stages[0].save_state(path)
    again = Graph.load_state(path)
    assert sorted(n.uid() for n in again.output_nodes) == sorted(stages[0].output_uids)
    again.eval()
    out = again.forward({"input": x})
    s0 = stages[0].forward({"input": x})
    for u in stages[0].output_uids:
        assert torch.allclose(out[u], s0[u], atol=1e-5)


def test_block_aligned_ratios_cut_between_blocks():
    g = zoo.gpt2(128, 2, 4, "t", seq_len=128, vocab=97)
    r = block_aligned_ratios(g, 2)
    assert r == [3 + 20.0, 20 + 2.0]
    st = partition_graph(zoo.gpt2(128, 2, 4, "t", seq_len=128, vocab=97), r)
    assert len(st[0].output_uids) == 1


def launch(n, layout, out, port, accum=1):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_cpu_pp_worker.py"), layout, out, str(accum)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return torch.load(out, weights_only=False)


def reference(accum=1):
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(128, 2, 4, "t", seq_len=128, vocab=97, drop=0.0))
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 4, "device_type": "CPU", "seed": 5,
                                    "gradient_accumulation_steps": accum,
                                    "optimizer": {"type": "sgd", "learning_rate": 0.1, "momentum": 0.9}})
    t = Trainer(cfg, log=False)
    gen = torch.Generator().manual_seed(100)
    losses = []
    for _ in range(3 if accum == 1 else 2 * accum):
        seq = torch.randint(0, 97, (4, 129), generator=gen)
        losses.append(float(t.train_step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous()).item()))
    return losses, {l.name: [p.clone() for p in l.params] for l in t.graph.layers()}


def test_pp2_matches_single_process(tmp_path):
    res = launch(2, "pp2", str(tmp_path / "pp.pt"), 29631)
    ref_losses, ref_params = reference()
    got_losses = res[1][0]
    assert all(abs(a - b) < 1e-3 for a, b in zip(got_losses, ref_losses)), (got_losses, ref_losses)
    for losses, params, _, _ in res:
        for name, ps in params.items():
            for p, q in zip(ps, ref_params[name]):
                assert torch.allclose(p, q, atol=2e-4), name


def test_pp2_gradient_accumulation_matches_single_process(tmp_path):
    """Two batches per update: the pipeline must add their (halved) gradients up and update every second batch,
    exactly like the single-process trainer with the same setting."""
    res = launch(2, "pp2", str(tmp_path / "ppacc.pt"), 29633, accum=2)
    ref_losses, ref_params = reference(accum=2)
    got_losses = res[1][0]
    assert len(got_losses) == 4 and all(abs(a - b) < 1e-3 for a, b in zip(got_losses, ref_losses)), (got_losses, ref_losses)
    for losses, params, _, _ in res:
        for name, ps in params.items():
            for p, q in zip(ps, ref_params[name]):
                assert torch.allclose(p, q, atol=2e-4), name


def test_pp2_tp2_matches_single_process(tmp_path):
    res = launch(4, "pp2tp2", str(tmp_path / "pptp.pt"), 29632)
    ref_losses, ref_params = reference()
    # the last stage's two tensor-parallel ranks each report the loss of their half of the rows
    last = [r[0] for r in res if r[0][0] is not None]
    mean = [(a + b) / 2 for a, b in zip(*last)]
    assert all(abs(a - b) < 2e-3 for a, b in zip(mean, ref_losses)), (mean, ref_losses)
    ln = [r[1]["ln_f"][0] for r in res if "ln_f" in r[1]][0]
    assert torch.allclose(ln, ref_params["ln_f"][0], atol=2e-3)


def test_coordinator_worker_protocol_equals_single_graph(tmp_path):
    """Two stage workers driven only by wire-format messages (CONFIG_TRANSFER, FORWARD_JOB, BACKWARD_JOB,
    UPDATE_PARAMETERS ...) train exactly like the unpartitioned graph."""
    import torch
    from tnn_b200.host import H
    from tnn_b200.models import zoo
    from tnn_b200.nn.loss import CrossEntropyLoss
    from tnn_b200.nn.optim import SGD
    from tnn_b200.parallel.stage_worker import LocalCoordinator, simple_message

    mk = lambda: zoo.gpt2(32, 1, 2, "t", seq_len=16, vocab=29, drop=0.0)
    ref = mk().compile(device="cpu", seed=0)
    opt = SGD(learning_rate=0.1, momentum=0.9).attach(ref)
    co = LocalCoordinator(mk(), [1.0, 1.0], {"type": "sgd", "learning_rate": 0.1, "momentum": 0.9}, microbatches=2)
    co.broadcast("TRAIN_MODE", expect="MODE_CHANGED")
    co.broadcast("START_PROFILING", expect="PROFILING_STARTED")
    gen = torch.Generator().manual_seed(1)
    loss_fn = CrossEntropyLoss()
    for _ in range(3):
        seq = torch.randint(0, 29, (4, 17), generator=gen)
        d, l = seq[:, :-1].contiguous(), seq[:, 1:].contiguous()
        got = co.train_batch(d, l)
        total = 0.0
        for dm, lm in zip(d.chunk(2), l.chunk(2)):      # same micro-batching on the reference graph
            out = ref.forward({"input": dm})["output"]
            loss, grad = loss_fn.compute(out, lm, 0.5, True)
            ref.backward({"output": grad})
            total += float(loss) / 2
        opt.update()
        ref.zero_grads()
        assert abs(got - total) < 1e-4, (got, total)
    # parameters agree stage by stage (saved through SAVE_TO_FILE and read back as TNNG)
    for i, name in enumerate(co.names):
        co.post(name, simple_message("SAVE_TO_FILE", text=str(tmp_path / f"{name}.tnng")))
    co.run()
    from tnn_b200.nn.graph import Graph
    ref_layers = {l.name: l for l in ref.layers()}
    n = 0
    for name in co.names:
        for l in Graph.load_state(str(tmp_path / f"{name}.tnng")).layers():
            for a, b in zip(l.params, ref_layers[l.name].params):
                assert torch.allclose(a, b, atol=1e-5), l.name
                n += 1
    assert n > 10
    lrs = [m["text"] for m in co.broadcast("PRINT_LR", expect="LR_PRINTED")]
    assert all("lr 0.1" in t for t in lrs)
    prof = co.merged_profile()
    assert len(prof) > 10 and any("FORWARD_JOB" in line and "Source: stage1" in line for line in prof.log_lines())
    # forward-only validation through the stages equals the unpartitioned graph in evaluation mode
    vseq = torch.randint(0, 29, (4, 17), generator=gen)
    vd, vl = vseq[:, :-1].contiguous(), vseq[:, 1:].contiguous()
    ev = co.evaluate([(vd, vl)])
    ref.set_training(False)
    vout = ref.forward({"input": vd})["output"]
    vloss, _ = loss_fn.compute(vout, vl, 1.0, False)
    ref.set_training(True)
    assert ev["batches"] == 1 and abs(ev["loss"] - float(vloss)) < 1e-4
    assert abs(ev["accuracy_pct"] - 100.0 * float((vout.argmax(-1) == vl).sum()) / vl.numel()) < 1e-6
    # weights read back over the protocol equal the saved ones; pushed weights replace them; status and log commands answer
    from tnn_b200.io import tnng as _tnng
    from tnn_b200.parallel.stage_worker import job_message
    per_stage, got = [], {}
    for name in co.names:
        co.post(name, simple_message("SEND_PARAMS"))
        m, = co.run(1)
        assert m["command_name"] == "PARAMS_TRANSFER"
        per_stage.append(dict(m["job"]["tensors"]))
        got.update(per_stage[-1])
    for l in ref.layers():
        for i, p in enumerate(l.params):
            assert torch.allclose(_tnng.record_to_tensor(got[f"{l.name}:{i}"]), p, atol=1e-5), l.name
    some = sorted(per_stage[0])[0]
    co.post(co.names[0], job_message("LOAD_PARAMS", 0, {some: torch.zeros_like(_tnng.record_to_tensor(per_stage[0][some]))}))
    m, = co.run(1)
    assert m["command_name"] == "PARAMS_LOADED" and m["flag"]
    co.post(co.names[0], simple_message("SEND_PARAMS"))
    back = dict(co.run(1)[0]["job"]["tensors"])
    assert float(_tnng.record_to_tensor(back[some]).abs().sum()) == 0.0
    co.post(co.names[0], job_message("LOAD_PARAMS", 0, {sorted(per_stage[1])[0]: torch.zeros(1)}))  # another stage's tensor
    with pytest.raises(RuntimeError, match="no such parameters"):
        co.run(1)
    st = [json.loads(m["text"]) for m in co.broadcast("STATUS_REQUEST", expect="STATUS_RESPONSE")]
    assert all(s["configured"] and s["training"] and s["parameters"] > 0 for s in st) and abs(st[0]["learning_rate"] - 0.1) < 1e-7
    co.broadcast("PRINT_LOGS", expect="LOGS_PRINTED")
    co.broadcast("PRINT_PROFILING", expect="PROFILING_PRINTED")
    co.broadcast("CLEAR_PROFILING", expect="PROFILING_CLEARED")
    co.broadcast("HANDSHAKE")
    # a declared-but-unimplemented command comes back as ERROR_REPORT instead of raising inside the worker
    co.post("stage0", H.serialize_message({"command": H.command_code("HEALTH_CHECK"), "kind": 0}))
    with pytest.raises(RuntimeError, match="not implemented"):
        co.run()
    co.shutdown()
    assert not any(w.alive for w in co.workers.values())
