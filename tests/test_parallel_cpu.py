"""Multi-process (gloo, CPU) checks of the parallel runtime's host logic and math: data parallel and
tensor parallel training steps must reproduce the single-process run on the combined batch."""
import os
import subprocess
import sys

import torch

from tnn_b200.models import zoo
from tnn_b200.parallel.runtime import default_layout, parse_layout
from tnn_b200.trainer import Trainer
from tnn_b200.utils.config import TrainingConfig

HERE = os.path.dirname(os.path.abspath(__file__))


def launch(n, mode, out, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_cpu_parallel_worker.py"), mode, out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return torch.load(out, weights_only=False)


def reference(batches):
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(128, 2, 2, "t", seq_len=128, vocab=97, drop=0.0))
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 2, "device_type": "CPU", "seed": 5,
                                    "optimizer": {"type": "sgd", "learning_rate": 0.1, "momentum": 0.9}})
    t = Trainer(cfg, log=False)
    losses = [float(t.train_step(s[:, :-1].contiguous(), s[:, 1:].contiguous()).item()) for s in batches]
    g = t.graph
    t.close()
    return losses, g


def test_layout_strings():
    assert parse_layout("pp4tp2") == {"dp": 1, "tp": 2, "pp": 4}
    assert default_layout(8, "gpt2_small") == "dp8" and default_layout(1, "gpt2_small") == "single"
    assert default_layout(4, "imagenet_resnet50") == "dp4"


def test_dp2_equals_single_process(tmp_path):
    res = launch(2, "dp", str(tmp_path / "dp.pt"), 29621)
    gens = [torch.Generator().manual_seed(100 + r) for r in range(2)]
    batches = [torch.cat([torch.randint(0, 97, (2, 129), generator=g) for g in gens]) for _ in range(3)]
    ref_losses, g = reference(batches)
    assert torch.allclose(res["masters"][0], res["masters"][1])
    assert torch.allclose(res["masters"][0], g.master_flat, atol=2e-4), float((res["masters"][0] - g.master_flat).abs().max())
    mean_loss = [(a + b) / 2 for a, b in zip(*res["losses"])]
    assert all(abs(a - b) < 1e-3 for a, b in zip(mean_loss, ref_losses))


def test_tp2_equals_single_process(tmp_path):
    res = launch(2, "tp", str(tmp_path / "tp.pt"), 29622)
    gen = torch.Generator().manual_seed(100)
    batches = [torch.randint(0, 97, (2, 129), generator=gen) for _ in range(3)]
    ref_losses, g = reference(batches)
    mean_loss = [(a + b) / 2 for a, b in zip(*res["losses"])]
    assert all(abs(a - b) < 2e-3 for a, b in zip(mean_loss, ref_losses)), (mean_loss, ref_losses)
    # a replicated parameter (final layernorm gamma) and a sharded one (fc1 weight rows) after 3 steps
    full = {l.name: l for l in g.layers()}
    lay = res["layout"]
    o, n, shape, _ = lay["ln_f"][0]
    assert torch.allclose(res["masters"][0][o:o + n], full["ln_f"].params[0].reshape(-1), atol=2e-3)
    o, n, shape, _ = lay["t_block_0_mlp_fc1"][0]
    got = torch.cat([m[o:o + n].view(shape) for m in res["masters"]], 0)
    assert torch.allclose(got, full["t_block_0_mlp_fc1"].params[0], atol=2e-3), float((got - full["t_block_0_mlp_fc1"].params[0]).abs().max())
    # the gathered checkpoint is an ordinary TNNG file of the unsharded model: every parameter matches the reference run
    from tnn_b200.nn.graph import Graph
    loaded = Graph.load_state(str(tmp_path / "tp.pt") + ".tnng", device="cpu")
    ref_layers = {l.name: l for l in g.layers()}
    n_checked = 0
    for l in loaded.layers():
        for a, b in zip(l.params, ref_layers[l.name].params):
            assert a.shape == b.shape and torch.allclose(a.float(), b.float(), atol=3e-3), l.name
            n_checked += 1
    assert n_checked > 20


def test_snapshot_with_optimizer_resumes_exactly(tmp_path):
    """A data-parallel and a tensor-parallel job each write a snapshot with optimizer state after three steps; a
    second trainer that loads it must reproduce the next two steps bit for bit (weights, AdamW moments, bias
    correction step, scheduler position). The data-parallel job leaves the same ``.opt`` sidecar a single process
    writes, the tensor-parallel one a sidecar per rank."""
    for mode, port in (("resume_dp", 29624), ("resume_tp", 29625)):
        res = launch(2, mode, str(tmp_path / f"{mode}.pt"), port)
        for st in res:
            assert st["step"][0] == st["step"][1] == 3 and st["global"][0] == st["global"][1], st
            assert st["lr"][0] == st["lr"][1] and st["lr"][0] < 1e-2, st      # the scheduler had stepped twice
            assert st["diff"] < 1e-7 and st["moved"] > 1e-3, st
        names = res[0]["sidecars"]
        if mode == "resume_dp":
            assert any(n.endswith(".tnng.opt") for n in names), names
        else:
            assert sum(".opt.rank" in n for n in names) == 2, names


def test_grad_hook_order_and_bucket_plan():
    """Backward reports final gradient ranges from the end of the flat buffer; the bucket plan follows that order."""
    import torch
    from tnn_b200.models import zoo
    from tnn_b200.parallel.dp import plan_buckets

    g = zoo.gpt2(128, 2, 3, "t", seq_len=64, vocab=203, drop=0.0).compile(device="cpu", seed=1)
    assert g.grad_hook_usable()
    pts = g.grad_ready_points()
    assert pts == sorted(pts, reverse=True) and pts[-1] == 0
    fired = []
    written = []

    def hook(floor):
        fired.append(floor)
        # at the time of the call the gradients at offsets >= floor must already hold their final values
        written.append(g.grads_flat[floor:].clone())

    g.grad_hook = hook
    g.train()
    ids = torch.randint(0, 203, (2, 64))
    out = g(ids)
    g.backward({"output": torch.ones_like(out)})
    assert fired == pts
    for floor, snap in zip(fired, written):
        assert torch.equal(snap, g.grads_flat[floor:])
    total = g.total_elems
    plan = plan_buckets(pts, 0, total, n_buckets=3, min_bucket=8)
    assert plan[0][1] == total and plan[-1][0] == 0
    assert all(a[0] == b[1] for a, b in zip(plan, plan[1:]))          # contiguous, descending
    assert all(lo % 8 == 0 for lo, _ in plan) and len(plan) >= 2
    assert all(lo in [p // 8 * 8 for p in pts] for lo, _ in plan)        # every boundary is a reported point
    assert plan_buckets(pts, 0, total, n_buckets=1, min_bucket=8) == [(0, total)]
    # a ResNet: many segments, floors still descend
    r = zoo.create("cifar10_resnet9").compile(device="cpu", seed=1)
    assert r.grad_hook_usable()
    rp = r.grad_ready_points()
    assert rp == sorted(rp, reverse=True)
