"""Multi-GPU tests (need >= 2 GPUs): fused NVLink kernels vs the NCCL baseline vs one process."""
import json
import os
import subprocess
import sys

import pytest
import torch

from tnn_b200.models import zoo
from tnn_b200.trainer import Trainer
from tnn_b200.utils.config import TrainingConfig

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def launch(n, mode, kind, out):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(HERE, "_parallel_worker.py"), mode, kind, out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, "\n".join(l for l in r.stdout.splitlines() if "WORKER-ERROR" in l or "Error" in l)[:3000] + r.stdout[-2500:] + r.stderr[-500:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[7:])


def single_process_reference(global_batch_sets, tmp, optimizer=None, device="CUDA"):
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(128, 2, 2, "t", seq_len=128, vocab=203, drop=0.0))
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 4, "device_type": device, "seed": 5,
                                    "optimizer": optimizer or {"type": "adamw", "learning_rate": 1e-2, "weight_decay": 0.01}})
    t = Trainer(cfg, log=False)
    losses = []
    for seq in global_batch_sets:
        losses.append(float(t.train_step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous()).item()))
    p = (t.graph.master_flat if optimizer is not None else t.graph.params_flat).float().cpu()  # fp32 master on request
    t.close()
    return losses, p


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("kind", ["fused", "nccl"])
def test_dp2_matches_single_process(kind, tmp_path):
    out = str(tmp_path / "dp.pt")
    res = launch(2, "dp", kind, out)
    assert res["max_rank_diff"] == 0.0
    if kind == "fused":  # the fused path ran bucketed, overlapped with backward
        assert res["dp_overlap"] and res["dp_sites"] > 1, res
    gens = [torch.Generator().manual_seed(100 + r) for r in range(2)]
    sets = [torch.cat([torch.randint(0, 203, (2, 129), generator=g) for g in gens]) for _ in range(4)]
    ref_losses, ref_params = single_process_reference(sets, tmp_path)
    got = torch.load(out)
    # rank 0 reports the loss of its half of the batch; parameters must agree with the full-batch run
    rel = (got["params"] - ref_params).norm() / ref_params.norm()
    assert rel < 2e-2, float(rel)
    assert abs(res["losses"][-1] - ref_losses[-1]) < 0.3


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_dp2_fused_snapshot_resumes(tmp_path):
    """The sharded optimizer's moments and fp32 master slices are gathered into the snapshot's ``.opt`` sidecar; a
    fresh data-parallel job that loads it repeats the next two AdamW steps (same step count, same parameters up to
    the nondeterministic order of the fp32 gradient atomics)."""
    res = launch(2, "dpresume", "fused", str(tmp_path / "dpresume"))
    assert res["sidecar"] and res["steps"][0] == res["steps"][1] == 3, res
    assert res["diff"] <= 2e-2 * res["scale"], res


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_dp2_weight_decay_spares_running_statistics(tmp_path):
    """AdamW with a large decay on a batch-norm model: the fused reduce + update kernel and the NCCL path must
    agree, and the running statistics (stored as parameters, never trained) must come out undecayed."""
    outs = {}
    for kind in ("fused", "nccl"):
        out = str(tmp_path / f"{kind}.pt")
        launch(2, "dpbn", kind, out)
        outs[kind] = torch.load(out)
    frozen = ~outs["nccl"]["trainable"]
    a, b = outs["fused"]["params"][frozen], outs["nccl"]["params"][frozen]  # running statistics and slab padding
    assert int((b != 0).sum()) >= 2 * 64
    assert torch.allclose(a, b, rtol=2e-2, atol=2e-2), float((a - b).abs().max())
    # a decayed running variance would have lost 1 - 0.95^4 = 19 % of its value
    rel = (outs["fused"]["params"] - outs["nccl"]["params"]).norm() / outs["nccl"]["params"].norm()
    assert rel < 3e-2, float(rel)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("kind", ["fused", "nccl"])
def test_tp2_trains(kind, tmp_path):
    res = launch(2, "tp", kind, str(tmp_path / "tp.pt"))
    assert res["losses"][-1] < res["losses"][0]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_matches_single_process(tmp_path):
    """Tensor parallelism must not change the training run: same initial weights and batches as one process; what
    four SGD steps changed in the fp32 master weights is compared (the two ranks see the same sequences, each half
    of the rows). The exact answer is the same run in fp32 on the CPU; how far bf16 arithmetic alone moves a run
    away from it is measured with the single-GPU run, and the fused kernels and the NCCL path must each stay within
    a small multiple of that distance - from the exact run and from each other."""
    g = torch.Generator().manual_seed(100)
    sets = [torch.randint(0, 203, (4, 129), generator=g) for _ in range(4)]
    sgd = {"type": "sgd", "learning_rate": 0.05, "momentum": 0.9}
    _, exact = single_process_reference(sets, tmp_path, sgd, device="CPU")
    ref_losses, ref_params = single_process_reference(sets, tmp_path, sgd)
    start = zoo.create("tiny_gpt").compile(device="cpu", seed=5).master_flat.float()
    d_ref = exact - start
    assert float(d_ref.norm()) > 0   # the run did move the parameters
    floor = float((ref_params - exact).norm() / d_ref.norm())   # bf16 on one GPU against fp32
    deltas, rels, losses = {}, {}, {}
    for kind in ("fused", "nccl"):
        out = str(tmp_path / f"tpeq_{kind}.pt")
        res = launch(2, "tpeq", kind, out)
        deltas[kind] = torch.load(out)["params"] - start
        rels[kind] = float((deltas[kind] - d_ref).norm() / d_ref.norm())
        losses[kind] = res["losses"]
    rels["between"] = float((deltas["fused"] - deltas["nccl"]).norm() / d_ref.norm())
    # per-parameter breakdown for the failure message: where the fused run departs from the single-process one
    full = zoo.create("tiny_gpt").compile(device="cpu", seed=5)
    worst = []
    for l in full.layers():
        for (o, n, _, _), spec in zip(full.layer_slices[id(l)], l.param_specs()):
            d = float(d_ref[o:o + n].norm())
            if d > 0:  # share of the total squared error, relative errors of both paths, share of the update norm
                ef = float((deltas["fused"][o:o + n] - d_ref[o:o + n]).norm())
                en = float((deltas["nccl"][o:o + n] - d_ref[o:o + n]).norm())
                worst.append((round(ef ** 2 / float((deltas["fused"] - d_ref).norm()) ** 2, 3), round(ef / d, 3), round(en / d, 3),
                              round(d ** 2 / float(d_ref.norm()) ** 2, 3), l.name + "." + spec.name))
    worst.sort(reverse=True)
    info = (rels, floor, losses, ref_losses, worst[:12])
    print("tp2 equivalence:", json.dumps(info))
    bound = 2.0 * floor + 0.03
    assert rels["fused"] < bound and rels["nccl"] < bound and rels["between"] < bound, info
    assert rels["fused"] < 1.5 * rels["nccl"] + 0.01, info
    assert abs(losses["fused"][-1] - ref_losses[-1]) < 0.3 and abs(losses["fused"][-1] - losses["nccl"][-1]) < 0.05, info


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("push_mode", ["ln", "split", "gemm"])
def test_tp2_kernels_match_fp32_and_nccl(push_mode):
    """The fused hand-offs across two real GPUs against fp32 on gathered operands and against the NCCL path,
    ragged widths included, three calls per site in a row; rows pushed by the layer-norm kernel, by the consuming GEMM's copy thread, or half and half."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29617", os.path.join(HERE, "_tp_kernel_worker.py"), push_mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, "\n".join(l for l in r.stdout.splitlines() if "WORKER-ERROR" in l)[:3000] + r.stdout[-2000:] + r.stderr[-500:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["all_ranks_ok"], res
    assert res["ag_worst"] < 3e-2 and res["rs_worst"] < 3e-2, res


def launch_pp(n, layout, kind, out):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29613", os.path.join(HERE, "_pp_gpu_worker.py"), layout, kind, out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, "\n".join(l for l in r.stdout.splitlines() if "WORKER-ERROR" in l or "Error" in l)[:3000] + r.stdout[-2500:] + r.stderr[-500:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pp2_1f1b_trains_and_saves_stage(tmp_path):
    from tnn_b200.nn.graph import Graph
    res = launch_pp(2, "pp2", "nccl", str(tmp_path / "ckpt"))
    assert res["losses"][-1] < res["losses"][0] - 0.5
    g = Graph.load_state(res["stage_file"])  # stage 0 file written by rank 0: a TNNG graph of its own
    assert g.input_nodes[0].uid() == "input" and len(g.edges) > 10


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_pp2_tp2_fused_trains(tmp_path):
    res = launch_pp(4, "pp2tp2", "fused", str(tmp_path / "ckpt"))
    assert res["losses"][-1] < res["losses"][0] - 0.5


# ------------------------------------------------------------------------------------- 8 GPUs
@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_dp8_matches_single_process(tmp_path):
    """Eight data-parallel ranks with the fused reduce + AdamW + broadcast kernel (bucketed, overlapped with the
    backward pass) against one process on the combined batch of sixteen sequences."""
    out = str(tmp_path / "dp8.pt")
    res = launch(8, "dp", "fused", out)
    assert res["max_rank_diff"] == 0.0 and res["dp_overlap"], res
    gens = [torch.Generator().manual_seed(100 + r) for r in range(8)]
    sets = [torch.cat([torch.randint(0, 203, (2, 129), generator=g) for g in gens]) for _ in range(4)]
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(128, 2, 2, "t", seq_len=128, vocab=203, drop=0.0))
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 16, "device_type": "CUDA", "seed": 5,
                                    "optimizer": {"type": "adamw", "learning_rate": 1e-2, "weight_decay": 0.01}})
    t = Trainer(cfg, log=False)
    for seq in sets:
        t.train_step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous())
    ref = t.graph.params_flat.float().cpu()
    t.close()
    got = torch.load(out)["params"]
    rel = (got - ref).norm() / ref.norm()
    assert rel < 2e-2, float(rel)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_tp2dp4_fused_tracks_nccl(tmp_path):
    """The benchmark's named layout on a tiny model: four data-parallel replicas of a tensor-parallel pair. The
    fused kernels and the NCCL path start from the same shards and see the same batches; their losses must agree
    step by step and fall."""
    runs = {kind: launch(8, "tp", kind, str(tmp_path / f"tp2dp4_{kind}.pt")) for kind in ("fused", "nccl")}
    lf, ln = runs["fused"]["losses"], runs["nccl"]["losses"]
    assert lf[-1] < lf[0] and ln[-1] < ln[0], (lf, ln)
    assert all(abs(a - b) < 0.05 for a, b in zip(lf, ln)), (lf, ln)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_pp4_tp2_fused_trains(tmp_path):
    """Four pipeline stages of one transformer block each, every stage a tensor-parallel pair with the fused
    hand-offs, 1F1B with two micro-batches: the layout of the GPT-2 medium benchmark configuration."""
    res = launch_pp(8, "pp4tp2", "fused", str(tmp_path / "ckpt"))
    assert res["losses"][-1] < res["losses"][0] - 0.5, res
