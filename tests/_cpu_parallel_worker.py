"""gloo worker for the CPU multi-process tests: data / tensor parallel steps vs one process."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.models import zoo  # noqa: E402
from tnn_b200.utils.config import TrainingConfig  # noqa: E402


def main():
    mode, out = sys.argv[1], sys.argv[2]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(128, 2, 2, "t", seq_len=128, vocab=97, drop=0.0))
    from tnn_b200.parallel.runtime import ParallelTrainer
    from tnn_b200.parallel.tp import copy_full_to_shards
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 1 if mode == "tp" else 2, "device_type": "CPU",
                                    "seed": 5, "optimizer": {"type": "sgd", "learning_rate": 0.1, "momentum": 0.9}})
    if mode.startswith("resume"):
        return resume(mode, out, rank, world)
    t = ParallelTrainer(cfg, layout="tp2" if mode == "tp" else f"dp{world}", fused=False, log=False)
    if mode == "tp":
        full = zoo.create("tiny_gpt").compile(seed=5)
        copy_full_to_shards(t.graph, full, t.topo)
    gen = torch.Generator().manual_seed(100 + t.data_rank)
    losses = []
    for _ in range(3):
        seq = torch.randint(0, 97, (t.local_batch, 129), generator=gen)
        losses.append(float(t.train_step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous()).item()))
    if mode == "tp":
        t.save_snapshot(out + ".tnng")  # gathers the shards: one file that an unsharded job can load
    allm = [None] * world
    dist.all_gather_object(allm, (losses, t.graph.master_flat.clone()))
    if rank == 0:
        torch.save({"losses": [a[0] for a in allm], "masters": [a[1] for a in allm],
                    "layout": {l.name: t.graph.layer_slices[id(l)] for l in t.graph.layers()}}, out)
    t.close()
    dist.destroy_process_group()


def resume(mode, out, rank, world):
    """Train, snapshot with optimizer state, train on; then a second trainer loads the snapshot and repeats the last
    steps: weights, momentum, step count and learning rate must come back exactly. ``resume_tp``: tensor parallel."""
    from tnn_b200.parallel.runtime import ParallelTrainer
    tp = mode == "resume_tp"
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 1 if tp else 2, "device_type": "CPU", "seed": 5,
                                    "optimizer": {"type": "adamw", "learning_rate": 1e-2, "weight_decay": 0.01},
                                    "scheduler": {"type": "step_lr", "step_size": 2, "gamma": 0.5}})
    layout = "tp2" if tp else f"dp{world}"

    def batches(first, n, t):
        gen = torch.Generator().manual_seed(100 + t.data_rank)
        seqs = [torch.randint(0, 97, (t.local_batch, 129), generator=gen) for _ in range(first + n)]
        return seqs[first:]

    a = ParallelTrainer(cfg, layout=layout, fused=False, log=False)
    for s in batches(0, 3, a):
        a.train_step(s[:, :-1].contiguous(), s[:, 1:].contiguous())
    snap = out + ".snap.tnng"
    a.save_snapshot(snap, with_optimizer=True)
    for s in batches(3, 2, a):
        a.train_step(s[:, :-1].contiguous(), s[:, 1:].contiguous())
    b = ParallelTrainer(cfg, layout=layout, fused=False, log=False)
    b.load_snapshot(snap)
    state = {"step": (a.optimizer.step_count - 2, b.optimizer.step_count), "global": (a.global_step - 2, b.global_step)}
    for s in batches(3, 2, b):
        b.train_step(s[:, :-1].contiguous(), s[:, 1:].contiguous())
    state["lr"] = (a.optimizer.get_learning_rate(), b.optimizer.get_learning_rate())
    state["diff"] = float((a.graph.master_flat - b.graph.master_flat).abs().max())
    state["moved"] = float((a.graph.master_flat - zoo.create("tiny_gpt").compile(seed=5).master_flat).abs().max()) if not tp else 1.0
    state["sidecars"] = sorted(f for f in os.listdir(os.path.dirname(out)) if ".opt" in f)
    alls = [None] * world
    dist.all_gather_object(alls, state)
    if rank == 0:
        torch.save(alls, out)
    a.close()
    b.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
