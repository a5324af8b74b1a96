"""Worker launched by the multi-GPU tests through ``torch.distributed.run`` (one rank per GPU)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.models import zoo  # noqa: E402
from tnn_b200.ops import _lib  # noqa: E402
from tnn_b200.utils.config import TrainingConfig  # noqa: E402


def main():
    mode = sys.argv[1]
    fused = sys.argv[2] == "fused"
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    os.environ.setdefault("TNNB_DP_MIN_BUCKET", "4096")  # several buckets even for the tiny models: overlapped reduction
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(128, 2, 2, "t", seq_len=128, vocab=203, drop=0.0))
    from tnn_b200.parallel.runtime import ParallelTrainer
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 2, "device_type": "CUDA", "seed": 5,
                                    "optimizer": {"type": "adamw", "learning_rate": 1e-2, "weight_decay": 0.01}})
    if mode == "dpbn":  # batch-norm model under a strongly decaying AdamW: running statistics must not be decayed
        def tiny_bn_cnn():
            b = zoo._start((1, 16, 16, 3))
            b.conv(32, 3, 1, 1, True, "c1").bn(True, "bn1").maxpool(2, 2, 0, "p1")
            b.conv(64, 3, 1, 1, False, "c2").bn(True, "bn2").avgpool(8, 1, 0, "gap")
            return zoo._finish(b.flatten().dense(10, True, "fc"))
        zoo.register_model("tiny_bn_cnn", tiny_bn_cnn)
        cfg = TrainingConfig.from_dict({"model_name": "tiny_bn_cnn", "batch_size": 8, "device_type": "CUDA", "seed": 5,
                                        "optimizer": {"type": "adamw", "learning_rate": 1e-2, "weight_decay": 5.0}})
        t = ParallelTrainer(cfg, layout=f"dp{world}", fused=fused, log=False, heap_bytes=256 << 20)
        gen = torch.Generator().manual_seed(100 + t.data_rank)
        losses = []
        for step in range(4):
            x = torch.randn(t.local_batch, 16, 16, 3, generator=gen) * 2.0 + 0.5
            y = torch.randint(0, 10, (t.local_batch,), generator=gen)
            losses.append(float(t.train_step(x, y).item()))
        _lib.check_status()
        t._refresh_master()  # with the sharded optimizer a rank holds fp32 master values for its own slices only
        if rank == 0:
            torch.save({"params": t.graph.master_flat.float().cpu(), "trainable": t.graph.trainable_mask.cpu(), "losses": losses},
                       sys.argv[3])
            print("RESULT " + json.dumps({"losses": losses}), flush=True)
        t.close()
        dist.destroy_process_group()
        return
    if mode == "dpresume":
        # fused (sharded) optimizer: snapshot with optimizer state after 3 steps, 2 more steps; a second trainer loads
        # the snapshot and must reproduce those 2 steps
        def seqs(t, first, n):
            g = torch.Generator().manual_seed(100 + t.data_rank)
            return [torch.randint(0, 203, (t.local_batch, 129), generator=g) for _ in range(first + n)][first:]
        a = ParallelTrainer(cfg, layout=f"dp{world}", fused=fused, log=False, heap_bytes=256 << 20)
        for sq in seqs(a, 0, 3):
            a.train_step(sq[:, :-1].contiguous(), sq[:, 1:].contiguous())
        snap = sys.argv[3] + ".snap.tnng"
        a.save_snapshot(snap, with_optimizer=True)
        for sq in seqs(a, 3, 2):
            a.train_step(sq[:, :-1].contiguous(), sq[:, 1:].contiguous())
        b = ParallelTrainer(cfg, layout=f"dp{world}", fused=fused, log=False, heap_bytes=256 << 20)
        b.load_snapshot(snap)
        steps = (a.optimizer.step_count - 2, b.optimizer.step_count)
        for sq in seqs(b, 3, 2):
            b.train_step(sq[:, :-1].contiguous(), sq[:, 1:].contiguous())
        _lib.check_status()
        pa, pb = a.graph.params_flat.float(), b.graph.params_flat.float()
        out = {"steps": steps, "diff": float((pa - pb).abs().max()), "scale": float(pa.abs().max()),
               "sidecar": os.path.exists(snap + ".opt")}
        if rank == 0:
            print("RESULT " + json.dumps(out), flush=True)
        a.close()
        b.close()
        dist.destroy_process_group()
        return
    if mode == "tpeq":
        # plain SGD: the update is proportional to the gradient, so rounding noise stays proportional too (the first
        # Adam steps move every element by the full learning rate in the direction of a sign that noise can flip)
        cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 2, "device_type": "CUDA", "seed": 5,
                                        "optimizer": {"type": "sgd", "learning_rate": 0.05, "momentum": 0.9}})
    layout = {"dp": f"dp{world}", "tp": f"tp2dp{world // 2}" if world > 2 else "tp2",
              "tpeq": f"tp2dp{world // 2}" if world > 2 else "tp2"}[mode]
    t = ParallelTrainer(cfg, layout=layout, fused=fused, log=False, heap_bytes=256 << 20)
    if mode == "tpeq":  # start from the weights the single-process run starts from
        from tnn_b200.parallel.tp import copy_full_to_shards
        full = zoo.create(cfg.model_name).compile(device="cpu", seed=cfg.seed)
        copy_full_to_shards(t.graph, full, t.topo)
    gen = torch.Generator().manual_seed(100 + t.data_rank)
    losses = []
    for step in range(4):
        seq = torch.randint(0, 203, (t.local_batch, 129), generator=gen)
        loss = t.train_step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous())
        losses.append(float(loss.item()))
    _lib.check_status()
    if mode == "tpeq":  # gather the shards into an unsharded model and hand its parameters back
        from tnn_b200.parallel.tp import gather_full_state
        g = t.graph
        if hasattr(t.optimizer, "sites"):
            # sharded optimizer: a rank holds fp32 master values only for the slices it updates. Collect the exact
            # fp32 values of the replicated region from their owners (the sharded region is updated by this rank
            # alone when dp = 1); the compute copy would only give them rounded to bf16.
            mine = torch.zeros_like(g.trainable_mask)
            for s in t.optimizer.sites:
                mine[s["lo"]:s["hi"]] = True
            b = g.shard_boundary
            rep = torch.where(mine[:b], g.master_flat[:b], torch.zeros_like(g.master_flat[:b]))
            dist.all_reduce(rep)
            g.master_flat[:b].copy_(rep)
            assert bool(mine[b:].all()) or world > 2
        full = zoo.create(cfg.model_name).compile(device="cpu", seed=cfg.seed)
        gather_full_state(t.graph, full, t.topo)
        if rank == 0:
            torch.save({"params": full.master_flat.float().cpu(), "losses": losses}, sys.argv[3])
            print("RESULT " + json.dumps({"losses": losses}), flush=True)
        t.close()
        dist.destroy_process_group()
        return
    master = t.graph.params_flat.float().clone()
    gathered = [torch.zeros_like(master) for _ in range(world)]
    dist.all_gather(gathered, master)
    if rank == 0:
        out = {"losses": losses, "param_sum": float(t.graph.params_flat.float().sum()), "n": t.graph.num_parameters(),
               "dp_sites": len(getattr(t.optimizer, "sites", [])), "dp_overlap": bool(getattr(t.optimizer, "overlap", False))}
        if mode == "dp":
            out["max_rank_diff"] = max(float((g - gathered[0]).abs().max()) for g in gathered)
        torch.save({"params": t.graph.params_flat.float().cpu(), "losses": losses}, sys.argv[3])
        print("RESULT " + json.dumps(out), flush=True)
    t.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback

        print("WORKER-ERROR rank", os.environ.get("RANK"), traceback.format_exc()[-1500:].replace("\n", " | "), flush=True)
        os._exit(1)
