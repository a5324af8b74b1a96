"""gloo worker: pipeline-parallel (optionally x tensor-parallel) training vs one process."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.models import zoo  # noqa: E402
from tnn_b200.utils.config import TrainingConfig  # noqa: E402


def main():
    layout, out = sys.argv[1], sys.argv[2]
    accum = int(sys.argv[3]) if len(sys.argv) > 3 else 1
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(128, 2, 4, "t", seq_len=128, vocab=97, drop=0.0))
    from tnn_b200.parallel.pp import PipelineTrainer
    from tnn_b200.parallel.tp import copy_full_to_shards
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 4, "device_type": "CPU", "seed": 5,
                                    "optimizer": {"type": "sgd", "learning_rate": 0.1, "momentum": 0.9},
                                    "gradient_accumulation_steps": accum,
                                    "parallel": {"microbatches": 2 if "tp" in layout else 4}})
    t = PipelineTrainer(cfg, layout, fused=False)
    # same weights as the single-process model: copy every layer of this stage from a full graph
    full = zoo.create("tiny_gpt").compile(seed=5)
    if t.topo.tp > 1:
        copy_full_to_shards(t.stage, full, t.topo)
    else:
        byname = {l.name: l for l in full.layers()}
        for l in t.stage.layers():
            for p, q in zip(l.params, byname[l.name].params):
                p.copy_(q)
    gen = torch.Generator().manual_seed(100)
    losses = []
    for _ in range(3 if accum == 1 else 2 * accum):
        seq = torch.randint(0, 97, (4, 129), generator=gen)
        loss = t.train_step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous())
        losses.append(float(loss) if loss is not None else None)
    res = [None] * dist.get_world_size()
    dist.all_gather_object(res, (losses, {l.name: [p.clone() for p in l.params] for l in t.stage.layers()},
                                 t.stage.input_uids, t.stage.output_uids))
    if rank == 0:
        torch.save(res, out)
    t.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
