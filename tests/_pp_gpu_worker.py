"""NCCL worker for the multi-GPU pipeline tests (pp2 on 2 GPUs, pp2tp2 on 4)."""
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
    layout, fused, out = sys.argv[1], sys.argv[2] == "fused", sys.argv[3]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(128, 2, 4, "t", seq_len=128, vocab=203, drop=0.0))
    from tnn_b200.parallel.pp import PipelineTrainer
    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 4, "device_type": "CUDA", "seed": 5,
                                    "optimizer": {"type": "adamw", "learning_rate": 5e-3},
                                    "parallel": {"microbatches": 4 if "tp" not in layout else 2}})
    t = PipelineTrainer(cfg, layout, fused=fused, heap_bytes=256 << 20)
    gen = torch.Generator().manual_seed(100 + t.data_rank)
    seq = torch.randint(0, 203, (t.local_batch, 129), generator=gen)
    losses = []
    for _ in range(8):
        loss = t.train_step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous())
        losses.append(float(loss.item()) if loss is not None else None)
    _lib.check_status()
    name = t.save_stage(out)
    allr = [None] * dist.get_world_size()
    dist.all_gather_object(allr, losses)
    if dist.get_rank() == 0:
        print("RESULT " + json.dumps({"losses": [l for l in allr if l[0] is not None][0], "stage_file": name}), flush=True)
    t.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback

        print("WORKER-ERROR rank", os.environ.get("RANK"), traceback.format_exc()[-1500:].replace("\n", " | "), flush=True)
        os._exit(1)
