"""gloo worker for the failure-detection test: trains a tiny model data-parallel on CPU; the rank named by
TNNB_FAULT leaves between steps, the others must notice on the host (heartbeats) before their next collective."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.models import zoo  # noqa: E402
from tnn_b200.parallel.health import GuardedRunner, RankFailure  # noqa: E402
from tnn_b200.utils.config import TrainingConfig  # noqa: E402


def main():
    out_dir = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["HEALTH_PORT"]), world, rank == 0, timeout=__import__("datetime").timedelta(seconds=30))
    dist.init_process_group("gloo", timeout=__import__("datetime").timedelta(seconds=20))
    zoo.register_model("tiny_gpt", lambda: zoo.gpt2(32, 1, 1, "t", seq_len=16, vocab=31, drop=0.0))
    from tnn_b200.parallel.runtime import ParallelTrainer

    cfg = TrainingConfig.from_dict({"model_name": "tiny_gpt", "batch_size": 2, "device_type": "CPU", "seed": 3,
                                    "optimizer": {"type": "sgd", "learning_rate": 0.05}, "snapshot_dir": out_dir})
    t = ParallelTrainer(cfg, layout=f"dp{world}", fused=False, log=False)
    runner = GuardedRunner(t, store, rank, world, timeout=1.5, interval=0.2)
    gen = torch.Generator().manual_seed(10 + rank)
    result = {"rank": rank, "steps": 0, "detected": None}
    try:
        for step in range(8):
            seq = torch.randint(0, 31, (2, 17), generator=gen)
            runner.step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous())
            result["steps"] = step + 1
            if step == 1:  # collective: every rank takes part, the first one writes
                result["snapshot"] = t.save_snapshot(os.path.join(out_dir, "ckpt_step2.tnng"), with_optimizer=True)
            time.sleep(0.6)  # a step every 0.6 s: the lost rank is noticed within a few steps
    except RankFailure as e:
        result["detected"] = e.dead
    runner.close()
    with open(os.path.join(out_dir, f"result_{rank}.json"), "w") as f:
        json.dump(result, f)
    # no collective after a failure: leave without the usual process-group teardown
    os._exit(0)


if __name__ == "__main__":
    main()
