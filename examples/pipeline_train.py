"""Pipeline / tensor / data parallel training, one process per GPU:

    torchrun --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 examples/pipeline_train.py \
        --config configs/gpt2_medium_tp2_pp2.json --layout pp2tp2

Replaces the reference's coordinator + worker processes (examples/tcp_coordinator.cpp:27-128,
examples/tcp_worker.cpp:39-141): the batch is split into micro-batches on every stage-0 rank, stages
exchange activations and gradients with NCCL point-to-point calls under the 1F1B schedule, and each
stage applies its own optimizer step. On a machine without GPUs the same command runs on the gloo
backend when the config says ``"device_type": "CPU"``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(["train"] + sys.argv[1:]))
