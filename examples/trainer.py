"""``python examples/trainer.py --config configs/gpt2_small.json`` - train from a JSON configuration.
Reference: examples/trainer.cpp:15-85. Under ``torchrun`` every process becomes one rank of a parallel job."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(["train"] + sys.argv[1:]))
