"""``python examples/tcp_coordinator.py --config configs/tcp_cnn_mnist.json`` - partition a model, deploy the stages to
TCP workers (start those first) and train (same as ``python -m tnn_b200 tcp-coordinator``).
Reference: examples/tcp_coordinator.cpp:27-128."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(["tcp-coordinator"] + sys.argv[1:]))
