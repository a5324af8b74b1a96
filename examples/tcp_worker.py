"""``python examples/tcp_worker.py 8001 [--gpu]`` - one pipeline stage served over TCP until the coordinator sends
SHUTDOWN (same as ``python -m tnn_b200 tcp-worker``). Reference: examples/tcp_worker.cpp:39-141."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(["tcp-worker"] + sys.argv[1:]))
