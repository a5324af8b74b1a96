"""``python examples/inferencer.py --config x.json`` - validation loss and accuracy of ``model_path`` (a TNNG
snapshot) or of a freshly initialised ``model_name``. Reference: examples/inferencer.cpp:12-70."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(["infer"] + sys.argv[1:]))
