"""Greedy decoding: 50 new tokens from a 30-token prompt cut out of a token file, stopping at token 50256.

    python examples/gpt2_inference.py --model-path model_snapshots/gpt2_small.tnng \
        --vocab data/open-web-text/vocab.bin --tokens data/open-web-text/train.bin

Without ``--vocab`` the token ids are printed instead of text; without ``--model-path`` a randomly
initialised ``--model`` is used. Reference: examples/gpt2_inference.cpp:16-114."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(["generate"] + sys.argv[1:]))
