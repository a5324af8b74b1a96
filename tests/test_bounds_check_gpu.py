"""The bounds-checked build of the kernel library (``-DTNNB_BOUNDS_CHECK``, loaded with ``TNNB_BOUNDS_CHECK=1``).

A child process loads the checked library, runs a small training step and a set of kernels on valid inputs (no
record may appear), then feeds an out-of-range label and an out-of-range token id. Both builds skip such
entries without touching memory outside the tensors; the checked build must also report them, with the index
and the limit, and the CUDA context must stay usable afterwards.
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent('''
    import os, sys
    sys.path.insert(0, os.environ["TNNB_ROOT"])
    import torch
    from tnn_b200.ops import _lib, raw
    from tnn_b200.models import zoo
    assert _lib.bounds_checked() and _lib.lib_path().endswith(os.path.join("dbg", "libtnnb_kernels.so"))
    dev = torch.device("cuda", 0)
    # ---- valid work: a conv / batch-norm / pool model and a token model, forward + backward ----
    g = zoo.create("cifar10_resnet9").compile(device="cuda:0", seed=1)
    g.train()
    y = g(torch.randn(8, 32, 32, 3))
    g.backward({"output": torch.ones_like(y)})
    t = zoo.gpt2(128, 2, 1, "t", seq_len=128, vocab=203, drop=0.0).compile(device="cuda:0", seed=2)
    t.train()
    ids = torch.randint(0, 203, (2, 128), device=dev)
    out = t(ids)
    from tnn_b200.nn.loss import CrossEntropyLoss
    loss, grad = CrossEntropyLoss().compute(out, ids)
    t.backward({"output": grad})
    _lib.check_status()
    assert _lib.fetch_bounds_violations() == [], "valid inputs produced a bounds record"
    # ---- a label outside the vocabulary ----
    logits = torch.randn(4, 208, device=dev).bfloat16()[:, :203]
    labels = torch.tensor([1, 2, 999, 3], device=dev)
    raw.softmax_ce(logits, labels, 203, 0.25, 0.25)
    v = _lib.fetch_bounds_violations()
    assert len(v) == 1 and v[0]["file"] == "loss_optim.cu" and v[0]["index"] == 999 and v[0]["limit"] == 203, v
    assert _lib.fetch_bounds_violations() == []  # the record was cleared
    # ---- a token id outside the table ----
    wte = torch.randn(50, 64, device=dev).bfloat16()
    bad = torch.tensor([[3, 77, 4]], device=dev)
    e = raw.embedding_fwd(bad, wte, None, 1, 50, 0.0, 0)
    assert torch.equal(e.reshape(3, 64)[1], wte[0])  # read as row 0, like the regular build
    try:
        _lib.check_bounds()
        raise SystemExit("no IndexError")
    except IndexError as ex:
        assert "elementwise.cu" in str(ex) and "77" in str(ex)
    # ---- the context is still usable ----
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    print("CHILD-OK")
''')


def test_checked_build_reports_and_survives():
    from tnn_b200 import _build

    _build.build_kernels(bounds_check=True)
    env = dict(os.environ, TNNB_BOUNDS_CHECK="1", TNNB_ROOT=ROOT)
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "CHILD-OK" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]


def test_regular_build_refuses_to_report():
    from tnn_b200.ops import _lib

    if _lib.bounds_checked():
        pytest.skip("this process runs the checked build")
    with pytest.raises(RuntimeError, match="not the bounds-checked build"):
        _lib.fetch_bounds_violations()
