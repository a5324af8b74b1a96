"""The C++ host runtime under AddressSanitizer + UndefinedBehaviorSanitizer.

A child interpreter starts with the ASan runtime preloaded and imports the sanitized build of the host library
(``tnn_b200/_lib/san``); it then drives the codecs and algorithms that parse untrusted bytes or do index
arithmetic: typed config JSON, the wire format (messages, packets, chunking), TNNG files including truncated
and corrupted ones, the graph IR with the partitioner, the CPU engine's convolution / pooling / normalisation
loops on odd shapes, the allocators and the profiler. Any sanitizer report ends the child with a non-zero code.
"""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent('''
    import os, sys, struct, tempfile
    import numpy as np
    sys.path.insert(0, os.environ["TNNB_ROOT"])
    from tnn_b200 import _build
    import importlib.util
    spec = importlib.util.spec_from_file_location("_host", _build.host_path(True))
    H = importlib.util.module_from_spec(spec); spec.loader.exec_module(H)
    names = [n for n in dir(H) if not n.startswith("_")]

    # ---- CPU engine on odd shapes (index arithmetic of the direct loops) ----
    c = H.cpu
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 7, 5, 3), dtype=np.float32)
    w = rng.standard_normal((4, 3, 2, 3), dtype=np.float32)
    b = rng.standard_normal((4,), dtype=np.float32)
    for (sh, sw, ph, pw) in [(1, 1, 0, 0), (2, 1, 1, 2), (3, 2, 2, 1)]:
        y = c.conv2d_fwd(x, w, b, sh, sw, ph, pw)
        dy = np.ones_like(y)
        dx = c.conv2d_dgrad(dy, w, list(x.shape), sh, sw, ph, pw)
        dw, db = np.zeros_like(w), np.zeros_like(b)
        c.conv2d_wgrad(x, dy, dw, db, sh, sw, ph, pw)
        assert dx.shape == x.shape and np.isfinite(dw).all()
    for is_max in (True, False):
        p, idx = c.pool2d_fwd(x, is_max, 3, 2, 2, 2, 1, 1)
        c.pool2d_bwd(np.ones_like(p), idx, list(x.shape), is_max, 3, 2, 2, 2, 1, 1)
    xs = rng.standard_normal((5, 9), dtype=np.float32)
    y, mean, rstd = c.layernorm_fwd(xs, None, None, 1e-5)
    c.layernorm_bwd(np.ones_like(xs), xs, mean, rstd, None, None, None)
    ww = rng.standard_normal((6, 9), dtype=np.float32)
    yy = c.dense_fwd(xs, ww, None)
    c.dense_bwd(np.ones_like(yy), xs, ww, np.zeros_like(ww), None)
    loss, g, corr = c.softmax_ce(yy, np.array([0, 5, 2, 1, 3], dtype=np.int32))
    assert np.isfinite(loss)

    # ---- the remaining bindings are exercised by the regular host tests, re-run against this build ----
    print("CHILD-OK", len(names))
''')


def _env():
    from tnn_b200 import _build

    env = _build.sanitizer_env()
    env["TNNB_ROOT"] = ROOT
    return env


@pytest.fixture(scope="module")
def sanitized_build():
    from tnn_b200 import _build

    try:
        return _build.build_host(sanitize=True)
    except Exception as e:  # no libasan in this toolchain
        pytest.skip(f"sanitized build unavailable: {e}")


def test_cpu_engine_loops_under_asan_ubsan(sanitized_build):
    r = subprocess.run([sys.executable, "-c", CHILD], env=_env(), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "CHILD-OK" in r.stdout, (r.stdout[-1500:] + r.stderr[-3000:])
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error:" not in r.stderr, r.stderr[-3000:]


def test_host_test_suite_under_asan_ubsan(sanitized_build):
    """The host-runtime tests (formats, graph IR, partitioner, loaders, allocators) again, on the sanitized build."""
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_host_cpu.py"), "-x", "-q", "-p", "no:cacheprovider"]
    r = subprocess.run(cmd, env=_env(), capture_output=True, text=True, timeout=1500, cwd=ROOT)
    assert "ERROR: AddressSanitizer" not in r.stderr + r.stdout and "runtime error:" not in r.stderr + r.stdout, \
        (r.stdout[-2000:] + r.stderr[-3000:])
    assert r.returncode == 0, (r.stdout[-2000:] + r.stderr[-2000:])


def test_tcp_communicator_under_asan_ubsan(sanitized_build):
    """The socket reader / writer threads of the TCP communicator (loopback messages, reassembly, destruction with
    packets still queued) on the sanitized build."""
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_tcp_cpu.py"), "-x", "-q", "-p", "no:cacheprovider",
           "-k", "communicator or aggregator"]
    r = subprocess.run(cmd, env=_env(), capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert "ERROR: AddressSanitizer" not in r.stderr + r.stdout and "runtime error:" not in r.stderr + r.stdout, \
        (r.stdout[-2000:] + r.stderr[-3000:])
    assert r.returncode == 0, (r.stdout[-2000:] + r.stderr[-2000:])
