"""Loader of the compiled host runtime (``_lib/_host*.so``, built by :mod:`tnn_b200._build`).

``from tnn_b200.host import H`` gives the pybind11 module with the typed config, TNNG and
wire-format codecs, the graph IR / partitioner, the profiler, the CPU engine (``H.cpu``),
the allocators, dataset loaders and the tokenizer.
"""
from __future__ import annotations

import importlib.util
import os

from . import _build


def _load():
    # TNNB_HOST_SANITIZE=1 selects the AddressSanitizer / UBSan build (start the process with _build.sanitizer_env())
    sanitize = os.environ.get("TNNB_HOST_SANITIZE", "") == "1"
    path = _build.host_path(sanitize)
    if not os.path.exists(path):
        _build.build_host(sanitize=sanitize)
    spec = importlib.util.spec_from_file_location("_host", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


H = _load()
