"""Reference arm, first choice: the reference's own C++/CUDA/cuDNN engine through its stock ``trainer --config``.

``build_reference_engine.py`` compiles the unmodified reference sources into ``baseline/_ref/tunx_build/bin/trainer``
(its examples/trainer.cpp). This module drives that binary the way a user of the reference would:

* a working directory with ``data/open-web-text/{train.bin,val.bin,vocab.bin}`` - uniform random token ids as
  uint16, the format its OpenWebText loader maps (include/data_loading/open_webtext_data_loader.hpp:70-100; the
  vocabulary path is hard-wired relative to the working directory);
* the reference's own ``configs/gpt2_config.json`` (copied beside the binary at build time) with only
  ``max_steps``, ``batch_size``, ``dataset_path`` and the print interval changed;
* two runs, of W and of W + K steps. The program prints ``Training completed in <ms>ms`` for its whole step loop
  (src/nn/train.cpp:424,548-551: from before the first batch to after the last optimizer update, before the
  snapshot is written); the difference of the two is the time of exactly K steady-state steps, with the cuDNN
  plan building of the first step cancelled out. Its own per-step ``time_ms`` column stops before the optimizer
  update (src/nn/train.cpp:505-514) and is not used.

Every step of that loop uploads the batch from host memory and reads the loss back (``compute_loss`` returns a
host float), so the number is an end-to-end number by construction.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import struct
import subprocess
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
VOCAB = 50257


def build_dir(fixed: bool) -> str:
    """``tunx_build`` holds the build of the unmodified sources, ``tunx_build_fixed`` the one made with
    ``build_reference_engine.py --fix-block-engine`` (one header gains two forwarding methods; see that script)."""
    return os.path.join(HERE, "_ref", "tunx_build_fixed" if fixed else "tunx_build")


def available(fixed: bool = False) -> bool:
    b = build_dir(fixed)
    return os.path.exists(os.path.join(b, "bin", "trainer")) and os.path.exists(os.path.join(b, "configs", "gpt2_config.json"))


def _write_dataset(root: str, n_tokens: int) -> None:
    import numpy as np

    d = os.path.join(root, "data", "open-web-text")
    os.makedirs(d, exist_ok=True)
    rng = np.random.default_rng(1234)
    for name in ("train.bin", "val.bin"):
        rng.integers(0, VOCAB, size=n_tokens if name == "train.bin" else 4096, dtype=np.uint16).tofile(os.path.join(d, name))
    with open(os.path.join(d, "vocab.bin"), "wb") as f:  # u32 count, then per token u32 length + bytes
        f.write(struct.pack("<I", VOCAB))
        for i in range(VOCAB):
            tok = b"t%d " % i
            f.write(struct.pack("<I", len(tok)) + tok)


def _run(trainer: str, root: str, cfg: dict, steps: int, timeout: float):
    cfg = dict(cfg, max_steps=steps)
    path = os.path.join(root, f"cfg_{steps}.json")
    with open(path, "w") as f:
        json.dump(cfg, f)
    r = subprocess.run([trainer, "--config", path], cwd=root, capture_output=True, text=True, timeout=timeout)
    out = r.stdout + r.stderr
    m = re.search(r"Training completed in (\d+)ms", out)
    losses = re.findall(r"Batch ID: (\d+), Batch's Loss: ([0-9.naninf-]+)", out)
    shutil.rmtree(os.path.join(root, "model_snapshots"), ignore_errors=True)
    if r.returncode != 0 or not m:
        tail = " | ".join(l for l in out.strip().splitlines()[-6:])
        raise RuntimeError(f"trainer exited {r.returncode} after {steps} steps: {tail[-600:]}")
    return float(m.group(1)), (float(losses[-1][1]) if losses else None)


def run_engine(model: str, batch: int, warm: int, steps: int, dtype: str = "", timeout: float = 900.0, fixed: bool = False) -> dict:
    """Time K steps of the reference engine; returns the fields of the bench line it determines. Raises on failure."""
    if model != "gpt2_small":
        raise RuntimeError("the engine arm covers gpt2_small (flash_gpt2_small); the reference's 224x224 image loaders "
                           "decode files through stb_image, which is not available offline")
    build = build_dir(fixed)
    trainer = os.path.join(build, "bin", "trainer")
    with open(os.path.join(build, "configs", "gpt2_config.json")) as f:
        cfg = json.load(f)
    root = tempfile.mkdtemp(prefix="tnnb_refeng_")
    try:
        _write_dataset(root, 4 * 1024 * 1024)
        cfg.update(batch_size=batch, dataset_path="data/open-web-text", progress_print_interval=max(1, warm), device_type="CUDA",
                   model_path="")
        if dtype:
            cfg.update(io_dtype=dtype, param_dtype=dtype, compute_dtype=dtype)
        if os.environ.get("TNNB_REF_MODEL"):  # e.g. gpt2_small: the reference's GPT-2 small without the cuDNN attention block
            cfg.update(model_name=os.environ["TNNB_REF_MODEL"])
        t_short, _ = _run(trainer, root, cfg, warm, timeout)
        t_long, loss = _run(trainer, root, cfg, warm + steps, timeout)
    finally:
        shutil.rmtree(root, ignore_errors=True)
    ms = max(t_long - t_short, 1e-3)
    value = batch * 1024 * steps / (ms / 1e3)
    used = {k: cfg.get(k) for k in ("io_dtype", "param_dtype", "compute_dtype")}
    return {
        "value": round(value, 1), "ms_per_step": round(ms / steps, 3), "loss_last": loss,
        "dtype": "/".join(str(v) for v in used.values()) + " (io/param/compute of the reference's gpt2_config.json"
                 + (", overridden by TNNB_REF_DTYPE)" if dtype else ")"),
        "path": f"reference C++/cuDNN engine: examples/trainer.cpp --config configs/gpt2_config.json (model {cfg['model_name']}), "
                f"built by baseline/build_reference_engine.py{' --fix-block-engine (Block forwards engine and backend handle to its sub-layers; the unmodified build dereferences a null engine on the first step)' if fixed else ''}; wall clock of the step loop, ({warm + steps}-step run) - ({warm}-step run)",
        "h2d_bytes_per_step": batch * 1024 * (4 + 4), "d2h_bytes_per_step": 8,
        "run_ms": {"short": t_short, "long": t_long},
    }
