"""``bench.py --impl reference``: time the reference's own code on the same metric and configuration.

What "the reference" can mean on this machine (recorded in DESIGN.md):

* Its C++/CUDA/cuDNN engine (``trainer --config``) cannot be built offline: CMake fetches asio,
  nlohmann_json, googletest, stb, spdlog and cudnn-frontend from the network at configure time and
  requires libibverbs and TBB, none of which exist here. ``pip install /root/reference`` installs
  only the metadata of its documentation helper package (no importable code).
* Its PyTorch trainer ``torch/torch_trainer.py`` is runnable. This arm imports that file
  UNMODIFIED from ``baseline/_ref/tunx_torch`` and uses its own model class
  (``GPT2Small`` / ``ResNet50ImageNet100``), its own model registry entry (batch size, optimizer type,
  learning rate), the optimizer construction of its ``main`` and its own ``train_epoch`` loop, fed
  by its own ``OpenWebTextDataset`` reading a synthetic ``train.bin`` of uniform random token ids
  (or by a synthetic image iterable for ResNet-50). None of this repository's models, kernels or
  engine are on that path. ``torch.compile(max-autotune)``, which the script's ``main`` also applies,
  is off by default because its autotuning alone takes longer than the whole benchmark;
  ``TNNB_REF_COMPILE=1`` turns it on.

The reference trainer is single-GPU, so for N > 1 this arm reports ``unavailable``.
"""
from __future__ import annotations

import csv
import io
import json
import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref", "tunx_torch")


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run_reference(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1 or args.gpus > 1:
        if rank == 0:
            _unavailable("the reference trainer (C++ engine and torch/torch_trainer.py alike) is single-GPU; it has no data- or "
                         "tensor-parallel mode to run at N > 1")
        return
    if not os.path.exists(os.path.join(REF_DIR, "torch_trainer.py")):
        _unavailable("baseline/_ref/tunx_torch/torch_trainer.py is missing (copy /root/reference/torch there); the C++ engine "
                     "cannot be built offline (network FetchContent, libibverbs, TBB)")
        return
    import numpy as np
    import torch

    if not torch.cuda.is_available():
        _unavailable("no CUDA device")
        return
    sys.path.insert(0, REF_DIR)
    try:
        import torch_trainer as ref  # the reference file, unmodified
    except Exception as e:  # missing optional dependency of the script
        _unavailable(f"cannot import the reference torch_trainer.py: {type(e).__name__}: {e}")
        return
    import torch.optim as optim

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    is_lm = args.model.startswith("gpt2")
    warm, steps = max(3, args.warmup), args.steps
    tmp = tempfile.mkdtemp(prefix="tnnb_ref_")
    if is_lm:
        batch = args.per_gpu_batch or 8
        n_windows = (warm + steps) * batch
        rng = np.random.default_rng(1234)
        path = os.path.join(tmp, "train.bin")
        rng.integers(0, 50257, size=n_windows * 1024 + 1, dtype=np.uint16).tofile(path)
        os.environ["OPENWEBTEXT_PATH"] = path
        os.environ["OPENWEBTEXT_VAL_PATH"] = path
        os.environ["BATCH_SIZE"] = str(batch)
        cfg = ref.get_model_config("gpt2_small")
        ds = cfg["train_dataset"]()
        items, metric, unit, name = 1024, "tokens_per_sec", "tokens/s", "gpt2_small"
    else:
        batch = args.per_gpu_batch or 256
        os.environ["BATCH_SIZE"] = str(batch)
        cfg = ref.get_model_config("resnet50_imagenet100")

        class _Synthetic(torch.utils.data.Dataset):  # N(0,1) NCHW images, uniform labels
            def __init__(self, n):
                g = torch.Generator().manual_seed(1234)
                self.x = torch.randn(min(n, 4 * batch), 3, 224, 224, generator=g)
                self.y = torch.randint(0, 100, (n,), generator=g)
                self.n = n

            def __len__(self):
                return self.n

            def __getitem__(self, i):
                return self.x[i % self.x.shape[0]], self.y[i]

        ds = _Synthetic((warm + steps) * batch)
        items, metric, unit, name = 1, "images_per_sec", "images/s", "resnet50"

    model = cfg["model_cls"]().to(dev)
    if os.environ.get("TNNB_REF_COMPILE") == "1":
        model = torch.compile(model, mode="max-autotune")
    criterion = cfg["criterion"]
    if cfg["optimizer_type"] == "adamw":
        optimizer = optim.AdamW(model.parameters(), lr=cfg["lr"], betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    else:
        optimizer = optim.Adam(model.parameters(), lr=cfg["lr"], betas=(0.9, 0.999), eps=1e-3, weight_decay=3e-4, amsgrad=False)

    def loader(lo, hi):
        sub = torch.utils.data.Subset(ds, range(lo * batch, hi * batch))
        return torch.utils.data.DataLoader(sub, batch_size=batch, shuffle=False, num_workers=0, pin_memory=True)

    sink = csv.writer(io.StringIO())
    ref.train_epoch(model, loader(0, warm), criterion, optimizer, dev, cfg, 0, sink)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    loss, _ = ref.train_epoch(model, loader(warm, warm + steps), criterion, optimizer, dev, cfg, 1, sink)
    e1.record()
    torch.cuda.synchronize()
    ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)
    value = batch * items * steps / (ms / 1e3)
    x0, y0 = ds[0]
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": round(value, 1), "unit": unit, "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": round(ms / steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (the reference trainer's stock precision; TF32 matmul via set_float32_matmul_precision('high'))",
        "data": "synthetic", "config": {"model": name, "global_batch": batch, "seq_len": 1024 if is_lm else None,
                                        "parallelism": "single", "path": "reference torch/torch_trainer.py train_epoch, eager"},
        "e2e": {"value": round(value, 1), "unit": unit,
                "h2d_bytes_per_step": int(batch * (x0.numel() * x0.element_size() + (y0.numel() * y0.element_size() if hasattr(y0, 'numel') else 8))),
                "d2h_bytes_per_step": 12},
        "loss_last": round(float(loss), 4),
        "note": "the timed loop is the reference's own train_epoch: it uploads each batch and reads loss/accuracy back every step",
    }), flush=True)
