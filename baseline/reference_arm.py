"""``bench.py --impl reference``: time the reference's own code on the same metric and configuration.

Two forms of "the reference" can run here, tried in this order:

1. Its C++/CUDA/cuDNN engine through the stock ``trainer --config`` binary, built from the reference sources by
   ``build_reference_engine.py`` (see ``reference_engine_arm.py``). The build of the UNMODIFIED sources starts,
   builds the graph and then dies with SIGSEGV in the first forward pass of every model that contains a block
   (``flash_gpt2_small``, the ResNets): ``Graph::compile`` gives the engine object to the top-level layers only
   and ``Block`` does not forward it, so ``DenseLayerImpl::forward_impl`` inside ``FlashAttentionBlockImpl``
   calls through a null engine. It is therefore not attempted by default; ``TNNB_REF_ARM=engine`` attempts it,
   ``TNNB_REF_ARM=engine-fixed`` runs the build made with ``--fix-block-engine`` (two forwarding methods added
   to one header at build time) and labels its line accordingly.
2. (default) Its PyTorch trainer ``torch/torch_trainer.py``, imported UNMODIFIED from ``baseline/_ref/tunx_torch``: its
   own model class (``GPT2Small`` / ``ResNet50ImageNet100``), model registry entry (batch size, optimizer
   type, learning rate), the optimizer construction of its ``main``, ``torch.compile(mode="max-autotune")``
   as its ``main`` applies it (compile time falls into the warm-up; eager only if compiling raises, or with
   ``TNNB_REF_COMPILE=0``, and the line says which) and its own ``train_epoch`` loop, fed by its own
   ``OpenWebTextDataset`` reading a synthetic ``train.bin`` of uniform random token ids (or by a synthetic
   image iterable for ResNet-50).

None of this repository's models, kernels or engine are on either path. Both are single-GPU programs (the
reference has no data- or tensor-parallel mode), so for N > 1 this arm reports ``unavailable``.
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
    """Print the reference arm's line for ``args.model``. For the default model (GPT-2 small) the line also carries a
    ``resnet50`` sub-record - the other half of the headline metric - measured by a second run of this arm in a
    child process (so that a failure or an over-long ``torch.compile`` of the CNN cannot lose the GPT-2 number);
    ``TNNB_BENCH_RESNET=0`` leaves it out."""
    line = _measure(args)
    if line is None:
        return
    rank = int(os.environ.get("RANK", "0"))
    if args.model == "gpt2_small" and rank == 0 and os.environ.get("TNNB_BENCH_RESNET", "1") != "0":
        import subprocess
        cmd = [sys.executable, os.path.join(os.path.dirname(HERE), "bench.py"), "--impl", "reference", "--model", "resnet50", "--gpus", "1",
               "--steps", str(args.steps), "--warmup", str(args.warmup)]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=float(os.environ.get("TNNB_REF_RESNET_TIMEOUT", "900")))
            rows = [l for l in r.stdout.splitlines() if l.startswith("{")]
            sub = json.loads(rows[-1]) if rows else {"unavailable": f"exit {r.returncode}: {r.stderr.strip()[-200:]}"}
        except subprocess.TimeoutExpired:
            sub = {"unavailable": "the reference ResNet-50 run did not finish within its time limit (torch.compile max-autotune)"}
        except Exception as e:
            sub = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        keep = ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "dtype", "config", "e2e", "loss_last", "unavailable")
        line["resnet50"] = {k: sub[k] for k in keep if k in sub}
    print(json.dumps(line), flush=True)


def _measure(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1 or args.gpus > 1:
        if rank == 0:
            _unavailable("the reference trainer (C++ engine and torch/torch_trainer.py alike) is single-GPU; it has no data- or "
                         "tensor-parallel mode to run at N > 1")
        return
    import numpy as np
    import torch

    if not torch.cuda.is_available():
        _unavailable("no CUDA device")
        return
    engine_error = None
    which = os.environ.get("TNNB_REF_ARM", "torch")
    if args.model == "gpt2_small" and which in ("engine", "engine-fixed"):
        from . import reference_engine_arm as eng

        fixed = which == "engine-fixed"
        if eng.available(fixed):
            batch = args.per_gpu_batch or 8
            warm, steps = max(3, args.warmup), args.steps
            try:
                r = eng.run_engine("gpt2_small", batch, warm, steps, dtype=os.environ.get("TNNB_REF_DTYPE", ""), fixed=fixed)
                return ({
                    "impl": "reference", "metric": "tokens_per_sec", "value": r["value"], "unit": "tokens/s", "n_gpus": 1,
                    "steps": steps, "warmup": warm, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                    "vs_baseline": None, "dtype": r["dtype"], "data": "synthetic",
                    "config": {"model": "gpt2_small", "global_batch": batch, "seq_len": 1024, "parallelism": "single", "path": r["path"]},
                    "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": r["h2d_bytes_per_step"],
                            "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
                    "loss_last": r["loss_last"], "run_ms": r["run_ms"],
                    "note": "the timed loop is the reference trainer's own: it uploads each batch from host memory and reads the loss "
                            "back every step, so value and e2e are the same measurement",
                })
            except Exception as e:  # fall through to the reference's PyTorch trainer, and say why
                engine_error = f"{type(e).__name__}: {e}"[:500]
        else:
            engine_error = "the reference trainer binary is not present (python baseline/build_reference_engine.py --src <checkout>)"
    elif args.model == "gpt2_small":
        engine_error = ("not attempted: the build of the unmodified C++ engine dies with SIGSEGV in the first forward pass "
                        "(null engine inside blocks, DenseLayerImpl::forward_impl); TNNB_REF_ARM=engine-fixed runs the patched build")
    if not os.path.exists(os.path.join(REF_DIR, "torch_trainer.py")):
        _unavailable("neither the built reference engine nor baseline/_ref/tunx_torch/torch_trainer.py (a copy of the reference's "
                     "torch/ directory) is present" + (f"; engine: {engine_error}" if engine_error else ""))
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
    compiled = "eager (TNNB_REF_COMPILE=0)"
    if os.environ.get("TNNB_REF_COMPILE", "1") != "0":
        eager_model = model
        try:  # as the script's main() does; the first batches trigger the compilation, so check it here
            model = torch.compile(model, mode="max-autotune")
            xb = next(iter(torch.utils.data.DataLoader(ds, batch_size=batch)))[0].to(dev)
            model(xb)
            compiled = "torch.compile(mode='max-autotune')"
        except Exception as e:
            model = eager_model
            compiled = f"eager (torch.compile raised {type(e).__name__})"
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
    return ({
        "impl": "reference", "metric": metric, "value": round(value, 1), "unit": unit, "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": round(ms / steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (the reference trainer's stock precision; TF32 matmul via set_float32_matmul_precision('high'))",
        "data": "synthetic", "config": {"model": name, "global_batch": batch, "seq_len": 1024 if is_lm else None,
                                        "parallelism": "single", "path": "reference torch/torch_trainer.py train_epoch, " + compiled},
        "e2e": {"value": round(value, 1), "unit": unit,
                "h2d_bytes_per_step": int(batch * (x0.numel() * x0.element_size() + (y0.numel() * y0.element_size() if hasattr(y0, 'numel') else 8))),
                "d2h_bytes_per_step": 12},
        "loss_last": round(float(loss), 4), **({"engine_error": engine_error} if engine_error else {}),
        "note": "the timed loop is the reference's own train_epoch: it uploads each batch and reads loss/accuracy back every step",
    })
