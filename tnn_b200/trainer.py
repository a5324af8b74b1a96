"""Single-process trainer / validator driven by a :class:`TrainingConfig`.

Counterpart of the reference's ``train_model`` / ``validate_model`` (src/nn/train.cpp:201-660):
epoch mode (train + validation + best snapshot) or step mode (``max_steps``), gradient
accumulation, per-step CSV rows, progress lines and snapshots under
``model_snapshots/<model_name>`` in the TNNG format. Differences that matter for speed:

* the whole step (input upload, forward, loss + its gradient, backward, optimizer, gradient
  clear) is issued without a host synchronisation - loss and correct-count stay on the device
  until a progress line or CSV row needs them;
* with ``cuda_graph`` the step is captured once and replayed, so the hundreds of launches of a
  step cost one graph launch on the host;
* the optimizer state can be saved beside the weights (``<snapshot>.opt``) for a true resume.

With a ``parallel`` block in the config (or ``torchrun``) the same class drives one rank of a
data / tensor / pipeline parallel job; see :mod:`tnn_b200.parallel`.
"""
from __future__ import annotations

import math
import os
import time
from typing import Dict, Optional, Tuple

import torch

from .data.loaders import BaseLoader, create_loaders
from .models import zoo
from .nn.graph import Graph
from .nn.loss import CrossEntropyLoss, Loss, create_loss
from .nn.optim import Optimizer, create_optimizer
from .nn.schedulers import ReduceLROnPlateau, Scheduler, create_scheduler
from .ops import _lib, raw
from .ops.gemm import LAUNCHES
from .utils.config import TrainingConfig
from .utils.csv_logger import CsvLogger


def resolve_device(device_type: str) -> torch.device:
    if device_type.upper() == "CUDA" and torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def load_or_create_graph(cfg: TrainingConfig, device: torch.device) -> Graph:
    """``model_path`` (a TNNG file) wins over ``model_name`` (src/nn/train.cpp:343-409)."""
    if cfg.model_path:
        return Graph.load_state(cfg.model_path, device=device)
    g = zoo.create(cfg.model_name)
    g.compile(device=device, seed=cfg.seed)
    return g


class Trainer:
    def __init__(self, cfg: TrainingConfig, graph: Optional[Graph] = None, device: Optional[torch.device] = None,
                 train_loader: Optional[BaseLoader] = None, val_loader: Optional[BaseLoader] = None,
                 loss: Optional[Loss] = None, optimizer: Optional[Optimizer] = None, log: bool = True):
        self.cfg = cfg
        self.device = device or resolve_device(cfg.device_type)
        torch.set_num_threads(max(1, int(cfg.num_threads)))
        self.graph = graph if graph is not None else load_or_create_graph(cfg, self.device)
        self.loss = loss or create_loss(cfg.loss)
        self.optimizer = (optimizer or create_optimizer(cfg.optimizer)).attach(self.graph)
        self.scheduler: Scheduler = create_scheduler(cfg.scheduler, self.optimizer)
        self.train_loader, self.val_loader = train_loader, val_loader
        self.logger = None
        if log:
            lm = cfg.log_mode
            self.logger = CsvLogger(lm.get("log_dir", "logs"), cfg.model_name, lm.get("log_batch", True),
                                    lm.get("log_val", True), lm.get("log_epoch", True))
        self.accum = max(1, int(cfg.gradient_accumulation_steps))
        # One GPU, one backward pass per step: optionally run the update bucket by bucket on a second stream while
        # backward is still going (nn/optim.py OverlappedUpdate; `overlap_update` in the config or TNNB_OVERLAP_UPDATE=1).
        # Off by default: on GPT-2 small it measured the same step time as one update after backward (11.93 ms both).
        want = os.environ.get("TNNB_OVERLAP_UPDATE", "1" if getattr(cfg, "overlap_update", False) else "0") == "1"
        if optimizer is None and self.accum == 1 and want and isinstance(self.optimizer, Optimizer):
            from .nn.optim import OverlappedUpdate
            if OverlappedUpdate.usable(self.optimizer, self.graph):
                ov = OverlappedUpdate(self.optimizer, self.graph)
                if len(ov.spans) > 1:
                    self.optimizer = ov
                else:
                    self.graph.grad_hook = None
        self.global_step = 0
        self.micro_step = 0
        self.is_lm = self._is_language_model()
        # device-side step counter that feeds the dropout seeds (see ops.raw.SEED_OFF)
        self.step_counter = torch.zeros(1, dtype=torch.int64, device=self.device)
        if self.device.type == "cuda":
            raw.SEED_OFF["tensor"] = self.step_counter
        self._graphed = None
        self._pf = None            # (data, labels, device copies, ready event) of a batch uploaded ahead of its step
        self._pf_stream = None
        self._pf_free = None       # recorded once the staging copies have been consumed
        self._print_memory_once = bool(getattr(cfg, "print_layer_memory_usage", False))
        self.launches_per_step = 0
        # per-layer timing (profiler_type NORMAL: last step, CUMULATIVE: summed over steps)
        self.layer_profiler = None
        if str(cfg.profiler_type).upper() in ("NORMAL", "CUMULATIVE"):
            from .utils.profiling import LayerProfiler
            self.layer_profiler = LayerProfiler(self.device, source=f"rank{os.environ.get('RANK', '0')}",
                                                cumulative=str(cfg.profiler_type).upper() == "CUMULATIVE")
            self.graph.profiler = self.layer_profiler

    def _is_language_model(self) -> bool:
        from .nn.layers import Embedding
        return any(isinstance(l, Embedding) for l in self.graph.layers())

    # ------------------------------------------------------------------ one step
    def _to_device(self, data: torch.Tensor, labels: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        d = data.to(self.device, non_blocking=True)
        l = labels.to(self.device, non_blocking=True)
        if d.is_floating_point():
            d = d.to(self.graph.io_dtype)
        return d, l

    def _fwd_bwd(self, d: torch.Tensor, l: torch.Tensor, scale: float):
        g = self.graph
        in_uid, out_uid = g.input_nodes[0].uid(), g.output_nodes[0].uid()
        tracking = self._print_memory_once and g.alloc_hook is None
        if tracking:
            g.track_memory(True)   # allocator readings around every edge of this first step
        out = g.forward({in_uid: d})[out_uid]
        if self._print_memory_once:
            print("per-layer memory after the first forward pass:\n" + g.format_memory_report(), flush=True)
        in_place = isinstance(self.loss, CrossEntropyLoss) and out.is_cuda
        if in_place:
            loss, grad = self.loss.compute(out, l, scale, True, in_place=True)
        else:
            loss, grad = self.loss.compute(out, l, scale, True)
        g.backward({out_uid: grad})
        if self._print_memory_once:
            self._print_memory_once = False
            if tracking:
                print("device memory per edge (allocator readings, first step):\n" + g.alloc_hook.format(), flush=True)
                g.track_memory(False)
        return loss

    def train_step(self, data: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """Upload one batch and run forward, loss, backward and (every ``accum`` calls) the update.
        Returns the mean loss of the batch as a 1-element device tensor (no synchronisation)."""
        if self._graphed is not None:
            return self._graphed_step(data, labels)
        src = self._take_prefetched(data, labels) if self.device.type == "cuda" else None
        if src is not None:  # the step owns its inputs: the staging copies are overwritten by the next prefetch
            d, l = self._to_device(src[0].clone(), src[1].clone())
            self._release_prefetched()
        else:
            d, l = self._to_device(data, labels)
        self._resident = (d, l)
        return self._step_on_device(d, l)

    def step_resident(self) -> torch.Tensor:
        """One more step on the batch that is already on the device (no host->device traffic, no
        host synchronisation): what the device-timed benchmark number measures."""
        if self._graphed is not None:
            self.optimizer.prepare_step()
            self._graphed.replay()
            self.scheduler.step()
            self.global_step += 1
            return self._g_loss
        return self._step_on_device(*self._resident)

    def _step_on_device(self, d: torch.Tensor, l: torch.Tensor) -> torch.Tensor:
        g = self.graph
        g.set_training(True)
        g.set_step(self.global_step)
        lp = self.layer_profiler
        if lp is not None:
            lp.begin_step()
        loss = self._fwd_bwd(d, l, 1.0 / self.accum)
        if lp is not None:
            lp.end_step()
            if self.cfg.print_layer_profiling and self.global_step % max(1, self.cfg.progress_print_interval) == 0:
                print(lp.table(top=20), flush=True)
        self.micro_step += 1
        if self.micro_step % self.accum == 0:
            self.optimizer.update()
            if not getattr(self.optimizer, "clears_grads", False):
                g.zero_grads()
            self.scheduler.step()
            self.global_step += 1
            self.step_counter.add_(1)
        return loss

    # ------------------------------------------------------------ CUDA graph mode
    def _profiling(self) -> bool:
        return self.layer_profiler is not None

    def enable_cuda_graph(self, data: torch.Tensor, labels: torch.Tensor, warmup: int = 2) -> None:
        """Capture one full step and replay it afterwards; each replay is preceded by the upload of the batch into the
        graph's input buffers."""
        if self.device.type != "cuda" or self._profiling():  # events inside a captured graph carry no timing
            return
        if self.accum != 1:
            raise ValueError("cuda_graph needs gradient_accumulation_steps == 1")
        for _ in range(warmup):
            self.train_step(data, labels)
        self.optimizer.enable_device_hyper()
        # Graph inputs: device buffers in the caller's dtypes. Every step copies the batch straight from the caller's
        # (pinned) tensors into them - one DMA, no staging copy on the host - and the captured graph starts from there.
        self._d_data = torch.empty(data.shape, dtype=data.dtype, device=self.device)
        self._d_labels = torch.empty(labels.shape, dtype=labels.dtype, device=self.device)
        self._d_data.copy_(data)
        self._d_labels.copy_(labels)
        self.graph.set_training(True)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # one eager step on the capture stream (lazy attribute setup, caches)
            self.optimizer.prepare_step()
            self._captured_body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        cg = torch.cuda.CUDAGraph()
        n0 = LAUNCHES["count"]
        self.optimizer.prepare_step()
        with torch.cuda.graph(cg):
            self._g_loss = self._captured_body()
        self.launches_per_step = LAUNCHES["count"] - n0
        self._graphed = cg
        self.optimizer.step_count -= 1  # the capture pass issued no work
        self.global_step += 1           # the eager pass on the side stream was a real step
        self.scheduler.step()

    def _captured_body(self):
        d, l = self._to_device(self._d_data, self._d_labels)
        loss = self._fwd_bwd(d, l, 1.0)
        self.optimizer.update(prepared=True)
        if not getattr(self.optimizer, "clears_grads", False):
            self.graph.zero_grads()
        self.step_counter.add_(1)
        return loss

    def prefetch(self, data: torch.Tensor, labels: torch.Tensor) -> None:
        """Start the host-to-device copy of the NEXT batch on a copy stream, to run while the current step computes;
        ``train_step`` called later with the same two tensors then takes the device copies (one device-to-device copy
        into the step's inputs) instead of waiting for PCIe. With 77 MB of bf16 images per ResNet-50 step the upload
        is 1.4 ms that would otherwise sit in front of every step."""
        if self.device.type != "cuda":
            return
        if self._pf_stream is None:
            self._pf_stream = torch.cuda.Stream(device=self.device)
        old = self._pf
        if old is not None and old[2].shape == data.shape and old[2].dtype == data.dtype and old[3].shape == labels.shape \
                and old[3].dtype == labels.dtype:
            sd, sl = old[2], old[3]
        else:
            sd = torch.empty(data.shape, dtype=data.dtype, device=self.device)
            sl = torch.empty(labels.shape, dtype=labels.dtype, device=self.device)
        if self._pf_free is not None:
            self._pf_stream.wait_event(self._pf_free)  # the previous contents have been read by their step
        with torch.cuda.stream(self._pf_stream):
            sd.copy_(data, non_blocking=True)
            sl.copy_(labels, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        self._pf = (data, labels, sd, sl, ev)

    def _take_prefetched(self, data, labels):
        """Device copies of this batch if ``prefetch`` uploaded it, else None. Orders the current stream after the copy."""
        pf = self._pf
        if pf is None or pf[0] is not data or pf[1] is not labels:
            return None
        torch.cuda.current_stream().wait_event(pf[4])
        return pf[2], pf[3]

    def _release_prefetched(self):
        self._pf_free = torch.cuda.Event()
        self._pf_free.record()

    def _graphed_step(self, data, labels):
        src = self._take_prefetched(data, labels)
        if src is not None:
            self._d_data.copy_(src[0], non_blocking=True)
            self._d_labels.copy_(src[1], non_blocking=True)
            self._release_prefetched()
        else:
            self._d_data.copy_(data, non_blocking=True)
            self._d_labels.copy_(labels, non_blocking=True)
        self.optimizer.prepare_step()
        self._graphed.replay()
        self.scheduler.step()
        self.global_step += 1
        return self._g_loss

    # ------------------------------------------------------------------ validation
    @torch.no_grad()
    def validate(self, loader: Optional[BaseLoader] = None, max_batches: Optional[int] = None) -> Dict[str, float]:
        """Mean loss / accuracy over a loader in eval mode (src/nn/train.cpp:596-660)."""
        if loader is None:
            self._ensure_loaders()
            loader = self.val_loader
        g = self.graph
        g.set_training(False)
        tot_loss, tot_corr, tot_rows, n = 0.0, 0, 0, 0
        for data, labels in loader:
            d, l = self._to_device(data, labels)
            out = g.forward({g.input_nodes[0].uid(): d})[g.output_nodes[0].uid()]
            loss, _ = self.loss.compute(out, l, 1.0, False)
            tot_loss += float(loss.item())
            c = self.loss.corrects()
            if c is not None:
                tot_corr += int(c.item())
            tot_rows += l.numel() if (c is not None) else 0
            n += 1
            if max_batches and n >= max_batches:
                break
        g.set_training(True)
        mean = tot_loss / max(1, n)
        return {"loss": mean, "accuracy_pct": 100.0 * tot_corr / max(1, tot_rows), "perplexity": math.exp(min(mean, 80.0)),
                "batches": n}

    # ------------------------------------------------------------------------ fit
    def _ensure_loaders(self) -> None:
        cfg = self.cfg
        if self.train_loader is None or self.val_loader is None:
            tr, va = create_loaders(cfg.dataset_name, cfg.dataset_path, cfg.batch_size, cfg.seed,
                                    cfg.prefetch_depth if cfg.prefetch_data else 0, cfg.model_name)
            self.train_loader = self.train_loader or tr
            self.val_loader = self.val_loader or va

    def fit(self) -> Dict[str, float]:
        self._ensure_loaders()
        return self._fit_steps() if self.cfg.step_mode else self._fit_epochs()

    def _log_step(self, epoch, loss_t, t_ms, avg):
        loss = float(loss_t.item())
        corr = self.loss.corrects()
        acc = None
        if corr is not None and self._last_rows:
            acc = 100.0 * int(corr.item()) / self._last_rows
        if self.logger:
            self.logger.log_train_step(epoch=epoch, step=self.global_step, loss=loss, batch_loss=loss, avg_loss=avg(loss),
                                       avg_perplexity=math.exp(min(avg(None), 80.0)), accuracy_pct=acc,
                                       perplexity=math.exp(min(loss, 80.0)), time_ms=round(t_ms, 3))
        return loss, acc

    def _fit_steps(self) -> Dict[str, float]:
        cfg = self.cfg
        run = {"sum": 0.0, "n": 0}

        def avg(x):
            if x is not None:
                run["sum"] += x
                run["n"] += 1
            return run["sum"] / max(1, run["n"])

        last = {}
        it = iter(self.train_loader)

        def fetch():
            nonlocal it
            while True:
                try:
                    return next(it)
                except StopIteration:
                    it = iter(self.train_loader)

        nxt = fetch()
        while self.global_step < cfg.max_steps:
            data, labels = nxt
            t0 = time.perf_counter()
            if cfg.cuda_graph and self._graphed is None and self.device.type == "cuda" and self.accum == 1:
                self.enable_cuda_graph(data, labels)
            loss_t = self.train_step(data, labels)
            if self.global_step < cfg.max_steps:
                nxt = fetch()
                self.prefetch(*nxt)  # uploaded while the step just launched is computing
            self._last_rows = labels.numel()
            want = self.logger is not None or (self.global_step % max(1, cfg.progress_print_interval) == 0)
            if want:
                loss, acc = self._log_step(0, loss_t, (time.perf_counter() - t0) * 1e3, avg)
                last = {"loss": loss, "accuracy_pct": acc}
                if self.global_step % max(1, cfg.progress_print_interval) == 0:
                    print(f"step {self.global_step}/{cfg.max_steps} loss {loss:.4f} lr {self.optimizer.get_learning_rate():.3g}"
                          f" {(time.perf_counter() - t0) * 1e3:.1f} ms", flush=True)
        self.save_snapshot()
        return last

    def _fit_epochs(self) -> Dict[str, float]:
        cfg = self.cfg
        best = float("inf")
        result = {}
        for epoch in range(cfg.epochs):
            run = {"sum": 0.0, "n": 0}

            def avg(x):
                if x is not None:
                    run["sum"] += x
                    run["n"] += 1
                return run["sum"] / max(1, run["n"])

            t_epoch = time.perf_counter()
            for data, labels in self.train_loader:
                t0 = time.perf_counter()
                loss_t = self.train_step(data, labels)
                self._last_rows = labels.numel()
                loss, acc = self._log_step(epoch, loss_t, (time.perf_counter() - t0) * 1e3, avg)
                if self.global_step % max(1, cfg.progress_print_interval) == 0:
                    print(f"epoch {epoch} step {self.global_step} loss {loss:.4f} acc {acc}", flush=True)
            val = self.validate() if self.val_loader is not None else {"loss": avg(None), "accuracy_pct": None, "perplexity": None}
            if isinstance(self.scheduler, ReduceLROnPlateau):
                self.scheduler.step(val["loss"])
            if self.logger:
                self.logger.log_validation(epoch=epoch, step=self.global_step, loss=val["loss"], avg_loss=val["loss"],
                                           accuracy_pct=val.get("accuracy_pct"), perplexity=val.get("perplexity"))
                self.logger.log_epoch(epoch=epoch, step=self.global_step, loss=avg(None), avg_loss=avg(None),
                                      time_ms=round((time.perf_counter() - t_epoch) * 1e3, 3))
            print(f"epoch {epoch}: train loss {avg(None):.4f} val loss {val['loss']:.4f} val acc {val.get('accuracy_pct')}", flush=True)
            if val["loss"] < best:
                best = val["loss"]
                self.save_snapshot()
            result = {"loss": avg(None), "val_loss": val["loss"], "val_accuracy_pct": val.get("accuracy_pct")}
        return result

    # ---------------------------------------------------------------- checkpoints
    def snapshot_path(self) -> str:
        return os.path.join(self.cfg.snapshot_dir, self.cfg.model_name)

    def save_snapshot(self, path: Optional[str] = None, with_optimizer: bool = True) -> str:
        """Weights as a TNNG file; optimizer / scheduler / step counters in a ``.opt`` sidecar so that
        training can resume exactly (the TNNG file alone is a weights-only checkpoint)."""
        path = path or self.snapshot_path()
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self.graph.save_state(path)
        if with_optimizer:
            torch.save({"optimizer": {k: v.detach().cpu() for k, v in self.optimizer.state_dict().items()},
                        "scheduler": self.scheduler.state_dict(), "global_step": self.global_step,
                        "step_counter": int(self.step_counter.item()), "rng": torch.get_rng_state()}, path + ".opt")
        return path

    def load_snapshot(self, path: str) -> None:
        g2 = Graph.load_state(path, device="cpu")
        self.graph.master_flat.copy_(g2.master_flat.to(self.graph.master_flat.device))
        self.graph.sync_params_from_master()
        side = path + ".opt"
        if os.path.exists(side):
            st = torch.load(side, map_location="cpu", weights_only=False)
            self.optimizer.load_state_dict({k: v.to(self.device) if isinstance(v, torch.Tensor) and v.dim() > 0 else v
                                            for k, v in st["optimizer"].items()})
            self.scheduler.load_state_dict(st["scheduler"])
            self.global_step = int(st["global_step"])
            self.step_counter.fill_(int(st["step_counter"]))
            torch.set_rng_state(st["rng"])

    def close(self):
        if self.logger:
            self.logger.close()
        if raw.SEED_OFF["tensor"] is self.step_counter:
            raw.SEED_OFF["tensor"] = None


def train_model(cfg: TrainingConfig, **kw) -> Dict[str, float]:
    t = Trainer(cfg, **kw)
    try:
        return t.fit()
    finally:
        t.close()
