"""Per-step / validation / epoch CSV logs with the reference's file names and columns
(src/nn/csv_logger.cpp:16-132): ``<log_dir>/tunx_<model>_{batch,val,epoch}_<timestamp>.csv``."""
from __future__ import annotations

import os
import time

COLUMNS = ["epoch", "step", "timestamp_ms", "loss", "batch_loss", "avg_loss", "avg_perplexity", "accuracy_pct", "perplexity",
           "time_ms"]


class CsvLogger:
    def __init__(self, log_dir: str, model_name: str, log_batch=True, log_val=True, log_epoch=True, prefix: str = "tunx"):
        os.makedirs(log_dir, exist_ok=True)
        ts = time.strftime("%Y%m%d_%H%M%S")
        self.files = {}
        for kind, on in (("batch", log_batch), ("val", log_val), ("epoch", log_epoch)):
            if on:
                path = os.path.join(log_dir, f"{prefix}_{model_name}_{kind}_{ts}.csv")
                f = open(path, "w")
                f.write(",".join(COLUMNS) + "\n")
                f.flush()
                self.files[kind] = f
        self.paths = {k: f.name for k, f in self.files.items()}

    def _row(self, kind, **kw):
        f = self.files.get(kind)
        if f is None:
            return
        kw.setdefault("timestamp_ms", int(time.time() * 1000))
        f.write(",".join("" if kw.get(c) is None else str(kw.get(c)) for c in COLUMNS) + "\n")
        f.flush()  # every row, like the reference

    def log_train_step(self, **kw):
        self._row("batch", **kw)

    def log_validation(self, **kw):
        self._row("val", **kw)

    def log_epoch(self, **kw):
        self._row("epoch", **kw)

    def close(self):
        for f in self.files.values():
            f.close()
        self.files = {}


class WorkerCsvLogger:
    """step,event_type,time_ms,mem rows per pipeline worker (include/nn/csv_logger.hpp:76-99)."""

    def __init__(self, path: str):
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self.f = open(path, "w")
        self.f.write("step,event_type,time_ms,mem\n")

    def log(self, step: int, event_type: str, time_ms: float, mem: int = 0):
        self.f.write(f"{step},{event_type},{time_ms},{mem}\n")
        self.f.flush()

    def close(self):
        self.f.close()
