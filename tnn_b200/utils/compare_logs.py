"""Throughput and loss comparison of training logs (the arithmetic of the reference's plotting scripts).

The reference compares its own per-step CSV with the log of its PyTorch trainer: throughput is
``batch_size / (time_ms / 1000)`` (torch/plot_compare_resnet50.py:37-39), converted to TFLOP/s with fixed costs per
sample - 12.3 GFLOP per ResNet-50 image (torch/plot_compare_resnet50.py:41-45) and ``6 x 117 M`` FLOP per GPT-2 small
token (torch/plot_compare_gpt2_loss.py:227) - and the loss curves are smoothed with a rolling mean. This module does
the same on any number of logs and prints a table (and writes the per-step series as one CSV); it draws nothing, so it
needs no plotting library.

    python -m tnn_b200.utils.compare_logs --batch-size 256 --model resnet50 logs/tunx_*_batch_*.csv other/batch_log.csv

Accepted files: this framework's and the reference's ``*_batch_*.csv`` (columns ``step, batch_loss | loss, time_ms``)
and the reference PyTorch trainer's batch log (``epoch, step, loss, accuracy_pct, time_ms``, or rows tagged
``phase == train_batch`` with ``batch_total_time`` in seconds).
"""
from __future__ import annotations

import argparse
import csv
import json
import statistics
import sys
from typing import Dict, List, Optional

GFLOP_PER_SAMPLE = {"resnet50": 12.3, "gpt2_small": 6 * 117e6 / 1e9}  # gpt2: per token


def _num(v) -> Optional[float]:
    try:
        return float(v)
    except (TypeError, ValueError):
        return None


def load_steps(path: str) -> List[Dict[str, float]]:
    """Rows of one log as ``{"loss": ..., "time_ms": ..., "accuracy_pct": ...}`` in file order; rows without a loss
    (validation lines, broken lines) are dropped like the reference's ``dropna`` does."""
    out = []
    with open(path, newline="") as f:
        for row in csv.DictReader(f):
            if row.get("phase") not in (None, "", "train_batch"):
                continue
            loss = _num(row.get("batch_loss")) if row.get("batch_loss") not in (None, "") else _num(row.get("loss"))
            if loss is None:
                continue
            t = _num(row.get("time_ms"))
            if t is None and _num(row.get("batch_total_time")) is not None:
                t = _num(row.get("batch_total_time")) * 1e3
            acc = _num(row.get("accuracy_pct")) if row.get("accuracy_pct") not in (None, "") else _num(row.get("accuracy_percent"))
            out.append({"loss": loss, "time_ms": t, "accuracy_pct": acc, "batch_size": _num(row.get("batch_size"))})
    return out


def rolling_mean(xs: List[float], k: int) -> List[float]:
    if k <= 1:
        return list(xs)
    out, s = [], 0.0
    for i, x in enumerate(xs):
        s += x
        if i >= k:
            s -= xs[i - k]
        out.append(s / min(i + 1, k))
    return out


def summarize(path: str, batch_size: int, samples_per_item: int = 1, gflop_per_sample: float = 0.0, skip: int = 0,
              smooth: int = 20) -> Dict[str, float]:
    """``samples_per_item`` is the sequence length for language models (throughput in tokens/s)."""
    rows = load_steps(path)
    if rows and rows[0]["batch_size"]:
        batch_size = int(rows[0]["batch_size"])
    timed = [r["time_ms"] for r in rows[skip:] if r["time_ms"] and r["time_ms"] > 0]
    res: Dict[str, float] = {"file": path, "steps": len(rows), "batch_size": batch_size}
    if timed:
        per_step = batch_size * samples_per_item
        med = statistics.median(timed)
        res.update(median_ms=round(med, 3), mean_ms=round(statistics.fmean(timed), 3),
                   throughput=round(per_step / (med / 1e3), 1))
        if gflop_per_sample:
            res["tflops"] = round(per_step * gflop_per_sample / (med / 1e3) / 1e3, 2)
    if rows:
        sm = rolling_mean([r["loss"] for r in rows], smooth)
        res.update(first_loss=round(rows[0]["loss"], 5), final_loss_smoothed=round(sm[-1], 5), min_loss_smoothed=round(min(sm), 5))
        accs = [r["accuracy_pct"] for r in rows if r["accuracy_pct"] is not None]
        if accs:
            res["final_accuracy_pct"] = round(rolling_mean(accs, smooth)[-1], 3)
    return res


def write_series(paths: List[str], out_csv: str, smooth: int) -> None:
    """One row per global step, one smoothed-loss and one time column per log."""
    series = [load_steps(p) for p in paths]
    sm = [rolling_mean([r["loss"] for r in s], smooth) for s in series]
    with open(out_csv, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["global_step"] + [f"{c}[{i}]" for i in range(len(paths)) for c in ("loss_smoothed", "time_ms")])
        for step in range(max((len(s) for s in series), default=0)):
            row = [step + 1]
            for s, m in zip(series, sm):
                row += [m[step], s[step]["time_ms"]] if step < len(s) else ["", ""]
            w.writerow(row)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="tnn_b200.utils.compare_logs", description=__doc__.split("\n\n")[0])
    ap.add_argument("logs", nargs="+")
    ap.add_argument("--batch-size", type=int, default=128, help="used when a log has no batch_size column (reference default 128)")
    ap.add_argument("--seq-len", type=int, default=1, help="tokens per sample for language models")
    ap.add_argument("--model", default="", choices=["", *GFLOP_PER_SAMPLE], help="fixed cost per sample for the TFLOP/s column")
    ap.add_argument("--gflop-per-sample", type=float, default=0.0)
    ap.add_argument("--skip", type=int, default=0, help="leading steps left out of the timing statistics (warm-up)")
    ap.add_argument("--smooth", type=int, default=20)
    ap.add_argument("--series-csv", default="", help="also write the per-step smoothed losses and times to this file")
    a = ap.parse_args(argv)
    g = a.gflop_per_sample or GFLOP_PER_SAMPLE.get(a.model, 0.0)
    rows = [summarize(p, a.batch_size, a.seq_len, g, a.skip, a.smooth) for p in a.logs]
    base = rows[0].get("throughput")
    for r in rows:
        if base and r.get("throughput"):
            r["vs_first"] = round(r["throughput"] / base, 3)
        print(json.dumps(r))
    if a.series_csv:
        write_series(a.logs, a.series_csv, a.smooth)
    return 0


if __name__ == "__main__":
    sys.exit(main())
