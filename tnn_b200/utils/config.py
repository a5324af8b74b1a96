"""Training configuration: every key of the reference's ``TrainingConfig``
(include/nn/train.hpp:39-81, parser src/nn/train.cpp:131-199) plus an optional ``parallel`` block.

Unknown keys are ignored and missing keys keep their defaults, as in the reference, so its
``configs/*.json`` files load unchanged. ``//`` and ``/* */`` comments are tolerated (``.jsonc``).
"""
from __future__ import annotations

import json
import re
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class ParallelConfig:
    dp: int = 1                      # data-parallel replicas
    tp: int = 1                      # tensor-parallel width
    pp: int = 1                      # pipeline stages
    microbatches: int = 1
    partition_ratios: List[float] = field(default_factory=list)
    fused_collectives: bool = True   # hand-written NVLink kernels instead of NCCL calls
    zero: bool = True                # shard optimizer state across the data-parallel group
    overlap_grad_reduce: bool = True  # start a bucket's fused reduce + update while backward is still running (pure DP)
    layout: str = ""                 # e.g. "dp8", "tp2dp4", "pp2tp2"; empty = data parallel over all ranks


@dataclass
class TrainingConfig:
    epochs: int = 10
    batch_size: int = 32
    max_steps: int = -1
    train_mode: str = "auto"          # epoch | batch | auto (batch when max_steps > 0)
    lr_initial: float = 1e-3
    gradient_accumulation_steps: int = 1
    progress_print_interval: int = 100
    num_threads: int = 8
    profiler_type: str = "NONE"       # NONE | NORMAL | CUMULATIVE
    print_layer_profiling: bool = False
    print_layer_memory_usage: bool = False
    num_microbatches: int = 2
    device_type: str = "CUDA"         # CPU | CUDA
    model_name: str = "mnist_cnn"
    model_path: str = ""
    dataset_name: str = "synthetic"
    dataset_path: str = ""
    io_dtype: str = "FP32"
    param_dtype: str = "FP32"
    compute_dtype: str = "FP32"
    prefetch_data: bool = True
    prefetch_depth: int = 2
    async_pipeline: bool = True
    augmentation: bool = False
    log_mode: Dict[str, Any] = field(default_factory=lambda: {"log_dir": "logs", "log_batch": True, "log_val": True, "log_epoch": True})
    optimizer: Dict[str, Any] = field(default_factory=lambda: {"type": "adam", "learning_rate": 1e-3})
    scheduler: Dict[str, Any] = field(default_factory=lambda: {"type": "no_op"})
    loss: Dict[str, Any] = field(default_factory=lambda: {"type": "logsoftmax_crossentropy"})
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    snapshot_dir: str = "model_snapshots"
    seed: int = 0
    cuda_graph: bool = False
    overlap_update: bool = False      # single GPU: optimizer buckets run on a second stream while backward continues
    # distributed (coordinator/worker) keys of configs/tcp_config.json; kept for compatibility
    host: str = "127.0.0.1"
    port: int = 9000
    worker_endpoints: List[Dict[str, Any]] = field(default_factory=list)
    partition_ratios: List[float] = field(default_factory=list)
    max_packet_size: int = 4 * 1024 * 1024
    skts_per_endpoint: int = 4
    local_worker_host: str = ""      # with a port: the last stage runs inside the coordinator process
    local_worker_port: int = 0

    @property
    def step_mode(self) -> bool:
        if self.train_mode == "batch":
            return True
        if self.train_mode == "epoch":
            return False
        return self.max_steps is not None and self.max_steps > 0

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: dict) -> "TrainingConfig":
        cfg = cls()
        for k, v in d.items():
            if k == "parallel" and isinstance(v, dict):
                pc = ParallelConfig()
                for pk, pv in v.items():
                    if hasattr(pc, pk):
                        setattr(pc, pk, pv)
                cfg.parallel = pc
            elif hasattr(cfg, k) and not isinstance(getattr(type(cfg), k, None), property):
                cur = getattr(cfg, k)
                if isinstance(cur, dict) and isinstance(v, dict):
                    merged = dict(cur) if k == "log_mode" else {}
                    merged.update(v)
                    setattr(cfg, k, merged)
                else:
                    setattr(cfg, k, v)
        if cfg.partition_ratios and not cfg.parallel.partition_ratios:
            cfg.parallel.partition_ratios = list(cfg.partition_ratios)
        if "optimizer" in d and "learning_rate" in d["optimizer"]:
            cfg.lr_initial = float(d["optimizer"]["learning_rate"])
        return cfg

    @classmethod
    def load_from_json(cls, path: str) -> "TrainingConfig":
        with open(path) as f:
            text = f.read()
        return cls.from_dict(json.loads(strip_json_comments(text)))


def strip_json_comments(text: str) -> str:
    """Remove // and /* */ comments that are outside of string literals, and trailing commas."""
    out, i, n, in_str = [], 0, len(text), False
    while i < n:
        c = text[i]
        if in_str:
            out.append(c)
            if c == "\\" and i + 1 < n:
                out.append(text[i + 1])
                i += 1
            elif c == '"':
                in_str = False
        elif c == '"':
            in_str = True
            out.append(c)
        elif text.startswith("//", i):
            while i < n and text[i] != "\n":
                i += 1
            continue
        elif text.startswith("/*", i):
            j = text.find("*/", i + 2)
            i = n if j < 0 else j + 2
            continue
        else:
            out.append(c)
        i += 1
    return re.sub(r",(\s*[}\]])", r"\1", "".join(out))
