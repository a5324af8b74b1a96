"""One rank of a data / tensor / pipeline parallel training job on a single NVSwitch node.

This is what replaces the reference's coordinator/worker runtime over TCP or RoCE
(include/distributed/{coordinator,worker}.hpp): an SPMD program, one process per GPU started by
``torchrun``, where the commands of the reference protocol (``FORWARD_JOB``, ``BACKWARD_JOB``,
``UPDATE_PARAMETERS`` ...) become method calls in program order. ``torch.distributed`` is used
for rendez-vous, handle exchange and pipeline send/recv; the bandwidth-heavy collectives are the
fused kernels of csrc/kernels/comm_fused.cu unless ``fused_collectives`` is switched off.

Layout strings: ``dp8``, ``tp2dp4``, ``pp4tp2``, ``pp2dp4`` ... Rank order is tp fastest, then dp,
then pp, so a tensor-parallel pair always sits on adjacent GPUs.
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..models import zoo
from ..nn.optim import create_optimizer
from ..trainer import Trainer
from ..utils.config import TrainingConfig
from .dp import FusedDPOptimizer, NcclDPOptimizer, Region
from .symm import SymmetricHeap


def parse_layout(layout: str) -> Dict[str, int]:
    out = {"dp": 1, "tp": 1, "pp": 1}
    for k, v in re.findall(r"(dp|tp|pp)(\d+)", layout.lower()):
        out[k] = int(v)
    return out


def default_layout(world: int, model_name: str) -> str:
    """Pure data parallelism: every zoo model (GPT-2 medium included) fits one 180 GB GPU many times over, so
    sharding the model only adds communication. Tensor / pipeline layouts are chosen explicitly
    (``tp2dp4``, ``pp2tp2`` ...)."""
    if world <= 1:
        return "single"
    return f"dp{world}"


class Topology:
    """Process groups of a (pp, dp, tp) grid; rank = (pp_idx * dp + dp_idx) * tp + tp_idx."""

    def __init__(self, layout: str):
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        d = parse_layout(layout)
        self.tp, self.dp, self.pp = d["tp"], d["dp"], d["pp"]
        if self.tp * self.dp * self.pp != self.world:
            if self.tp * self.pp <= self.world and self.world % (self.tp * self.pp) == 0 and d["dp"] == 1:
                self.dp = self.world // (self.tp * self.pp)
            else:
                raise ValueError(f"layout {layout!r} does not match world size {self.world}")
        self.tp_idx = self.rank % self.tp
        self.dp_idx = (self.rank // self.tp) % self.dp
        self.pp_idx = self.rank // (self.tp * self.dp)
        self.tp_ranks = [self.rank - self.tp_idx + t for t in range(self.tp)]
        self.dp_ranks = [(self.pp_idx * self.dp + d_) * self.tp + self.tp_idx for d_ in range(self.dp)]
        self.stage_ranks = [(self.pp_idx * self.dp + d_) * self.tp + t for d_ in range(self.dp) for t in range(self.tp)]
        self.pp_ranks = [(p * self.dp + self.dp_idx) * self.tp + self.tp_idx for p in range(self.pp)]
        self.tp_group = self.dp_group = self.stage_group = None
        if self.world > 1:
            # every rank must create every group, in the same order
            for p in range(self.pp):
                for d_ in range(self.dp):
                    ranks = [(p * self.dp + d_) * self.tp + t for t in range(self.tp)]
                    g = dist.new_group(ranks) if self.tp > 1 else None
                    if ranks == self.tp_ranks:
                        self.tp_group = g
                for t in range(self.tp):
                    ranks = [(p * self.dp + d_) * self.tp + t for d_ in range(self.dp)]
                    g = dist.new_group(ranks) if self.dp > 1 else None
                    if ranks == self.dp_ranks:
                        self.dp_group = g
                ranks = [(p * self.dp + d_) * self.tp + t for d_ in range(self.dp) for t in range(self.tp)]
                g = dist.new_group(ranks) if (self.pp > 1 and len(ranks) > 1) else None
                if ranks == self.stage_ranks:
                    self.stage_group = g

    def describe(self) -> str:
        parts = [f"{k}{v}" for k, v in (("pp", self.pp), ("tp", self.tp), ("dp", self.dp)) if v > 1]
        return "".join(parts) or "single"


class ParallelTrainer(Trainer):
    """Trainer for one rank. Differences from :class:`Trainer`: the flat parameter / gradient slabs
    live in the symmetric heap, the optimizer step is the fused reduce + update + broadcast kernel,
    transformer blocks run tensor-parallel when ``tp > 1`` and the model is cut into pipeline
    stages by the partitioner when ``pp > 1``."""

    def __init__(self, cfg: TrainingConfig, layout: str = "", fused: Optional[bool] = None, log: bool = True,
                 heap_bytes: Optional[int] = None):
        assert dist.is_initialized(), "ParallelTrainer needs torch.distributed (launch with torchrun)"
        local = int(os.environ.get("LOCAL_RANK", "0"))
        device = torch.device("cuda", local) if torch.cuda.is_available() and cfg.device_type.upper() == "CUDA" else torch.device("cpu")
        self.topo = Topology(layout or default_layout(dist.get_world_size(), cfg.model_name))
        topo = self.topo
        self.fused = (cfg.parallel.fused_collectives if fused is None else fused) and device.type == "cuda"
        self.local_batch = cfg.batch_size              # sequences / images this rank reads per step
        self.global_batch = cfg.batch_size * topo.dp * (topo.tp if topo.tp > 1 else 1)
        if topo.tp > 1:
            # the ranks of a tensor-parallel group work on the same sequences, each on its share of the rows
            self.local_batch = cfg.batch_size * topo.tp
        self.data_rank = topo.pp_idx * 0 + topo.dp_idx  # ranks that must read the same batch share this id
        self.heap = None
        graph = zoo.create(cfg.model_name)
        alloc = None
        if device.type == "cuda" and self.fused:
            nparams = 0
            heap_bytes = heap_bytes or int(os.environ.get("TNNB_HEAP_BYTES", str(6 << 30)))
            self.heap = SymmetricHeap(heap_bytes, None, device)
            alloc = lambda n, dt: self.heap.alloc((n,), dt)  # noqa: E731
        if topo.tp > 1:
            from .tp import shard_graph_for_tp
            shard_graph_for_tp(graph, topo)
        graph.compile(device=device, seed=cfg.seed, alloc=alloc)
        for l in graph.layers():
            l.seed_base = topo.rank * 7919
        opt = create_optimizer(cfg.optimizer)
        total = graph.total_elems
        scale = 1.0 / (topo.dp * topo.tp)
        if topo.tp > 1:
            from .tp import tp_regions
            from .tp_chain import install_tp_segments
            regions = tp_regions(graph, topo)
            install_tp_segments(graph, topo, self.heap, fused=self.fused)
        else:
            regions = [Region(0, total, topo.dp_ranks, topo.dp_group)]
        if self.fused:
            # gradient reduction overlapped with backward: pure data parallelism with one backward pass per step
            overlap = (cfg.parallel.overlap_grad_reduce and topo.tp == 1 and topo.pp == 1 and topo.dp > 1
                       and int(cfg.gradient_accumulation_steps) == 1 and os.environ.get("TNNB_DP_OVERLAP", "1") != "0")
            optimizer = FusedDPOptimizer(opt, graph, self.heap, regions, scale, overlap=overlap)
            optimizer.attach = lambda g: optimizer  # already bound
        else:
            optimizer = NcclDPOptimizer(opt, graph, regions, scale)
            optimizer.attach = lambda g: optimizer
        super().__init__(cfg, graph=graph, device=device, optimizer=optimizer, log=log and topo.rank == 0)

    def _fwd_bwd(self, d, l, scale):
        topo = self.topo
        if topo.tp > 1:
            # the head and the loss see this rank's share of the rows only
            flat = l.reshape(-1)
            rows = flat.numel() // topo.tp
            l = flat[topo.tp_idx * rows:(topo.tp_idx + 1) * rows]
        return super()._fwd_bwd(d, l, scale)

    def _refresh_master(self) -> None:
        """With the sharded optimizer every rank holds fp32 master values only for its own slice: refresh the
        other slices from the (broadcast) compute copy."""
        g = self.graph
        if g.master_flat is not g.params_flat and isinstance(self.optimizer, FusedDPOptimizer):
            mine = torch.zeros_like(g.trainable_mask)
            for s in getattr(self.optimizer, "sites", []):
                mine[s["lo"]:s["hi"]] = True
            g.master_flat.copy_(torch.where(mine, g.master_flat, g.params_flat.float()))

    def save_snapshot(self, path=None, with_optimizer: bool = False, gather_tp: bool = True) -> str:
        """Writes ONE TNNG file that any layout (or the reference) can read: tensor-parallel shards are gathered
        to full tensors first (collective over the tensor-parallel group), then the first rank writes.
        ``gather_tp=False`` writes each shard as held, to ``<path>.tp<i>``."""
        self._refresh_master()
        path = path or self.snapshot_path()
        if self.topo.tp > 1 and gather_tp:
            from ..models import zoo
            from .tp import gather_full_state
            full = zoo.create(self.cfg.model_name).compile(device="cpu", seed=self.cfg.seed)
            gather_full_state(self.graph, full, self.topo)
            if self.topo.dp_idx == 0 and self.topo.tp_idx == 0:
                os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
                full.save_state(path)
            return path
        if self.topo.tp > 1:
            path = f"{path}.tp{self.topo.tp_idx}"
        if self.topo.dp_idx == 0:
            return super().save_snapshot(path, with_optimizer=False)
        return path

    def close(self):
        super().close()
        if self.heap is not None:
            torch.cuda.synchronize()
            dist.barrier()
            self.heap.close()
            self.heap = None
