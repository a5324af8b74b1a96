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

    def _train_state(self) -> dict:
        return {"scheduler": self.scheduler.state_dict(), "global_step": self.global_step,
                "step_counter": int(self.step_counter.item()), "rng": torch.get_rng_state(),
                "layout": self.topo.describe(), "world": self.topo.world}

    def save_snapshot(self, path=None, with_optimizer: bool = False, gather_tp: bool = True) -> str:
        """Writes ONE TNNG file that any layout (or the reference) can read: tensor-parallel shards are gathered
        to full tensors first (collective over the tensor-parallel group), then the first rank writes.
        ``gather_tp=False`` writes each shard as held, to ``<path>.tp<i>``.

        ``with_optimizer=True`` also saves what an exact resume needs. Pure data parallelism: the moments and the
        fp32 master values are collected from the ranks that own them and written as the same ``<path>.opt``
        sidecar a single-process trainer writes, so the job can resume on any number of ranks. With tensor
        parallelism the optimizer state follows the shard layout: every rank writes ``<path>.opt.rank<r>``
        (moments, owned fp32 master slices, scheduler, step counters), which a job of the same layout reads back.
        Collective: every rank must call it."""
        topo = self.topo
        path = path or self.snapshot_path()
        fused_opt = isinstance(self.optimizer, FusedDPOptimizer)
        full = None
        if with_optimizer and topo.tp == 1 and fused_opt:
            full = self.optimizer.full_state(topo.dp_group)
            self.graph.master_flat.copy_(full.pop("master"))    # exact fp32 values for every slice, not bf16 copies
        else:
            self._refresh_master()
        if with_optimizer and topo.tp > 1:
            st = self._train_state()
            st["optimizer"] = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in self.optimizer.state_dict().items()}
            if fused_opt:
                st["master"] = [(s["lo"], s["hi"], self.graph.master_flat[s["lo"]:s["hi"]].detach().cpu()) for s in self.optimizer.sites]
            os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
            torch.save(st, f"{path}.opt.rank{topo.rank}")
        if topo.tp > 1 and gather_tp:
            from ..models import zoo
            from .tp import gather_full_state
            fullg = zoo.create(self.cfg.model_name).compile(device="cpu", seed=self.cfg.seed)
            gather_full_state(self.graph, fullg, topo)
            if topo.dp_idx == 0 and topo.tp_idx == 0:
                os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
                fullg.save_state(path)
        elif topo.tp > 1:
            if topo.dp_idx == 0:
                super().save_snapshot(f"{path}.tp{topo.tp_idx}", with_optimizer=False)
        elif topo.dp_idx == 0:
            if full is not None:
                super().save_snapshot(path, with_optimizer=False)
                st = self._train_state()
                st["optimizer"] = {k: v.detach().cpu() for k, v in full.items()}
                torch.save(st, path + ".opt")
            else:
                super().save_snapshot(path, with_optimizer=with_optimizer)
        if dist.is_initialized():
            dist.barrier()
        return path

    def load_snapshot(self, path: str) -> None:
        """Weights from a TNNG file of the unsharded model (sharded again here when the job is tensor parallel),
        then the optimizer / scheduler / step state: this rank's ``<path>.opt.rank<r>`` if the job that wrote it had
        this layout, else the unsharded ``<path>.opt`` (written by a single process or by a data-parallel job)."""
        from ..nn.graph import Graph
        topo = self.topo
        g2 = Graph.load_state(path, device="cpu")
        if topo.tp > 1:
            from .tp import copy_full_to_shards
            copy_full_to_shards(self.graph, g2, topo)
        else:
            self.graph.master_flat.copy_(g2.master_flat.to(self.graph.master_flat.device))
            self.graph.sync_params_from_master()
        fused_opt = isinstance(self.optimizer, FusedDPOptimizer)
        mine, plain = f"{path}.opt.rank{topo.rank}", path + ".opt"
        st = None
        if os.path.exists(mine):
            st = torch.load(mine, map_location="cpu", weights_only=False)
            if st.get("layout") != topo.describe() or st.get("world") != topo.world:
                raise ValueError(f"{mine} was written by a {st.get('layout')} job of {st.get('world')} ranks; this job is "
                                 f"{topo.describe()} on {topo.world}")
            dev = self.graph.master_flat.device
            self.optimizer.load_state_dict({k: (v.to(dev) if isinstance(v, torch.Tensor) and v.dim() > 0 else v)
                                            for k, v in st["optimizer"].items()})
            for lo, hi, vals in st.get("master", []):
                self.graph.master_flat[lo:hi].copy_(vals.to(dev))
        elif os.path.exists(plain):
            if topo.tp > 1:
                raise ValueError("an unsharded optimizer state cannot be loaded into a tensor-parallel job; resume with the "
                                 "layout that wrote the snapshot")
            st = torch.load(plain, map_location="cpu", weights_only=False)
            dev = self.graph.master_flat.device
            od = {k: (v.to(dev) if isinstance(v, torch.Tensor) and v.dim() > 0 else v) for k, v in st["optimizer"].items()}
            if fused_opt:
                self.optimizer.load_full_state(od)
            else:
                self.optimizer.load_state_dict(od)
        if st is not None:
            self.scheduler.load_state_dict(st["scheduler"])
            self.global_step = int(st["global_step"])
            self.step_counter.fill_(int(st["step_counter"]))
            torch.set_rng_state(st["rng"])
        if dist.is_initialized():
            dist.barrier()

    def close(self):
        super().close()
        if self.heap is not None:
            torch.cuda.synchronize()
            dist.barrier()
            self.heap.close()
            self.heap = None
