"""Pipeline parallelism: 1F1B over the stages produced by the graph partitioner.

The reference runs its pipeline as a coordinator that injects every micro-batch into stage 0 and
workers that forward activations / gradients to their neighbours over TCP or RoCE through host
memory, with the loss computed on the coordinator (include/distributed/coordinator.hpp:186-244,
worker.hpp:145-168). Here every rank owns one stage and runs the same program: the schedule is
the warm-up / steady 1F1B / cool-down order of ``one_f_one_b``, boundary tensors travel GPU to GPU
with NCCL point-to-point (``isend`` / ``irecv``; receives are posted before the compute they
overlap with), and the last stage computes the loss itself. ``FORWARD_JOB`` / ``BACKWARD_JOB`` /
``UPDATE_PARAMETERS`` of the reference protocol correspond to ``F`` / ``B`` entries of the schedule
and the optimizer call at the end of ``train_step``.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..models import zoo
from ..nn.graph import Graph, infer_shapes, partition_graph
from ..nn.loss import CrossEntropyLoss, create_loss
from ..nn.optim import create_optimizer
from ..nn.schedulers import create_scheduler
from ..utils.config import TrainingConfig
from .dp import FusedDPOptimizer, NcclDPOptimizer, Region
from .runtime import Topology
from .symm import SymmetricHeap


def one_f_one_b(stage: int, n_stages: int, n_micro: int) -> List[Tuple[str, int]]:
    """Order of forward (``("F", m)``) and backward (``("B", m)``) passes of one stage."""
    warm = min(n_stages - stage - 1, n_micro)
    ops: List[Tuple[str, int]] = [("F", m) for m in range(warm)]
    f, b = warm, 0
    while f < n_micro:
        ops.append(("F", f))
        f += 1
        ops.append(("B", b))
        b += 1
    while b < n_micro:
        ops.append(("B", b))
        b += 1
    return ops


def gpipe(stage: int, n_stages: int, n_micro: int) -> List[Tuple[str, int]]:
    """All forwards, then all backwards (the reference's "async" injection order)."""
    return [("F", m) for m in range(n_micro)] + [("B", m) for m in range(n_micro)]


def block_aligned_ratios(graph: Graph, n_stages: int) -> List[float]:
    """Partition ratios that cut a transformer graph only between blocks (edge counts per stage, which
    the largest-remainder rule reproduces exactly). Needed with tensor parallelism, whose fused
    segments cover whole blocks; other graphs get an even split."""
    from ..nn.graph import _GPTChain
    graph.sort()
    cons: Dict[int, List[int]] = {}
    for i, e in enumerate(graph.edges):
        for p in e.producers:
            cons.setdefault(id(p), []).append(i)
    outs = {id(n) for n in graph.output_nodes}
    starts = []
    i = 0
    while i < len(graph.edges):
        if _GPTChain._match_block(graph, i, cons, outs):
            starts.append(i)
            i += 10
        else:
            i += 1
    n_e = len(graph.edges)
    if len(starts) < n_stages:
        return [1.0] * n_stages
    per, extra = divmod(len(starts), n_stages)
    cuts, k = [], 0
    for s in range(n_stages - 1):
        k += per + (1 if s < extra else 0)
        cuts.append(starts[k])
    bounds = [0] + cuts + [n_e]
    return [float(bounds[j + 1] - bounds[j]) for j in range(n_stages)]


class PipelineTrainer:
    """One rank of a ``pp x dp`` (optionally ``x tp``) job. ``train_step(data, labels)`` takes the
    rank's whole batch, splits it into ``microbatches`` and runs one optimizer step."""

    def __init__(self, cfg: TrainingConfig, layout: str, fused: Optional[bool] = None, schedule: str = "1f1b",
                 graph: Optional[Graph] = None, heap_bytes: Optional[int] = None):
        assert dist.is_initialized()
        self.cfg = cfg
        self.topo = topo = Topology(layout)
        local = int(os.environ.get("LOCAL_RANK", "0"))
        on_gpu = torch.cuda.is_available() and cfg.device_type.upper() == "CUDA"
        self.device = torch.device("cuda", local) if on_gpu else torch.device("cpu")
        self.fused = (cfg.parallel.fused_collectives if fused is None else fused) and on_gpu and (topo.dp > 1 or topo.tp > 1)
        self.micro = max(1, int(cfg.parallel.microbatches if cfg.parallel.microbatches > 1 else cfg.num_microbatches))
        self.schedule = one_f_one_b if schedule == "1f1b" else gpipe
        full = graph if graph is not None else zoo.create(cfg.model_name)
        ratios = list(cfg.parallel.partition_ratios) or block_aligned_ratios(full, topo.pp)
        if len(ratios) != topo.pp:
            raise ValueError(f"{len(ratios)} partition ratios for {topo.pp} pipeline stages")
        if topo.tp > 1:
            from .tp import shard_graph_for_tp
            shard_graph_for_tp(full, topo)
        self.full = full
        stages = partition_graph(full, ratios)
        self.stage = stages[topo.pp_idx]
        self.first, self.last = topo.pp_idx == 0, topo.pp_idx == topo.pp - 1
        # tensors exchanged with the neighbours, in one fixed (sorted) order on both sides of a boundary
        self.recv_uids = sorted(self.stage.input_uids) if topo.pp_idx > 0 else []
        self.send_uids = sorted(stages[topo.pp_idx + 1].input_uids) if topo.pp_idx < topo.pp - 1 else []
        missing = [u for u in self.send_uids if u not in self.stage.output_uids]
        if missing:
            raise NotImplementedError(f"stage {topo.pp_idx + 1} needs {missing} from a stage further back than its neighbour")
        self.stage.input_requires_grad = not self.first
        self.heap = None
        alloc = None
        if self.fused:
            self.heap = SymmetricHeap(heap_bytes or int(os.environ.get("TNNB_HEAP_BYTES", str(6 << 30))), None, self.device)
            alloc = lambda n, dt: self.heap.alloc((n,), dt)  # noqa: E731
        self.stage.compile(device=self.device, seed=cfg.seed + 17 * topo.pp_idx, alloc=alloc)
        for l in self.stage.layers():
            l.seed_base = topo.rank * 7919
        opt = create_optimizer(cfg.optimizer)
        scale = 1.0 / (topo.dp * topo.tp)
        if topo.tp > 1:
            from .tp import tp_regions
            from .tp_chain import install_tp_segments
            regions = tp_regions(self.stage, topo)
            install_tp_segments(self.stage, topo, self.heap, fused=self.fused, ring=topo.pp)
        else:
            regions = [Region(0, self.stage.total_elems, topo.dp_ranks, topo.dp_group)]
        if self.fused:
            self.optimizer = FusedDPOptimizer(opt, self.stage, self.heap, regions, scale)
        elif topo.dp > 1 or topo.tp > 1:
            self.optimizer = NcclDPOptimizer(opt, self.stage, regions, scale)
        else:
            self.optimizer = opt.attach(self.stage)
        self.scheduler = create_scheduler(cfg.scheduler, self.optimizer)
        self.loss = create_loss(cfg.loss)
        # Rendezvous of a tensor-parallel group (fused path): the fused kernels of a stage hand rows to each other with
        # waits that are bounded at about two seconds, which is ample for ranks that run in step but not for a rank
        # whose boundary tensor is still on its way through the pipeline (a neighbour stage that is late, a
        # connection NCCL is still setting up, a checkpoint write). So the members of a group meet right after each
        # of them has received a micro-batch's boundary tensor - a flag store into every partner's memory and a
        # stream-ordered wait for theirs, with a limit of its own (ten seconds, reported separately) - and only then
        # enter the stage's kernels together.
        self._rv = None
        if self.fused and topo.tp > 1:
            import ctypes
            from ..ops import _lib
            lib = _lib.load()
            lib.tnnb_flag_wait.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p]
            lib.tnnb_flag_set.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p]
            flags = self.heap.alloc((16,), torch.int32)
            peers = self.heap.peer_ptrs(flags, topo.tp_ranks)
            self._rv = {"lib": lib, "flags": flags, "mine": flags.data_ptr(), "epoch": 0,
                        "others": [(t, peers[t]) for t in range(topo.tp) if t != topo.tp_idx]}
        self.prev = topo.pp_ranks[topo.pp_idx - 1] if not self.first else None
        self.next = topo.pp_ranks[topo.pp_idx + 1] if not self.last else None
        self.global_step = 0
        self._p2p_warm = False
        self._shapes: Optional[Dict[str, Tuple[int, ...]]] = None
        self.local_batch = cfg.batch_size * (topo.tp if topo.tp > 1 else 1)
        self.global_batch = self.local_batch * topo.dp
        self.data_rank = topo.dp_idx
        # One communicator per direction and neighbour pair: with a single communicator two neighbours
        # can each have a send queued ahead of the receive the other one is waiting for (1F1B makes the
        # forward and backward message orders differ on the two sides), which NCCL would deadlock on.
        self.fwd_group: Dict[Tuple[int, int], object] = {}
        self.bwd_group: Dict[Tuple[int, int], object] = {}
        for p in range(topo.pp - 1):
            for d_ in range(topo.dp):
                for t in range(topo.tp):
                    a, b = (p * topo.dp + d_) * topo.tp + t, ((p + 1) * topo.dp + d_) * topo.tp + t
                    self.fwd_group[(a, b)] = dist.new_group([a, b])
                    self.bwd_group[(a, b)] = dist.new_group([a, b])
        # NCCL builds a communicator on first use, which can take seconds; do it now, on every rank, so that no
        # rank sits in that set-up while its tensor-parallel partner is already inside a fused kernel whose
        # cross-rank waits are bounded.
        if on_gpu:
            tok = torch.zeros(1, device=self.device)
            for (a, b), grp in sorted(self.fwd_group.items()):
                if topo.rank in (a, b):
                    for g in (grp, self.bwd_group[(a, b)]):
                        if topo.rank == a:
                            dist.send(tok, b, group=g)
                        else:
                            dist.recv(tok, a, group=g)
            torch.cuda.synchronize()
        dist.barrier()

    # ------------------------------------------------------------------ shapes of the boundaries
    def _boundary_shapes(self, mb_input_shape: Tuple[int, ...]) -> Dict[str, Tuple[int, ...]]:
        if self._shapes is None or self._shapes.get("__in") != tuple(mb_input_shape):
            in_uid = self.full.input_nodes[0].uid()
            sh = infer_shapes(self.full, {in_uid: tuple(mb_input_shape)})
            if self.topo.tp > 1:
                # inside a tensor-parallel job the residual stream crosses a stage boundary as row shards
                for uid in set(self.stage.input_uids + self.stage.output_uids):
                    s = sh[uid]
                    if len(s) == 3:
                        sh[uid] = (1, s[0] * s[1] // self.topo.tp, s[2])
            sh["__in"] = tuple(mb_input_shape)
            self._shapes = sh
        return self._shapes

    # ------------------------------------------------------------------------------ p2p helpers
    def _group(self, peer: int, forward: bool):
        me = self.topo.rank
        key = (min(me, peer), max(me, peer))
        return (self.fwd_group if forward else self.bwd_group)[key]

    def _recv(self, uids: Sequence[str], src: int, shapes) -> Dict[str, torch.Tensor]:
        out, reqs = {}, []
        grp = self._group(src, forward=src < self.topo.rank)
        for uid in uids:
            t = torch.empty(shapes[uid], dtype=self.stage.io_dtype, device=self.device)
            reqs.append(dist.irecv(t, src=src, group=grp))
            out[uid] = t
        for r in reqs:
            r.wait()
        return out

    def _tp_rendezvous(self) -> None:
        """See the constructor: every member of the tensor-parallel group calls this at the same points of the schedule."""
        rv = self._rv
        if rv is None:
            return
        import ctypes
        from ..ops import _lib
        rv["epoch"] += 1
        st, status = _lib.stream(), _lib.ptr(_lib.status_word(self.device))
        for t, base in rv["others"]:   # my slot in the partner's flag array
            _lib.check_rc(rv["lib"].tnnb_flag_set(ctypes.c_void_p(base + 4 * self.topo.tp_idx), rv["epoch"], st), "tnnb_flag_set")
        for t, _ in rv["others"]:      # the partner's slot in mine
            _lib.check_rc(rv["lib"].tnnb_flag_wait(ctypes.c_void_p(rv["mine"] + 4 * t), rv["epoch"], 10_000_000_000, status, st),
                          "tnnb_flag_wait")

    def _send(self, tensors: Dict[str, torch.Tensor], uids: Sequence[str], dst: int) -> List:
        reqs = []
        grp = self._group(dst, forward=dst > self.topo.rank)
        for uid in uids:
            reqs.append(dist.isend(tensors[uid].contiguous(), dst=dst, group=grp))
        return reqs

    def _warm_p2p(self, shapes) -> None:
        """Exchange boundary-sized dummy tensors with both neighbours, in both directions, before the first real step.
        NCCL opens the channels of a point-to-point connection when a message first needs them (a 4-byte token uses
        one, an 8 MiB activation several), and each of those set-ups stalls the receiving rank for a while; if that
        happens inside a step, the stalled rank's tensor-parallel partner is already spinning in a fused kernel whose
        cross-rank waits are bounded, and the wait can run out. Done here, nothing is in flight yet."""
        self._p2p_warm = True
        if self.device.type != "cuda":
            return
        io = self.stage.io_dtype
        for _ in range(2):
            if self.prev is not None:
                self._recv(self.recv_uids, self.prev, shapes)
            if self.next is not None:
                acts = {u: torch.zeros(shapes[u], dtype=io, device=self.device) for u in self.send_uids}
                for r in self._send(acts, self.send_uids, self.next):
                    r.wait()
            if self.next is not None:
                self._recv(self.send_uids, self.next, shapes)
            if self.prev is not None:
                grads = {u: torch.zeros(shapes[u], dtype=io, device=self.device) for u in self.recv_uids}
                for r in self._send(grads, self.recv_uids, self.prev):
                    r.wait()
        torch.cuda.synchronize()
        dist.barrier()

    # ------------------------------------------------------------------------------- one step
    def train_step(self, data: torch.Tensor, labels: torch.Tensor) -> Optional[torch.Tensor]:
        """Runs the schedule for this rank's batch; the last stage returns the mean loss."""
        st, topo = self.stage, self.topo
        st.set_training(True)
        st.set_step(self.global_step)
        M = self.micro
        if data.shape[0] % M:
            raise ValueError(f"batch of {data.shape[0]} cannot be split into {M} micro-batches")
        mb = data.shape[0] // M
        shapes = self._boundary_shapes((mb,) + tuple(data.shape[1:]))
        if not self._p2p_warm:
            self._warm_p2p(shapes)
        if topo.tp > 1:
            self.stage.tp_context.seq_len = int(data.shape[1])
        d_chunks = data.to(self.device, non_blocking=True).chunk(M) if self.first else None
        l_chunks = labels.to(self.device, non_blocking=True).chunk(M) if self.last else None
        in_uid = self.full.input_nodes[0].uid()
        out_uid = self.full.output_nodes[0].uid()
        pending_sends: List = []
        losses = []
        scale = 1.0 / (M * max(1, int(self.cfg.gradient_accumulation_steps)))
        for op, m in self.schedule(topo.pp_idx, topo.pp, M):
            if op == "F":
                if self.first:
                    x = d_chunks[m]
                    inputs = {in_uid: x.to(st.io_dtype) if x.is_floating_point() else x}
                else:
                    inputs = self._recv(self.recv_uids, self.prev, shapes)
                    self._tp_rendezvous()
                outs = st.forward(inputs, pid=m)
                if self.last:
                    out = outs[out_uid]
                    lab = l_chunks[m]
                    if topo.tp > 1:
                        flat = lab.reshape(-1)
                        rows = flat.numel() // topo.tp
                        lab = flat[topo.tp_idx * rows:(topo.tp_idx + 1) * rows]
                    loss, grad = self.loss.compute(out, lab, scale, True)
                    losses.append(loss)
                    self._last_grad = getattr(self, "_last_grad", {})
                    self._last_grad[m] = {out_uid: grad}
                else:
                    pending_sends += self._send(outs, self.send_uids, self.next)
            else:
                if self.last:
                    grads = self._last_grad.pop(m)
                else:
                    grads = self._recv(self.send_uids, self.next, shapes)
                    self._tp_rendezvous()
                gin = st.backward(grads, pid=m)
                if not self.first:
                    pending_sends += self._send(gin, self.recv_uids, self.prev)
        for r in pending_sends:
            r.wait()
        # gradients of `gradient_accumulation_steps` batches (each already scaled by 1 / that count) add up in the
        # flat gradient buffer before one update - the reference divides the loss gradient by the count and updates
        # every count-th batch (src/nn/train.cpp:284-294, include/distributed/train.hpp:76-91)
        self._accum_count = getattr(self, "_accum_count", 0) + 1
        if self._accum_count >= max(1, int(self.cfg.gradient_accumulation_steps)):
            self._accum_count = 0
            self.optimizer.update()
            st.zero_grads()
            self.scheduler.step()
        self.global_step += 1
        if self.last:
            return torch.stack([l.reshape(()) for l in losses]).mean().reshape(1)
        return None

    def fit(self, train_loader=None, max_steps: Optional[int] = None, log_every: int = 10) -> Dict[str, float]:
        """Step-mode training loop: every rank draws the same batches (same loader seed per data-parallel
        replica), the last stage owns the loss. Returns ``{"steps", "loss"}`` (loss is NaN on other stages)."""
        from ..data.loaders import create_loaders
        cfg = self.cfg
        if train_loader is None:
            train_loader, _ = create_loaders(cfg.dataset_name, cfg.dataset_path, self.local_batch, seed=cfg.seed + self.data_rank,
                                             model_name=cfg.model_name, steps_per_epoch=max(1, cfg.max_steps if cfg.max_steps > 0 else 100))
        steps = max_steps if max_steps is not None else (cfg.max_steps if cfg.max_steps > 0 else None)
        last = float("nan")
        epoch = 0
        while True:
            for data, labels in train_loader:
                loss = self.train_step(data, labels)
                if loss is not None:
                    last = float(loss.item())
                    if log_every and self.global_step % log_every == 0 and self.topo.dp_idx == 0 and self.topo.tp_idx == 0:
                        print(f"step {self.global_step} loss {last:.4f}", flush=True)
                if steps is not None and self.global_step >= steps:
                    return {"steps": self.global_step, "loss": last}
            epoch += 1
            if steps is None and epoch >= cfg.epochs:
                return {"steps": self.global_step, "loss": last}

    def save_stage(self, path: str, gather_tp: bool = True) -> str:
        """Write this stage's graph state to ``<path>.stage<i>`` (the counterpart of the reference's SAVE_TO_FILE
        command: every worker saves its own stage, include/distributed/worker.hpp:279-296). Tensor-parallel
        shards are gathered to full tensors first, so a stage file is the same whatever the tensor-parallel width."""
        g = self.stage
        if g.master_flat is not g.params_flat and isinstance(self.optimizer, FusedDPOptimizer):
            mine = torch.zeros_like(g.trainable_mask)
            for s in self.optimizer.sites:
                mine[s["lo"]:s["hi"]] = True
            g.master_flat.copy_(torch.where(mine, g.master_flat, g.params_flat.float()))
        name = f"{path}.stage{self.topo.pp_idx}"
        if self.topo.tp > 1 and gather_tp:
            from .tp import gather_full_state
            ratios = list(self.cfg.parallel.partition_ratios) or block_aligned_ratios(zoo.create(self.cfg.model_name), self.topo.pp)
            full_stage = partition_graph(zoo.create(self.cfg.model_name), ratios)[self.topo.pp_idx]
            full_stage.compile(device="cpu", seed=self.cfg.seed)
            gather_full_state(g, full_stage, self.topo)
            if self.topo.dp_idx == 0 and self.topo.tp_idx == 0:
                os.makedirs(os.path.dirname(name) or ".", exist_ok=True)
                full_stage.save_state(name)
            return name
        if self.topo.tp > 1:
            name += f".tp{self.topo.tp_idx}"
        if self.topo.dp_idx == 0:
            os.makedirs(os.path.dirname(name) or ".", exist_ok=True)
            g.save_state(name)
        return name

    def close(self):
        if self.heap is not None:
            torch.cuda.synchronize()
            dist.barrier()
            self.heap.close()
            self.heap = None
