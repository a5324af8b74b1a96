"""Tensor parallelism for transformer blocks (Megatron column/row split with sequence parallelism).

Inside a tensor-parallel group of ``tp`` ranks every rank keeps ``1/tp`` of the attention heads and
of the MLP width, and - between those regions - ``1/tp`` of the rows (tokens) of the residual
stream. The two places per block where the row shards have to be combined are fused with the
kernels around them (csrc/kernels/tp_flags.cuh describes the protocol):

* all-gather -> GEMM (QKV and fc1 forward; out-proj and fc2 dgrad): the layer-norm kernel that produces a
  rank's rows stores them into every peer's gather buffer as well, and the GEMM (the tensor-parallel variant of
  the CTA-pair tcgen05 kernel) starts with the local rows and polls a counter before it touches a peer's rows;
* GEMM -> reduce-scatter (out-proj and fc2 forward; QKV and fc1 dgrad): the GEMM epilogue stores the partial
  sums of a peer's rows into that peer's inbox, and the layer-norm kernel that consumes the result adds the
  inbox to the local partial sum.

No kernel waits for a peer to arrive at the same call: data only ever flows from kernels that ran earlier.

With ``fused=False`` the same math runs through ``all_gather_into_tensor`` / ``reduce_scatter_tensor``
around the plain GEMM - the NCCL baseline. The head and the embedding are not split by features:
each rank runs them on its own rows with replicated weights, so nothing is computed twice and
their gradients are reduced over all ranks together with the layernorm and bias gradients.
The reference has no tensor parallelism (its only distributed mode is the pipeline).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..nn.graph import Graph, _EdgeSegment, _EmbedSegment, _GPTChain, _Segment, _accum, _flat2d
from ..nn.layers import Dense
from ..ops import _lib, raw
from ..ops.gemm import LAUNCHES, gemm
from .dp import Region
from .symm import SymmetricHeap, ptr_array


# ------------------------------------------------------------------ graph preparation
def shard_graph_for_tp(graph: Graph, topo) -> None:
    """Mark the attention blocks and MLP dense layers of every GPT block as tensor-parallel
    (called before ``compile`` so the flat buffers are sized for the shards)."""
    graph.sort()
    consumers_of = {}
    for i, e in enumerate(graph.edges):
        for p in e.producers:
            consumers_of.setdefault(id(p), []).append(i)
    outs = {id(n) for n in graph.output_nodes}
    i, found = 0, 0
    while i < len(graph.edges):
        if _GPTChain._match_block(graph, i, consumers_of, outs):
            es = graph.edges[i:i + 10]
            attn, fc1, fc2 = es[1].layer, es[5].layer, es[7].layer
            if attn.num_heads % topo.tp or fc1.output_features % (topo.tp * 64):
                raise ValueError("heads and MLP width must be divisible by the tensor-parallel size")
            attn.tp = fc1.tp = fc2.tp = topo.tp
            fc1.tp_mode, fc2.tp_mode = "col", "row"
            found += 1
            i += 10
        else:
            i += 1
    if not found:
        raise ValueError("tensor parallelism needs a model made of transformer blocks")


def tp_regions(graph: Graph, topo) -> List[Region]:
    """Replicated parameters are reduced over every rank of the stage, sharded ones over the
    data-parallel group only."""
    b = graph.shard_boundary
    return [Region(0, b, topo.stage_ranks, topo.stage_group if topo.pp > 1 else None),
            Region(b, graph.total_elems, topo.dp_ranks, topo.dp_group)]


def _reinit_shards(graph: Graph, topo, seed: int = 1234) -> None:
    """Shards of one parameter must differ between tensor-parallel ranks: redraw them from a
    generator keyed by the rank's position in the group (same on all data-parallel replicas)."""
    gen = torch.Generator().manual_seed(seed + 7919 * (topo.tp_idx + 1))
    for l in graph.layers():
        for (o, n, _, _), spec in zip(graph.layer_slices[id(l)], l.param_specs()):
            if spec.sharded and spec.init[0] == "normal":
                graph.master_flat[o:o + n].copy_(torch.empty(n).normal_(0.0, spec.init[1], generator=gen))
    graph.sync_params_from_master()


# --------------------------------------------------------------------- fused GEMM sites
_DECLARED = False


def _declare(lib):
    global _DECLARED
    if _DECLARED:
        return
    vp, ll, i, u = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_uint
    lib.tnnb_gemm_tp.argtypes = [i, vp, vp, vp, i, i, i, i, ll, ll, ll, vp, vp, vp, ll, i, i, i, i, vp, vp, vp, ll, vp, i, vp, vp, i, i, vp, vp]
    lib.tnnb_gemm_tp.restype = i
    lib.tnnb_tp_push.argtypes = [vp, vp, ll, i, i, vp, vp, ll, vp]
    lib.tnnb_tp_push.restype = i
    lib.tnnb_tp_push_bulk.argtypes = [vp, vp, ll, i, i, vp, vp, ll, i, vp, vp]
    lib.tnnb_tp_push_bulk.restype = i
    lib.tnnb_tp_resolve.argtypes = [vp, vp, ll, i, i, vp, vp, vp, u, vp, vp]
    lib.tnnb_tp_resolve.restype = i
    _DECLARED = True


class CommContext:
    """What the fused GEMMs of one tensor-parallel group share: the heap, the group and its ranks."""

    def __init__(self, topo, heap: Optional[SymmetricHeap], fused: bool, device):
        self.tp, self.idx, self.ranks, self.group = topo.tp, topo.tp_idx, topo.tp_ranks, topo.tp_group
        self.heap, self.fused, self.device = heap, fused and heap is not None, device
        self.lib = _lib.load() if self.fused else None
        self.seq_len = 0  # set by the pipeline runtime: stages after the first cannot read it off their input
        # How the rows of a gather site reach the peers (TNNB_TP_PUSH selects one; measured on 2 B200 with the
        # GPT-2 small shapes, 12.6 MB per hand-off, layer norm + all-gather GEMM for QKV; plain kernels: 8 + 29 us):
        #   "ln"    the producing layer-norm kernel stores the rows into the peers' buffers itself (default): the
        #           kernel takes 33 us instead of 8, the GEMM then finds every row in place: 66 us.
        #   "gemm"  one extra warp of the consuming GEMM kernel sends them through the bulk-copy unit (local memory ->
        #           shared memory -> peer) while the tensor cores work on the local tiles: 68 - 72 us (66 us with six
        #           warps of plain stores before) - the copy shares the unit with the GEMM's own operand loads, and
        #           the GEMM's remote tiles cannot finish before the last rows have landed.
        #   "split" the layer-norm kernel sends the first ``ln_share`` of the rows, the GEMM's copy warp the rest: 69 us.
        # A copy-engine form (cudaMemcpyAsync on a side stream followed by a one-warp kernel that updates the counters)
        # was measured at 77 us and then removed: that kernel has to run beside the GEMM of its own GPU, which is
        # waiting for the other rank's counter update - two separate launches that depend on running at the same time.
        self.push_mode = os.environ.get("TNNB_TP_PUSH", "ln")
        self.ln_share = float(os.environ.get("TNNB_TP_LN_SHARE", "0.5"))
        if self.fused:
            _declare(self.lib)

    def new_pass_counter(self) -> torch.Tensor:
        """A device word that counts the passes through one set of sites (bumped once at the start of every
        pass; the kernels read it, so a captured CUDA graph sees a new value on every replay)."""
        return torch.zeros(1, dtype=torch.int32, device=self.device)


# EPI_* bits of csrc/kernels/gemm_tcgen05.h
_EPI_BIAS, _EPI_GELU, _EPI_DGELU = 1, 2, 4


class GatherSite:
    """A symmetric ``[M, K]`` buffer whose row block ``idx`` is produced locally and whose other row blocks are
    PUSHED into it by the ranks that own them (csrc/kernels/tp_flags.cuh), each push followed by an update of the
    receiver's row-block counters. :meth:`gemm` runs the tiles of the local rows first and polls the counters of
    the other row blocks only when it reaches them. By default the kernel that produces this rank's rows (a layer
    norm) also sends them; ``CommContext.push_mode`` lists the alternatives. After the call the whole buffer is
    valid locally (it is kept for the weight-gradient GEMM)."""

    def __init__(self, cc: CommContext, M: int, K: int, pass_ctr: Optional[torch.Tensor] = None):
        self.cc, self.M, self.K = cc, M, K
        self.rows = M // cc.tp
        self.pass_ctr = pass_ctr
        if cc.fused:
            self.buf = cc.heap.alloc((M, K), torch.bfloat16)
            # counters start at zero because the heap does (it is cleared when created and never recycles a block);
            # clearing them here would race with a peer that is already pushing rows
            self.ready = cc.heap.alloc((M // 128 + 1,), torch.int32)
            peers = [r for r in range(cc.tp) if r != cc.idx]
            bufs, rdy = cc.heap.peer_ptrs(self.buf, cc.ranks), cc.heap.peer_ptrs(self.ready, cc.ranks)
            self.n_push = len(peers)
            self.push_row0 = cc.idx * self.rows
            self.push_dst = ptr_array([bufs[r] + self.push_row0 * K * 2 for r in peers])  # peers' copies of my rows
            self.push_base = ptr_array([bufs[r] for r in peers])                         # peers' whole buffers
            self.push_ready = ptr_array([rdy[r] for r in peers])
            # rows [0, ln_rows) of this rank's shard travel with the producing kernel, the rest with the GEMM
            blocks = self.rows // 128
            share = {"ln": 1.0, "gemm": 0.0}.get(cc.push_mode, cc.ln_share)
            self.ln_blocks = min(blocks, max(0, int(round(blocks * share))))
            self.ln_rows = self.ln_blocks * 128
        else:
            self.buf = torch.empty(M, K, dtype=torch.bfloat16 if cc.device.type == "cuda" else torch.float32, device=cc.device)

    def mine(self) -> torch.Tensor:
        return self.buf[self.cc.idx * self.rows:(self.cc.idx + 1) * self.rows]

    def push_args(self):
        """Arguments that make a layer-norm kernel writing :meth:`mine` deliver the rows to the peers as well
        (``None`` on the NCCL path and when the consuming GEMM sends all of them)."""
        return self if (self.cc.fused and self.cc.push_mode in ("ln", "split") and self.ln_rows > 0) else None

    def push(self, src: Optional[torch.Tensor] = None, bulk_ctas: Optional[int] = None) -> None:
        """Stand-alone push: copy ``src`` (default: the rows already in :meth:`mine`) to the peers and publish.
        ``bulk_ctas``: use the bulk-copy kernel with that many blocks (0 = its default) instead of SM stores."""
        cc = self.cc
        if not cc.fused:
            if src is not None:
                self.mine().copy_(src)
            return
        mine = self.mine()
        if cc.push_mode not in ("ln", "split") or self.ln_rows == 0:
            if src is not None:
                mine.copy_(src)
            return
        if src is not None and self.ln_rows < self.rows:
            mine[self.ln_rows:].copy_(src[self.ln_rows:])   # these rows are sent by the GEMM
        s = mine if src is None else src.contiguous()
        if bulk_ctas is not None:
            rc = cc.lib.tnnb_tp_push_bulk(_lib.ptr(s), _lib.ptr(mine) if src is not None else None, self.ln_rows, self.K,
                                          self.n_push, self.push_dst, self.push_ready, self.push_row0, int(bulk_ctas),
                                          _lib.ptr(_lib.status_word(mine.device)), _lib.stream())
            _lib.check_rc(rc, "tnnb_tp_push_bulk")
            LAUNCHES["count"] += 1
            return
        rc = cc.lib.tnnb_tp_push(_lib.ptr(s), _lib.ptr(mine) if src is not None else None, self.ln_rows, self.K, self.n_push,
                                 self.push_dst, self.push_ready, self.push_row0, _lib.stream())
        _lib.check_rc(rc, "tnnb_tp_push")
        LAUNCHES["count"] += 1

    def gemm(self, w: torch.Tensor, b_t: bool = False, bias=None, gelu_preact: Optional[torch.Tensor] = None,
             dgelu_of: Optional[torch.Tensor] = None, force_bn: int = 0) -> torch.Tensor:
        """``epilogue(AllGather(rows) @ op(w).T)`` -> ``[M, N]``."""
        cc = self.cc
        N = w.shape[1] if b_t else w.shape[0]
        if not cc.fused:
            if cc.tp > 1:
                dist.all_gather_into_tensor(self.buf, self.mine().clone(), group=cc.group)
            if gelu_preact is not None:
                return gemm(self.buf, w, b_t=b_t, bias=bias, gelu=True, save_preact=gelu_preact)
            return gemm(self.buf, w, b_t=b_t, bias=bias, dgelu_of=dgelu_of)
        out = torch.empty(self.M, N, dtype=torch.bfloat16, device=cc.device)
        flags = (_EPI_BIAS if bias is not None else 0) | (_EPI_GELU if gelu_preact is not None else 0) | \
                (_EPI_DGELU if dgelu_of is not None else 0)
        aux = gelu_preact if gelu_preact is not None else dgelu_of
        rc = cc.lib.tnnb_gemm_tp(1, _lib.ptr(self.buf), _lib.ptr(w), _lib.ptr(out), self.M, N, self.K, int(b_t), self.K,
                                 w.stride(0), N, _lib.ptr(bias), _lib.ptr(dgelu_of), _lib.ptr(gelu_preact),
                                 aux.stride(0) if aux is not None else 0, flags, cc.tp, cc.idx, self.rows,
                                 _lib.ptr(self.pass_ctr), _lib.ptr(self.ready), None, 0, None,
                                 self.n_push if (cc.push_mode in ("gemm", "split") and self.ln_blocks < self.rows // 128) else 0,
                                 self.push_base, self.push_ready, self.ln_blocks, force_bn,
                                 _lib.ptr(_lib.status_word(cc.device)), _lib.stream())
        _lib.check_rc(rc, "tnnb_gemm_tp(all-gather)")
        LAUNCHES["count"] += 1
        return out


class ScatterSite:
    """Inbox and arrival counters of one GEMM -> reduce-scatter call site (output ``[M/tp, N]``).

    :meth:`gemm` computes this rank's partial sums of ALL rows: the rows it owns stay local (bias added), the
    others go straight from the epilogue into their owner's inbox. The sum over ranks is formed by whoever reads
    the result: a layer-norm kernel given :meth:`pull_args`, or :meth:`resolve`."""

    def __init__(self, cc: CommContext, M: int, N: int, pass_ctr: Optional[torch.Tensor] = None):
        self.cc, self.M, self.N = cc, M, N
        self.rows = M // cc.tp
        self.pass_ctr = pass_ctr
        if cc.fused:
            self.inbox = cc.heap.alloc((cc.tp, self.rows, N), torch.bfloat16)   # slot s: partial sums from rank s
            self.arrived = cc.heap.alloc((self.rows // 128 + 1,), torch.int32)   # zero from the heap, see GatherSite
            ib, ar = cc.heap.peer_ptrs(self.inbox, cc.ranks), cc.heap.peer_ptrs(self.arrived, cc.ranks)
            slot = self.rows * N * 2
            self._remote_out = [ib[o] + cc.idx * slot for o in range(cc.tp)]  # my slot on owner o
            self.arrived_ptrs = ptr_array(ar)
            peers = [r for r in range(cc.tp) if r != cc.idx]
            self.n_pull = len(peers)
            self.pull_src = ptr_array([self.inbox[r].data_ptr() for r in peers])
            self.units = 4 * ((N + 31) // 32) * self.n_pull   # what one pass adds to each 128-row counter

    def gemm(self, a: torch.Tensor, w: torch.Tensor, b_t: bool = False, bias=None, force_bn: int = 0) -> torch.Tensor:
        """This rank's rows of ``a @ op(w).T`` (+ bias) -> ``[M/tp, N]``: the complete reduce-scatter result on the
        NCCL path, the local partial sum on the fused path (a holds this rank's K slice)."""
        cc = self.cc
        if not cc.fused:
            full = gemm(a, w, b_t=b_t)
            if cc.tp == 1:
                out = full
            else:
                if full.is_cuda:
                    out = torch.empty(self.rows, self.N, dtype=full.dtype, device=full.device)
                    dist.reduce_scatter_tensor(out, full, group=cc.group)
                else:  # gloo has no reduce-scatter: all-reduce and keep this rank's rows
                    dist.all_reduce(full, group=cc.group)
                    out = full[cc.idx * self.rows:(cc.idx + 1) * self.rows].clone()
            if bias is not None:
                out = (out.float() + bias.float()).to(out.dtype)
            return out
        out = torch.empty(self.rows, self.N, dtype=torch.bfloat16, device=cc.device)
        K = a.shape[1]
        outs = list(self._remote_out)
        outs[cc.idx] = out.data_ptr()
        rc = cc.lib.tnnb_gemm_tp(2, _lib.ptr(a), _lib.ptr(w), None, self.M, self.N, K, int(b_t), a.stride(0), w.stride(0), 0,
                                 _lib.ptr(bias), None, None, 0, _EPI_BIAS if bias is not None else 0, cc.tp, cc.idx, self.rows,
                                 _lib.ptr(self.pass_ctr), None, ptr_array(outs), self.N, self.arrived_ptrs, 0, None, None, 0, force_bn,
                                 _lib.ptr(_lib.status_word(cc.device)), _lib.stream())
        _lib.check_rc(rc, "tnnb_gemm_tp(reduce-scatter)")
        LAUNCHES["count"] += 1
        return out

    def pull_args(self):
        """Arguments that make a layer-norm kernel add the peers' partial sums to the local one (``None`` on the
        NCCL path, where :meth:`gemm` already returned the sum)."""
        return self if self.cc.fused else None

    def resolve(self, partial: torch.Tensor) -> torch.Tensor:
        """Stand-alone form of the sum: ``partial`` + the peers' partial sums."""
        cc = self.cc
        if not cc.fused:
            return partial
        out = torch.empty_like(partial)
        rc = cc.lib.tnnb_tp_resolve(_lib.ptr(partial), _lib.ptr(out), self.rows, self.N, self.n_pull, self.pull_src,
                                    _lib.ptr(self.arrived), _lib.ptr(self.pass_ctr), self.units,
                                    _lib.ptr(_lib.status_word(cc.device)), _lib.stream())
        _lib.check_rc(rc, "tnnb_tp_resolve")
        LAUNCHES["count"] += 1
        return out


# ------------------------------------------------------------- full model <-> shards
def _shard_of(layer, spec_name: str, full: torch.Tensor, tp: int, t: int) -> torch.Tensor:
    """The slice of a full (unsharded) parameter that tensor-parallel rank ``t`` holds."""
    from ..nn.blocks import FlashAttentionBlock
    if isinstance(layer, FlashAttentionBlock):
        E = layer.embed_dim
        Es = E // tp
        if spec_name in ("qkv_weight", "qkv_bias"):
            parts = [full[k * E + t * Es:k * E + (t + 1) * Es] for k in range(3)]
            return torch.cat(parts, 0)
        if spec_name == "out_weight":
            return full[:, t * Es:(t + 1) * Es]
        return full
    mode = getattr(layer, "tp_mode", None)
    if mode == "col":
        n = full.shape[0] // tp
        return full[t * n:(t + 1) * n]
    if mode == "row" and spec_name == "weight":
        n = full.shape[1] // tp
        return full[:, t * n:(t + 1) * n]
    return full


def _unshard(layer, spec_name: str, parts: List[torch.Tensor], tp: int) -> torch.Tensor:
    """Inverse of :func:`_shard_of`: the full parameter from the ``tp`` shards (in rank order)."""
    from ..nn.blocks import FlashAttentionBlock
    if isinstance(layer, FlashAttentionBlock):
        if spec_name in ("qkv_weight", "qkv_bias"):
            Es = parts[0].shape[0] // 3
            return torch.cat([p[k * Es:(k + 1) * Es] for k in range(3) for p in parts], 0)  # q of every rank, then k, then v
        if spec_name == "out_weight":
            return torch.cat(parts, 1)
        return parts[0]
    mode = getattr(layer, "tp_mode", None)
    if mode == "col":
        return torch.cat(parts, 0)
    if mode == "row" and spec_name == "weight":
        return torch.cat(parts, 1)
    return parts[0]


def gather_full_state(tp_graph: Graph, full_graph: Graph, topo, group=None) -> None:
    """Fill ``full_graph`` (the same model without tensor parallelism, same layer names) from the shards the ranks
    of a tensor-parallel group hold - what a checkpoint that other layouts can read needs. Collective over the
    group; every rank ends up with the full parameters in ``full_graph``."""
    group = group if group is not None else topo.tp_group
    full = {l.name: l for l in full_graph.layers()}
    for l in tp_graph.layers():
        dst = full[l.name]
        for (o, n, shape, _), spec, (fo, fn, fshape, _) in zip(tp_graph.layer_slices[id(l)], l.param_specs(),
                                                              full_graph.layer_slices[id(dst)]):
            mine = tp_graph.master_flat[o:o + n].view(shape).contiguous()
            if spec.sharded and topo.tp > 1:
                parts = [torch.empty_like(mine) for _ in range(topo.tp)]
                dist.all_gather(parts, mine, group=group)
                whole = _unshard(l, spec.name, parts, topo.tp)
            else:
                whole = mine
            if tuple(whole.shape) != tuple(fshape):
                raise ValueError(f"{l.name}.{spec.name}: gathered shape {tuple(whole.shape)} != {tuple(fshape)}")
            full_graph.master_flat[fo:fo + fn].copy_(whole.reshape(-1).to(full_graph.master_flat.device))
    full_graph.sync_params_from_master()


def copy_full_to_shards(tp_graph: Graph, full_graph: Graph, topo) -> None:
    """Initialise a tensor-parallel graph from an unsharded one with the same layer names (used to
    load a full checkpoint into a tensor-parallel job and by the equivalence tests)."""
    full = {l.name: l for l in full_graph.layers()}
    for l in tp_graph.layers():
        src = full[l.name]
        for (o, n, shape, _), spec, (fo, fn, fshape, _) in zip(tp_graph.layer_slices[id(l)], l.param_specs(),
                                                              full_graph.layer_slices[id(src)]):
            whole = full_graph.master_flat[fo:fo + fn].view(fshape)
            part = _shard_of(l, spec.name, whole, topo.tp, topo.tp_idx) if spec.sharded else whole
            tp_graph.master_flat[o:o + n].copy_(part.reshape(-1).to(tp_graph.master_flat.device))
    tp_graph.sync_params_from_master()
