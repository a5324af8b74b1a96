"""Tensor parallelism for transformer blocks (Megatron column/row split with sequence parallelism).

Inside a tensor-parallel group of ``tp`` ranks every rank keeps ``1/tp`` of the attention heads and
of the MLP width, and - between those regions - ``1/tp`` of the rows (tokens) of the residual
stream. The two places per block where the row shards have to be combined are fused with the
GEMMs around them by the kernels of csrc/kernels/comm_fused.cu:

* ``gemm_ag``  all-gather of the row shards -> GEMM   (QKV and fc1 forward; out-proj and fc2 dgrad)
* ``gemm_rs``  GEMM -> reduce-scatter of the rows     (out-proj and fc2 forward; QKV and fc1 dgrad)

With ``fused=False`` the same math runs through ``all_gather_into_tensor`` / ``reduce_scatter_tensor``
around the plain GEMM - the NCCL baseline. The head and the embedding are not split by features:
each rank runs them on its own rows with replicated weights, so nothing is computed twice and
their gradients are reduced over all ranks together with the layernorm and bias gradients.
The reference has no tensor parallelism (its only distributed mode is the pipeline).
"""
from __future__ import annotations

import ctypes
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
    lib.tnnb_gemm_comm.argtypes = [i, i, i, i, i, vp, ll, vp, ll, vp, ll, vp, i, i, i, u, vp, vp, vp, vp, vp, vp, vp, vp, vp, ll,
                                   i, vp, vp, vp]
    lib.tnnb_gemm_comm.restype = i
    _DECLARED = True


class CommContext:
    """What the fused GEMMs of one tensor-parallel group share: the heap, the group and its ranks."""

    def __init__(self, topo, heap: Optional[SymmetricHeap], fused: bool, device):
        self.tp, self.idx, self.ranks, self.group = topo.tp, topo.tp_idx, topo.tp_ranks, topo.tp_group
        self.heap, self.fused, self.device = heap, fused and heap is not None, device
        self.lib = _lib.load() if self.fused else None
        # call number of the current pass, read by the kernels from device memory so that a captured
        # CUDA graph sees a new value on every replay
        self.tick = torch.zeros(1, dtype=torch.int32, device=device)
        self.seq_len = 0  # set by the pipeline runtime: stages after the first cannot read it off their input
        if self.fused:
            _declare(self.lib)


class GatherSite:
    """A symmetric ``[M, K]`` buffer whose row block ``idx`` is written locally and whose other row
    blocks are pulled from the peers by ``gemm_ag``. After the call the whole buffer is valid
    locally (it is kept for the weight-gradient GEMM)."""

    def __init__(self, cc: CommContext, M: int, K: int):
        self.cc, self.M, self.K, self.epoch = cc, M, K, 0
        self.rows = M // cc.tp
        if cc.fused:
            self.buf = cc.heap.alloc((M, K), torch.bfloat16)
            self.barrier = cc.heap.alloc((16,), torch.int32).zero_()
            self.src = ptr_array(cc.heap.peer_ptrs(self.buf, cc.ranks))
            self.bar = ptr_array(cc.heap.peer_ptrs(self.barrier, cc.ranks))
            # 128 piece flags per row block, written by the ranks that push their rows into this rank's buffer
            self.piece_flags = cc.heap.alloc(((M // 128 + 1) * 128,), torch.int32).zero_()
            self.chunk_flags = ptr_array(cc.heap.peer_ptrs(self.piece_flags, cc.ranks))
            self.go = torch.zeros(1, dtype=torch.int32, device=cc.device)
        else:
            self.buf = torch.empty(M, K, dtype=torch.bfloat16 if cc.device.type == "cuda" else torch.float32, device=cc.device)

    def mine(self) -> torch.Tensor:
        return self.buf[self.cc.idx * self.rows:(self.cc.idx + 1) * self.rows]

    def gemm(self, w: torch.Tensor, b_t: bool = False, bias=None, gelu_preact: Optional[torch.Tensor] = None,
             dgelu_of: Optional[torch.Tensor] = None) -> torch.Tensor:
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
        pass  # the call number lives in cc.tick (device memory), bumped once per forward and backward pass
        epi, aux = (1, gelu_preact) if gelu_preact is not None else (2, dgelu_of) if dgelu_of is not None else (0, None)
        rc = cc.lib.tnnb_gemm_comm(1, self.M, N, self.K, int(b_t), _lib.ptr(self.buf), self.K, _lib.ptr(w), w.stride(0),
                                   _lib.ptr(out), N, _lib.ptr(bias), cc.tp, cc.idx, self.rows, 0, _lib.ptr(cc.tick), self.bar, self.src,
                                   self.chunk_flags, _lib.ptr(self.go), None, None, None, None, 0, epi,
                                   _lib.ptr(aux), _lib.ptr(_lib.status_word(cc.device)), _lib.stream())
        _lib.check_rc(rc, "tnnb_gemm_comm(all-gather)")
        LAUNCHES["count"] += 1
        return out


class ScatterSite:
    """Inbox and per-tile flags of one GEMM -> reduce-scatter call site (output ``[M/tp, N]``)."""

    def __init__(self, cc: CommContext, M: int, N: int):
        self.cc, self.M, self.N, self.epoch = cc, M, N, 0
        self.rows = M // cc.tp
        if cc.fused:
            tiles = 8 * (self.rows // 128) * ((N + 127) // 128)  # one flag per (tile, 32-row quarter, column half)
            self.inbox = cc.heap.alloc((cc.tp, self.rows, N), torch.bfloat16)
            self.flags = cc.heap.alloc((cc.tp, tiles), torch.int32).zero_()
            ib, fl = cc.heap.peer_ptrs(self.inbox, cc.ranks), cc.heap.peer_ptrs(self.flags, cc.ranks)
            slot_b, slot_f = self.rows * N * 2, tiles * 4
            # on owner o, the slot that belongs to me is slot index cc.idx
            self.inbox_remote = ptr_array([ib[o] + cc.idx * slot_b for o in range(cc.tp)])
            self.flag_remote = ptr_array([fl[o] + cc.idx * slot_f for o in range(cc.tp)])
            self.inbox_local = ptr_array([ib[cc.idx] + s * slot_b for s in range(cc.tp)])
            self.flag_local = ptr_array([fl[cc.idx] + s * slot_f for s in range(cc.tp)])

    def gemm(self, a: torch.Tensor, w: torch.Tensor, b_t: bool = False, bias=None) -> torch.Tensor:
        """``ReduceScatter_rows(a @ op(w).T) + bias`` -> ``[M/tp, N]`` (a holds this rank's K slice)."""
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
        pass  # see GatherSite.gemm
        K = a.shape[1]
        rc = cc.lib.tnnb_gemm_comm(2, self.M, self.N, K, int(b_t), _lib.ptr(a), a.stride(0), _lib.ptr(w), w.stride(0),
                                   _lib.ptr(out), self.N, _lib.ptr(bias), cc.tp, cc.idx, self.rows, 0, _lib.ptr(cc.tick), None, None,
                                   None, None, self.inbox_remote, self.inbox_local, self.flag_remote, self.flag_local,
                                   self.N, 0, None, _lib.ptr(_lib.status_word(cc.device)), _lib.stream())
        _lib.check_rc(rc, "tnnb_gemm_comm(reduce-scatter)")
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
