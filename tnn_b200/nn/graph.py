"""Graph builder and executor.

A :class:`Graph` is a DAG of edges ``(layer, producer nodes, consumer nodes)`` over
nodes identified by a string uid, built with the same surface as the reference
(include/nn/graph.hpp, examples/graph_api_v2_test.cpp:13-80)::

    g = Graph()
    x = g.input("input")
    h = Dense(784, 128)(x)
    y = ReLU()(h) + h            # Node operators insert add/sub/mul/div layers
    y.set_uid("output"); g.set_output(y); g.compile(device="cuda")

``compile`` sorts the edges (Kahn, FIFO - src/nn/graph.cpp:111-189), lays every
parameter into ONE flat buffer and every gradient into ONE flat fp32 buffer
(256-byte aligned per tensor, include/nn/graph_context.hpp:26-83) - which is what
the fused gradient reduce-scatter + optimizer kernels consume - and, for bf16
training, keeps an fp32 master copy beside it.

``forward(inputs, pid)`` / ``backward(grads, pid)`` keep all saved state keyed by the
micro-batch id, so a pipeline stage can have several micro-batches in flight
(include/nn/node.hpp:74-75). Runs of edges that form a GPT block
(src/nn/example_graphs.cpp:198-215) or the token/position embedding are executed by
fused segments (residual add + dropout + layernorm in one kernel, bias/GELU in GEMM
epilogues); every other edge runs layer by layer.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import raw
from ..ops.gemm import gemm
from .blocks import FlashAttentionBlock, layer_from_config
from .layers import (Add, BatchNorm, Conv2D, Dense, Div, Dropout, Embedding, GELU, Layer, LayerNorm, Mul,
                     PositionalEmbedding, Sub, _flat2d)

ALIGN_BYTES = 256


class Node:
    """A value in the graph. Supports ``+ - * /`` with other nodes."""

    def __init__(self, graph: "Graph", uid: str):
        self.graph, self._uid = graph, uid

    def uid(self) -> str:
        return self._uid

    def set_uid(self, uid: str):
        self.graph._rename(self, uid)

    def _bin(self, other: "Node", cls):
        return cls()(self, other)

    def __add__(self, o):
        return self._bin(o, Add)

    def __sub__(self, o):
        return self._bin(o, Sub)

    def __mul__(self, o):
        return self._bin(o, Mul)

    def __truediv__(self, o):
        return self._bin(o, Div)

    def __repr__(self):
        return f"Node({self._uid})"


class Edge:
    __slots__ = ("layer", "producers", "consumers")

    def __init__(self, layer: Layer, producers: Sequence[Node], consumers: Sequence[Node]):
        self.layer, self.producers, self.consumers = layer, list(producers), list(consumers)


def _layer_call(self: Layer, *nodes: Node) -> Node:
    """``layer(node, ...)`` adds an edge to the nodes' graph and returns the output node."""
    g = nodes[0].graph
    out = g.make_node()
    g.add_edge(self, list(nodes), [out])
    return out


Layer.__call__ = _layer_call


class AllocationTracker:
    """Per-segment readings of the device allocator (see ``Graph.track_memory``). ``rows`` holds
    ``(segment, pass, bytes_live_after - bytes_live_before, peak_above_start)``; on the CPU, where there is no
    allocator to ask, both figures are zero."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.rows: List[Tuple[str, str, int, int]] = []
        self._start = 0

    def enter(self) -> None:
        if self.cuda:
            torch.cuda.reset_peak_memory_stats(self.device)
            self._start = torch.cuda.memory_allocated(self.device)

    def leave(self, name: str, which: str) -> None:
        if self.cuda:
            now = torch.cuda.memory_allocated(self.device)
            peak = torch.cuda.max_memory_allocated(self.device)
            self.rows.append((name, which, now - self._start, max(0, peak - self._start)))
        else:
            self.rows.append((name, which, 0, 0))

    def peak_per_edge(self) -> Dict[str, Dict[str, int]]:
        """``{segment: {"forward_kept", "forward_peak", "backward_freed", "backward_peak"}}`` over everything seen."""
        out: Dict[str, Dict[str, int]] = {}
        for name, which, delta, peak in self.rows:
            d = out.setdefault(name, {"forward_kept": 0, "forward_peak": 0, "backward_freed": 0, "backward_peak": 0})
            if which == "forward":
                d["forward_kept"] = max(d["forward_kept"], delta)
                d["forward_peak"] = max(d["forward_peak"], peak)
            else:
                d["backward_freed"] = max(d["backward_freed"], -delta)
                d["backward_peak"] = max(d["backward_peak"], peak)
        return out

    def format(self) -> str:
        rows = self.peak_per_edge()
        w = max([len(n) for n in rows] + [5])
        mib = 2 ** 20
        lines = [f"{'edge':<{w}}  {'fwd kept MiB':>12}  {'fwd peak MiB':>12}  {'bwd freed MiB':>13}  {'bwd peak MiB':>12}"]
        lines += [f"{n:<{w}}  {d['forward_kept'] / mib:>12.2f}  {d['forward_peak'] / mib:>12.2f}  {d['backward_freed'] / mib:>13.2f}  "
                  f"{d['backward_peak'] / mib:>12.2f}" for n, d in rows.items()]
        return "\n".join(lines)


class Graph:
    def __init__(self):
        self.nodes: List[Node] = []
        self.edges: List[Edge] = []
        self.input_nodes: List[Node] = []
        self.output_nodes: List[Node] = []
        self._uids = set()
        self._counter = 0
        self.compiled = False
        self.device = torch.device("cpu")
        self.param_dtype = torch.float32
        self.io_dtype = torch.float32
        self.params_flat: Optional[torch.Tensor] = None   # compute copy (bf16 or fp32)
        self.master_flat: Optional[torch.Tensor] = None   # fp32 master (aliases params_flat for fp32)
        self.alloc_hook: Optional["AllocationTracker"] = None  # per-segment device-memory accounting (track_memory)
        self.grads_flat: Optional[torch.Tensor] = None    # fp32
        self.trainable_mask: Optional[torch.Tensor] = None
        self.layer_slices: Dict[int, List[Tuple[int, int, Tuple[int, ...], bool]]] = {}
        self.training = True
        self.profiler = None  # utils.profiling.LayerProfiler, set by the trainer when profiler_type != NONE
        # Called during backward() as grad_hook(floor): every gradient at flat offset >= floor is final for this pass.
        # The data-parallel optimizer uses it to start reducing finished buckets while backward is still running.
        self.grad_hook = None
        self.step = 0
        self.input_requires_grad = False
        self._ctx: Dict[int, dict] = {}
        self.segments: List["_Segment"] = []
        self.fuse = True

    # ------------------------------------------------------------------ construction
    def _gen_uid(self) -> str:
        while True:
            uid = f"node_{self._counter}"
            self._counter += 1
            if uid not in self._uids:
                self._uids.add(uid)
                return uid

    def make_node(self, uid: Optional[str] = None) -> Node:
        if uid is None:
            uid = self._gen_uid()
        else:
            if uid in self._uids:
                raise ValueError(f"duplicate node uid {uid!r}")
            self._uids.add(uid)
        n = Node(self, uid)
        self.nodes.append(n)
        return n

    def _rename(self, node: Node, uid: str):
        if uid != node._uid and uid in self._uids:
            raise ValueError(f"duplicate node uid {uid!r}")
        self._uids.discard(node._uid)
        self._uids.add(uid)
        node._uid = uid

    def input(self, uid: str = "input") -> Node:
        n = self.make_node(uid)
        self.input_nodes.append(n)
        return n

    def set_input(self, node: Node):
        if node not in self.input_nodes:
            self.input_nodes.append(node)

    def set_output(self, node: Node):
        if node not in self.output_nodes:
            self.output_nodes.append(node)

    def add_edge(self, layer: Layer, producers: Sequence[Node], consumers: Sequence[Node]):
        self.edges.append(Edge(layer, producers, consumers))
        self.compiled = False

    def node_by_uid(self, uid: str) -> Node:
        for n in self.nodes:
            if n._uid == uid:
                return n
        raise KeyError(uid)

    def layers(self) -> List[Layer]:
        """Unique layers in first-use order over the (sorted) edges."""
        seen, out = set(), []
        for e in self.edges:
            if id(e.layer) not in seen:
                seen.add(id(e.layer))
                out.append(e.layer)
        return out

    # ---------------------------------------------------------------------- sorting
    def ir(self) -> dict:
        """Index-based description of the graph for the C++ IR (sort / partition / TNNG)."""
        idx = {id(n): i for i, n in enumerate(self.nodes)}
        lidx: Dict[int, int] = {}
        for e in self.edges:
            lidx.setdefault(id(e.layer), len(lidx))
        return {"nodes": [n._uid for n in self.nodes],
                "inputs": [idx[id(n)] for n in self.input_nodes],
                "outputs": [idx[id(n)] for n in self.output_nodes],
                "edges": [(lidx[id(e.layer)], [idx[id(p)] for p in e.producers], [idx[id(c)] for c in e.consumers])
                          for e in self.edges]}

    def sort(self):
        """FIFO Kahn order of the edges and the matching node order, computed by the C++ graph IR."""
        from ..host import H
        out = H.topo_sort(self.ir())
        self.edges = [self.edges[i] for i in out["edge_perm"]]
        self.nodes = [self.nodes[i] for i in out["node_perm"]]

    # -------------------------------------------------------------------- compiling
    def compile(self, device="cpu", param_dtype: Optional[torch.dtype] = None, io_dtype: Optional[torch.dtype] = None,
                seed: Optional[int] = 0, init: bool = True, fuse: bool = True, alloc=None):
        """Sort, allocate the flat parameter / gradient buffers, bind and initialise every layer."""
        self.device = torch.device(device)
        on_gpu = self.device.type == "cuda"
        # The sm_100a kernels compute in bf16 with fp32 accumulation; fp32 is kept for the master
        # weights, gradients and optimizer state. On CPU everything is fp32 unless asked otherwise.
        self.param_dtype = param_dtype or (torch.bfloat16 if on_gpu else torch.float32)
        self.io_dtype = io_dtype or (torch.bfloat16 if on_gpu else torch.float32)
        if on_gpu and (self.param_dtype != torch.bfloat16 or self.io_dtype != torch.bfloat16):
            raise ValueError("CUDA graphs run in bf16 (fp32 master weights and gradients are kept automatically)")
        self.fuse = fuse
        self.sort()
        layers = self.layers()
        elem = torch.tensor([], dtype=self.param_dtype).element_size()
        align = max(1, ALIGN_BYTES // min(elem, 4))  # in elements; same element offsets in all three buffers
        off = 0
        self.layer_slices = {id(l): [None] * len(l.param_specs()) for l in layers}
        self.shard_boundary = None
        # Two passes: parameters replicated on every tensor-parallel rank first, then the ones a
        # tensor-parallel layer marks as sharded, so that each kind forms one contiguous range.
        for want_sharded in (False, True):
            if want_sharded:
                off = (off + 1023) // 1024 * 1024
                self.shard_boundary = off
            for l in layers:
                for k, spec in enumerate(l.param_specs()):
                    if bool(getattr(spec, "sharded", False)) != want_sharded:
                        continue
                    n = 1
                    for d in spec.shape:
                        n *= d
                    self.layer_slices[id(l)][k] = (off, n, spec.shape, spec.trainable)
                    off = (off + n + align - 1) // align * align
        total = max(off, align)
        # ``alloc(numel, dtype)`` lets the parameter and gradient slabs live in a symmetric heap so that
        # peer GPUs can read gradients and write parameters directly (tnn_b200.parallel).
        total = (total + 1023) // 1024 * 1024
        self.total_elems = total
        if alloc is not None:
            self.params_flat = alloc(total, self.param_dtype).zero_()
            self.grads_flat = alloc(total, torch.float32).zero_()
        else:
            self.params_flat = torch.zeros(total, dtype=self.param_dtype, device=self.device)
            self.grads_flat = torch.zeros(total, dtype=torch.float32, device=self.device)
        self.master_flat = self.params_flat if self.param_dtype == torch.float32 else torch.zeros(
            total, dtype=torch.float32, device=self.device)
        self.trainable_mask = torch.zeros(total, dtype=torch.bool, device=self.device)
        gen = None
        if seed is not None:
            gen = torch.Generator(device="cpu")
            gen.manual_seed(seed)
        for l in layers:
            ps, gs = [], []
            for (o, n, shape, trainable), spec in zip(self.layer_slices[id(l)], l.param_specs()):
                ps.append(self.params_flat[o:o + n].view(shape))
                gs.append(self.grads_flat[o:o + n].view(shape) if trainable else None)
                if trainable:
                    self.trainable_mask[o:o + n] = True
                if init:
                    kind, val = spec.init
                    m = self.master_flat[o:o + n]
                    if kind == "normal":
                        m.copy_(torch.empty(n).normal_(0.0, val, generator=gen))
                    elif kind == "ones":
                        m.fill_(1.0)
                    else:
                        m.zero_()
            l.bind(ps, gs)
            # fp32 views of the same parameters (batch-norm running statistics are kept in these)
            l.bind_masters([self.master_flat[o:o + n].view(shape) for (o, n, shape, _) in self.layer_slices[id(l)]])
            l.set_io_dtype(self.io_dtype)
        self.sync_params_from_master()
        self._build_segments()
        self.compiled = True
        return self

    def sync_params_from_master(self):
        if self.master_flat is not self.params_flat:
            self.params_flat.copy_(self.master_flat)

    def sync_master_from_params(self):
        if self.master_flat is not self.params_flat:
            self.master_flat.copy_(self.params_flat)

    def num_parameters(self) -> int:
        return int(sum(n for sl in self.layer_slices.values() for (_, n, _, _) in sl))

    def parameters(self) -> List[torch.Tensor]:
        return [p for l in self.layers() for p in l.params]

    def gradients(self) -> List[Optional[torch.Tensor]]:
        return [g for l in self.layers() for g in l.grads]

    def zero_grads(self):
        """One memset over the contiguous gradient slab (include/nn/graph_context.hpp:94)."""
        self.grads_flat.zero_()

    def set_training(self, flag: bool = True):
        self.training = flag
        for l in self.layers():
            l.set_training(flag)

    def set_recompute_qkv(self, flag: bool = True) -> int:
        """Switch every attention block between keeping its packed q/k/v projection for the backward pass and
        computing it again there (less saved activation memory, one more GEMM per block). Returns the number of
        blocks switched."""
        n = 0
        for l in self.layers():
            if hasattr(l, "recompute_qkv"):
                l.recompute_qkv = bool(flag)
                n += 1
        return n

    def train(self):
        self.set_training(True)

    def eval(self):
        self.set_training(False)

    def set_step(self, step: int):
        self.step = int(step)

    # -------------------------------------------------------------------- segments
    def _build_segments(self):
        consumers_of: Dict[int, List[int]] = {}
        for i, e in enumerate(self.edges):
            for p in e.producers:
                consumers_of.setdefault(id(p), []).append(i)
        outs = {id(n) for n in self.output_nodes}
        segs: List[_Segment] = []
        i = 0
        n_e = len(self.edges)
        while i < n_e:
            seg = None
            if self.fuse:
                seg = (_GPTChain.match(self, i, consumers_of, outs) or _EmbedSegment.match(self, i, consumers_of, outs)
                       or _BnAddSegment.match(self, i, consumers_of, outs))
            if seg is None:
                seg = _EdgeSegment(self, i)
            segs.append(seg)
            i = seg.end
        self.segments = segs

    def _layer_floor(self, layer: Layer) -> Optional[int]:
        offs = [sl[0] for sl in self.layer_slices.get(id(layer), []) if sl]
        return min(offs) if offs else None

    def segment_floors(self) -> List[Optional[int]]:
        """Per executor segment, the lowest flat-buffer offset of its layers' parameters (None: no parameters).
        Parameters are laid out in first-use order over the sorted edges, so once the backward of segment ``k`` has
        run, every gradient at an offset >= ``segment_floors()[k]`` is final - provided no layer is shared between
        segments (``grad_hook_usable``)."""
        out = []
        for seg in self.segments:
            fl = [self._layer_floor(self.edges[i].layer) for i in range(seg.start, seg.end)]
            fl = [f for f in fl if f is not None]
            out.append(min(fl) if fl else None)
        return out

    def grad_hook_usable(self) -> bool:
        """True when offsets grow with the segment index and every layer belongs to one edge only."""
        seen = set()
        for e in self.edges:
            if id(e.layer) in seen:
                return False
            seen.add(id(e.layer))
        last = -1
        for f in self.segment_floors():
            if f is None:
                continue
            if f < last:
                return False
            last = f
        return True

    def grad_ready_points(self) -> List[int]:
        """The floors ``grad_hook`` will be called with during one backward pass, in firing order (descending)."""
        pts: List[int] = []
        floors = self.segment_floors()
        for k in reversed(range(len(self.segments))):
            pts += self.segments[k].inner_floors(self)
            if floors[k] is not None:
                pts.append(floors[k])
        return pts

    # -------------------------------------------------------------------- execution
    def _pid_ctx(self, pid: int) -> dict:
        return self._ctx.setdefault(pid, {"values": {}, "seg": {}})

    def forward(self, inputs: Dict[str, torch.Tensor], pid: int = 0) -> Dict[str, torch.Tensor]:
        if not self.compiled:
            raise RuntimeError("Graph.compile() must run before forward()")
        st = self._ctx[pid] = {"values": {}, "seg": {}}
        vals: Dict[int, torch.Tensor] = st["values"]
        by_uid = {n._uid: n for n in self.nodes}
        for uid, t in inputs.items():
            if uid not in by_uid:
                raise KeyError(f"Input UID not found in graph: {uid}")
            if t.device != self.device:
                t = t.to(self.device, non_blocking=True)
            if t.is_floating_point() and t.dtype != self.io_dtype:
                t = t.to(self.io_dtype)
            vals[id(by_uid[uid])] = t
        prof = self.profiler
        mem = self.alloc_hook
        for k, seg in enumerate(self.segments):
            sctx = st["seg"][k] = {"_step": self.step, "_pid": pid}
            if mem is not None:
                mem.enter()
            if prof is None:
                seg.forward(vals, sctx)
            else:
                with prof.span(self.segment_name(k), "forward"):
                    seg.forward(vals, sctx)
            if mem is not None:
                mem.leave(self.segment_name(k), "forward")
        out = {n._uid: vals[id(n)] for n in self.output_nodes}
        if not self.training:
            self._ctx.pop(pid, None)
        else:
            st["values"] = {}  # saved tensors live in the segment contexts
        return out

    def backward(self, grads: Dict[str, torch.Tensor], pid: int = 0) -> Dict[str, torch.Tensor]:
        st = self._ctx.pop(pid, None)
        if st is None:
            raise RuntimeError(f"backward() without a matching forward() for micro-batch {pid}")
        by_uid = {n._uid: n for n in self.nodes}
        gvals: Dict[int, torch.Tensor] = {}
        for uid, g in grads.items():
            gvals[id(by_uid[uid])] = g.to(self.io_dtype) if g.dtype != self.io_dtype else g
        need_in = {id(n) for n in self.input_nodes} if not self.input_requires_grad else set()
        prof = self.profiler
        hook = self.grad_hook
        floors = self.segment_floors() if hook is not None else None
        mem = self.alloc_hook
        for k in reversed(range(len(self.segments))):
            if mem is not None:
                mem.enter()
            if prof is None:
                self.segments[k].backward(gvals, st["seg"][k], need_in)
            else:
                with prof.span(self.segment_name(k), "backward"):
                    self.segments[k].backward(gvals, st["seg"][k], need_in)
            st["seg"][k] = None  # what the segment saved for this pass is dead now
            if mem is not None:
                mem.leave(self.segment_name(k), "backward")
            if hook is not None and floors[k] is not None:
                hook(floors[k])
        return {n._uid: gvals[id(n)] for n in self.input_nodes if id(n) in gvals and gvals[id(n)] is not None}

    def segment_name(self, k: int) -> str:
        """Name of executor segment ``k``: the layer's name, or first..last layer of a fused chain."""
        seg = self.segments[k]
        names = [self.edges[i].layer.name for i in range(seg.start, seg.end)]
        return names[0] if len(names) == 1 else f"{names[0]}..{names[-1]}[{type(seg).__name__.lstrip('_')}]"

    def track_memory(self, on: bool = True) -> Optional["AllocationTracker"]:
        """Install (or remove) the allocation hook: while it is installed every executor segment's forward and
        backward pass is bracketed by readings of the device allocator, which gives, per edge of the graph, how
        much memory the pass left allocated and how far above its starting level it peaked (the reference gathers
        the same figures through its allocator's hooks in ``Graph::forward``, src/nn/graph.cpp:206-233). Not for a
        captured step: the readings synchronise nothing but they are host calls."""
        self.alloc_hook = AllocationTracker(self.device) if on else None
        return self.alloc_hook

    def memory_report(self, pid: int = 0) -> List[Tuple[str, int, int]]:
        """``(segment name, parameter bytes, bytes saved for backward)`` per executor segment.

        Call between a training ``forward`` and its ``backward``: the saved bytes are the tensors that the
        segment keeps for its backward pass for micro-batch ``pid``; a storage shared by several segments
        is counted once, for the first that holds it. This is what the trainer option
        ``print_layer_memory_usage`` prints (the reference parses that option, src/nn/train.cpp:159, but
        prints nothing for it)."""
        st = self._ctx.get(pid, {"seg": {}})
        seen: set = set()

        def walk(o) -> int:
            if isinstance(o, torch.Tensor):
                key = o.untyped_storage().data_ptr()
                if key in seen or key == 0:
                    return 0
                seen.add(key)
                return o.untyped_storage().nbytes()
            if isinstance(o, dict):
                return sum(walk(v) for v in o.values())
            if isinstance(o, (list, tuple)):
                return sum(walk(v) for v in o)
            return 0

        rows = []
        for k, seg in enumerate(self.segments):
            pbytes, counted = 0, set()
            for i in range(seg.start, seg.end):
                lay = self.edges[i].layer
                if id(lay) not in counted:  # a layer used by several edges owns its parameters once
                    counted.add(id(lay))
                    pbytes += sum(sl[1] for sl in self.layer_slices.get(id(lay), []) if sl) * self.params_flat.element_size()
            rows.append((self.segment_name(k), pbytes, walk(st["seg"].get(k, {}))))
        return rows

    def format_memory_report(self, pid: int = 0) -> str:
        rows = self.memory_report(pid)
        w = max([len(r[0]) for r in rows] + [5])
        lines = [f"{'layer':<{w}}  {'params MiB':>11}  {'saved MiB':>10}"]
        lines += [f"{n:<{w}}  {p / 2**20:>11.2f}  {a / 2**20:>10.2f}" for n, p, a in rows]
        lines.append(f"{'total':<{w}}  {sum(r[1] for r in rows) / 2**20:>11.2f}  {sum(r[2] for r in rows) / 2**20:>10.2f}")
        return "\n".join(lines)

    def __call__(self, x: torch.Tensor, pid: int = 0) -> torch.Tensor:
        """Single-input single-output convenience wrapper."""
        out = self.forward({self.input_nodes[0]._uid: x}, pid)
        return out[self.output_nodes[0]._uid]

    # ---------------------------------------------------------------- checkpointing
    def state(self) -> dict:
        """Plain-data description (nodes, edges, layer configs, parameter tensors in descriptor order)."""
        idx = {id(n): i for i, n in enumerate(self.nodes)}
        layers = self.layers()
        lidx = {id(l): i for i, l in enumerate(layers)}
        params = []
        for l in layers:
            desc = l.param_descriptors() if hasattr(l, "param_descriptors") else list(l.params)
            params.append([self._master_view(t) for t in desc])
        return {
            "nodes": [n._uid for n in self.nodes],
            "inputs": [idx[id(n)] for n in self.input_nodes],
            "outputs": [idx[id(n)] for n in self.output_nodes],
            "layers": [json.dumps(_sorted(l.get_config()), separators=(",", ":")) for l in layers],
            "edges": [(lidx[id(e.layer)], [idx[id(p)] for p in e.producers], [idx[id(c)] for c in e.consumers])
                      for e in self.edges],
            "params": params,
        }

    def _master_view(self, t: torch.Tensor) -> torch.Tensor:
        """fp32 master values of a parameter view (checkpoints store the master precision)."""
        if self.master_flat is self.params_flat or t.numel() == 0:
            return t.detach().float().cpu().contiguous()
        off = (t.data_ptr() - self.params_flat.data_ptr()) // self.params_flat.element_size()
        if t.is_contiguous():
            return self.master_flat[off:off + t.numel()].view(t.shape).detach().cpu().contiguous()
        return torch.as_strided(self.master_flat, t.shape, t.stride(), off).detach().cpu().contiguous()

    def save_state(self, path: str):
        from ..io import tnng
        tnng.write_file(path, self.state())

    @classmethod
    def from_state(cls, st: dict, device="cpu", **compile_kw) -> "Graph":
        g = cls()
        nodes = [g.make_node(uid) for uid in st["nodes"]]
        for i in st["inputs"]:
            g.set_input(nodes[i])
        for i in st["outputs"]:
            g.set_output(nodes[i])
        layers = [layer_from_config(json.loads(s)) for s in st["layers"]]
        for li, prod, cons in st["edges"]:
            g.add_edge(layers[li], [nodes[i] for i in prod], [nodes[i] for i in cons])
        if not st["inputs"] and not st["outputs"]:  # version-1 files: infer from degrees
            produced = {id(c) for e in g.edges for c in e.consumers}
            consumed = {id(p) for e in g.edges for p in e.producers}
            for n in nodes:
                if id(n) not in produced:
                    g.set_input(n)
                if id(n) not in consumed:
                    g.set_output(n)
        g.compile(device=device, init=False, **compile_kw)
        if st.get("params") is not None:
            if len(st["params"]) != len(layers):
                raise ValueError("Graph state parameter section does not match layer count")
            for l, tensors in zip(layers, st["params"]):
                desc = l.param_descriptors() if hasattr(l, "param_descriptors") else list(l.params)
                if len(desc) != len(tensors):
                    raise ValueError("Graph state parameter count does not match layer definition")
                for d, t in zip(desc, tensors):
                    g._load_param(d, t)
            g.sync_params_from_master()
        return g

    def _load_param(self, view: torch.Tensor, value: torch.Tensor):
        value = value.reshape(view.shape)
        if self.master_flat is self.params_flat:
            view.copy_(value.to(view.dtype))
            return
        off = (view.data_ptr() - self.params_flat.data_ptr()) // self.params_flat.element_size()
        torch.as_strided(self.master_flat, view.shape, view.stride(), off).copy_(value.float())

    @classmethod
    def load_state(cls, path: str, device="cpu", **compile_kw) -> "Graph":
        from ..io import tnng
        return cls.from_state(tnng.read_file(path), device=device, **compile_kw)


def infer_shapes(graph: "Graph", input_shapes: Dict[str, Tuple[int, ...]]) -> Dict[str, Tuple[int, ...]]:
    """Static shape of every node, from the layers' ``output_shape`` rules (no tensors involved)."""
    graph.sort()
    shapes = dict(input_shapes)
    for e in graph.edges:
        ins = [tuple(shapes[p.uid()]) for p in e.producers]
        shapes[e.consumers[0].uid()] = tuple(e.layer.output_shape(ins))
    return shapes


def partition_graph(graph: "Graph", ratios: Sequence[float]) -> List["Graph"]:
    """Cut the sorted edge list into contiguous pipeline stages by ``ratios`` with the C++
    partitioner (same algorithm and boundaries as src/partitioner/graph_partitioner.cpp:101-260:
    a stage's inputs are the nodes it consumes but does not produce, its outputs the nodes it
    produces that a later stage consumes or that nothing consumes). Stage graphs share the layer
    objects of ``graph`` and are returned uncompiled; ``stage.start_layer`` / ``stage.layer_count``
    give the position in the full edge list."""
    from ..host import H
    graph.sort()
    parts = H.partition(graph.ir(), [float(r) for r in ratios])
    stages = []
    for p in parts:
        g = Graph()
        nodes = [g.make_node(uid) for uid in p["nodes"]]
        for i in p["inputs"]:
            g.set_input(nodes[i])
        for i in p["outputs"]:
            g.set_output(nodes[i])
        for eid, (_, prod, cons) in zip(p["edge_ids"], p["edges"]):
            g.add_edge(graph.edges[eid].layer, [nodes[i] for i in prod], [nodes[i] for i in cons])
        g.start_layer, g.layer_count = int(p["start_layer"]), int(p["layer_count"])
        g.input_uids, g.output_uids = list(p["input_uids"]), list(p["output_uids"])
        stages.append(g)
    return stages


def _sorted(o):
    if isinstance(o, dict):
        return {k: _sorted(o[k]) for k in sorted(o)}
    if isinstance(o, list):
        return [_sorted(v) for v in o]
    return o


# ================================================================== execution segments
class _Segment:
    start: int
    end: int

    def forward(self, vals: dict, ctx: dict):
        raise NotImplementedError

    def backward(self, gvals: dict, ctx: dict, no_grad_nodes: set):
        raise NotImplementedError

    def inner_floors(self, g: "Graph") -> List[int]:
        """Floors a segment reports through ``g.grad_hook`` from inside its own backward (firing order)."""
        return []


def _accum(gvals: dict, node: Node, g: Optional[torch.Tensor]):
    """Fan-out gradient accumulation (include/nn/node.hpp:29-63)."""
    if g is None:
        return
    k = id(node)
    if k in gvals and gvals[k] is not None:
        gvals[k] = raw.binary(gvals[k], g, "add")
    else:
        gvals[k] = g


class _EdgeSegment(_Segment):
    """One edge executed through its layer's own forward/backward."""

    def __init__(self, g: Graph, i: int):
        self.start, self.end = i, i + 1
        self.edge = g.edges[i]
        self.absorb = bool(g.fuse)

    def forward(self, vals, ctx):
        e = self.edge
        out = e.layer.forward([vals[id(p)] for p in e.producers], ctx)
        vals[id(e.consumers[0])] = out

    def backward(self, gvals, ctx, no_grad_nodes):
        e = self.edge
        g = gvals.pop(id(e.consumers[0]), None)
        if g is None:
            return
        if all(id(p) in no_grad_nodes for p in e.producers):
            ctx["_skip_dgrad"] = True
        # Fan-out into a convolution (a residual block's input feeds the main path's first convolution and the
        # shortcut): when the other branch's gradient is already there, the convolution adds it while it writes its
        # own input gradient (GEMM epilogue for 1 x 1 filters) instead of a separate three-tensor add afterwards.
        absorbed = False
        if self.absorb and type(e.layer) is Conv2D and "_skip_dgrad" not in ctx:
            prev = gvals.get(id(e.producers[0]))
            if prev is not None and prev.dtype == g.dtype and tuple(prev.shape) == tuple(ctx["x"].shape):
                ctx["_add_to_dx"] = gvals.pop(id(e.producers[0]))
                absorbed = True
        gin = e.layer.backward(g, ctx)
        if absorbed:
            gvals[id(e.producers[0])] = gin[0]
            return
        for p, gi in zip(e.producers, gin):
            if id(p) not in no_grad_nodes:
                _accum(gvals, p, gi)


class _BnAddSegment(_Segment):
    """batch norm -> add in one pass: ``y = relu?(bn(x)) + other``, where the add consumes the norm's output and the
    value of another branch (the closing add of a bottleneck block, whose last norm carries the ReLU -
    src/nn/example_graphs.cpp:176-196). The norm's apply pass reads ``other`` and writes the sum, which replaces a
    separate kernel that reads two tensors and writes a third. Backward: the add hands its gradient to both
    operands unchanged and the norm's ReLU mask depends on ``bn(x)`` alone, so the layers' own backward passes run
    as they are. Off the GPU (fp32 reference path) the two layers run one after the other."""

    def __init__(self, g: Graph, i: int):
        self.start, self.end = i, i + 2
        self.bn_edge, self.add_edge = g.edges[i], g.edges[i + 1]
        self.bn: BatchNorm = self.bn_edge.layer
        mid = self.bn_edge.consumers[0]
        self.other = [p for p in self.add_edge.producers if p is not mid][0]
        self.bn_first = self.add_edge.producers[0] is mid

    @staticmethod
    def match(g: Graph, i: int, cons, outs):
        E = g.edges
        if i + 2 > len(E):
            return None
        a, b = E[i], E[i + 1]
        if not (isinstance(a.layer, BatchNorm) and type(b.layer) is Add and len(b.producers) == 2):
            return None
        if a.layer.use_relu and not a.layer.affine:  # the backward could not recompute the mask from x
            return None
        mid = a.consumers[0]
        if sum(p is mid for p in b.producers) != 1 or cons.get(id(mid), []) != [i + 1] or id(mid) in outs:
            return None
        return _BnAddSegment(g, i)

    def forward(self, vals, ctx):
        x = vals[id(self.bn_edge.producers[0])]
        other = vals[id(self.other)]
        bctx = ctx["bn"] = {"_step": ctx.get("_step"), "_pid": ctx.get("_pid")}
        fused = x.is_cuda and x.dtype == torch.bfloat16 and other.shape == x.shape and other.dtype == x.dtype
        if fused:
            bctx["_post_add"] = other
            out = self.bn.forward([x], bctx)
        else:
            y = self.bn.forward([x], bctx)
            out = self.add_edge.layer.forward([y, other] if self.bn_first else [other, y], ctx.setdefault("add", {}))
        vals[id(self.add_edge.consumers[0])] = out

    def backward(self, gvals, ctx, no_grad_nodes):
        g = gvals.pop(id(self.add_edge.consumers[0]), None)
        if g is None:
            return
        if id(self.other) not in no_grad_nodes:
            _accum(gvals, self.other, g)
        src = self.bn_edge.producers[0]
        if id(src) not in no_grad_nodes or self.bn.grads[0] is not None:
            gin = self.bn.backward(g, ctx["bn"])
            if id(src) not in no_grad_nodes:
                _accum(gvals, src, gin[0])


class _EmbedSegment(_Segment):
    """embedding -> pos_embedding -> dropout in one gather kernel (and one scatter kernel back)."""

    def __init__(self, g: Graph, i: int):
        self.start, self.end = i, i + 3
        self.e = g.edges[i:i + 3]
        self.emb: Embedding = self.e[0].layer
        self.pos: PositionalEmbedding = self.e[1].layer
        self.drop: Dropout = self.e[2].layer

    @staticmethod
    def match(g: Graph, i: int, cons, outs):
        E = g.edges
        if i + 3 > len(E):
            return None
        a, b, c = E[i:i + 3]
        if not (type(a.layer) is Embedding and type(b.layer) is PositionalEmbedding and type(c.layer) is Dropout):
            return None
        n1, n2 = a.consumers[0], b.consumers[0]
        if b.producers != [n1] or c.producers != [n2]:
            return None
        if cons.get(id(n1), []) != [i + 1] or cons.get(id(n2), []) != [i + 2] or id(n1) in outs or id(n2) in outs:
            return None
        return _EmbedSegment(g, i)

    def forward(self, vals, ctx):
        ids = vals[id(self.e[0].producers[0])]
        B, S = ids.shape
        if S != self.pos.seq_len:
            raise ValueError(f"pos_embedding {self.pos.name}: sequence length {S} != {self.pos.seq_len}")
        p = self.drop.dropout_rate if self.drop.training else 0.0
        seed = self.drop.step_seed(ctx)
        ctx.update(ids=ids, p=p, seed=seed)
        out = raw.embedding_fwd(ids, self.emb.params[0], self.pos.params[0], S, self.emb.padding_idx, p, seed)
        vals[id(self.e[2].consumers[0])] = out.reshape(B, S, self.emb.embed_dim)

    def backward(self, gvals, ctx, no_grad_nodes):
        g = gvals.pop(id(self.e[2].consumers[0]), None)
        if g is None:
            return
        raw.embedding_bwd(ctx["ids"], _flat2d(g), self.emb.grads[0], self.pos.grads[0], self.pos.seq_len,
                          self.emb.padding_idx, ctx["p"], ctx["seed"])


_BLOCK_TYPES = (LayerNorm, FlashAttentionBlock, Dropout, Add, LayerNorm, Dense, GELU, Dense, Dropout, Add)


class _GPTChain(_Segment):
    """A run of pre-LN transformer blocks (optionally closed by the final layer_norm).

    Per block the forward is 7 launches: LN1 | QKV GEMM+bias | flash attention | out-proj GEMM+bias |
    [residual add + dropout + LN2] | fc1 GEMM+bias+GELU | fc2 GEMM+bias; the block's trailing
    ``x + dropout(fc2)`` is folded into the next block's LN1 kernel (or the final layer_norm).
    The reference runs the same block as 10 layers plus 4 transposes, each its own launch
    (src/nn/example_graphs.cpp:198-215, src/nn/blocks_impl/flash_attention_block.cpp:39-138).
    """

    def __init__(self, g: Graph, start: int, n_blocks: int, final_ln: bool):
        self.g = g
        self.start = start
        self.end = start + 10 * n_blocks + (1 if final_ln else 0)
        self.blocks = [[g.edges[start + 10 * b + k] for k in range(10)] for b in range(n_blocks)]
        self.final = g.edges[self.end - 1] if final_ln else None
        self.in_node = self.blocks[0][0].producers[0]
        self.out_node = (self.final.consumers[0] if final_ln else self.blocks[-1][9].consumers[0])

    @staticmethod
    def _match_block(g: Graph, i: int, cons, outs) -> bool:
        E = g.edges
        if i + 10 > len(E):
            return False
        es = E[i:i + 10]
        for e, t in zip(es, _BLOCK_TYPES):
            if type(e.layer) is not t:
                return False
        x = es[0].producers[0]
        n = [e.consumers[0] for e in es]
        wiring = (es[1].producers == [n[0]] and es[2].producers == [n[1]] and es[3].producers == [x, n[2]]
                  and es[4].producers == [n[3]] and es[5].producers == [n[4]] and es[6].producers == [n[5]]
                  and es[7].producers == [n[6]] and es[8].producers == [n[7]] and es[9].producers == [n[3], n[8]])
        if not wiring:
            return False
        expect = {0: [i + 1], 1: [i + 2], 2: [i + 3], 3: [i + 4, i + 9], 4: [i + 5], 5: [i + 6], 6: [i + 7], 7: [i + 8],
                  8: [i + 9]}
        for k, c in expect.items():
            if sorted(cons.get(id(n[k]), [])) != c or id(n[k]) in outs:
                return False
        if sorted(cons.get(id(x), [])) != [i, i + 3]:
            return False
        ln1, attn, ln2, fc1, fc2 = es[0].layer, es[1].layer, es[4].layer, es[5].layer, es[7].layer
        if not (ln1.affine and ln2.affine and fc1.use_bias and fc2.use_bias and attn.head_dim == 64):
            return False
        return ln1.normalized_shape % 8 == 0 and ln1.normalized_shape <= 2048

    @staticmethod
    def match(g: Graph, i: int, cons, outs):
        nb = 0
        j = i
        while _GPTChain._match_block(g, j, cons, outs):
            nb += 1
            out = g.edges[j + 9].consumers[0]
            j += 10
            # the block output must feed exactly the next block (its LN1 and its residual add)
            if id(out) in outs or sorted(cons.get(id(out), [])) != [j, j + 3] or not _GPTChain._match_block(g, j, cons, outs):
                break
        if nb == 0:
            return None
        final_ln = False
        last_out = g.edges[j - 1].consumers[0]
        if (j < len(g.edges) and type(g.edges[j].layer) is LayerNorm and g.edges[j].producers == [last_out]
                and cons.get(id(last_out), []) == [j] and id(last_out) not in outs and g.edges[j].layer.affine):
            final_ln = True
        return _GPTChain(g, i, nb, final_ln)

    @staticmethod
    def _block_floor(g: Graph, es) -> int:
        return min(f for f in (g._layer_floor(e.layer) for e in es) if f is not None)

    def inner_floors(self, g: Graph) -> List[int]:
        return [self._block_floor(g, es) for es in reversed(self.blocks)]

    # The residual stream is carried as (x, pending): the true value is x + dropout(pending).
    def forward(self, vals, ctx):
        x3 = vals[id(self.in_node)]
        B, S, E = x3.shape
        x = _flat2d(x3).contiguous()
        pending, p_pend, seed_pend = None, 0.0, 0
        saved = []
        for es in self.blocks:
            ln1, attn, drop1, _, ln2, fc1, _, fc2, drop2, _ = (e.layer for e in es)
            s = {}
            x, h1, s["mean1"], s["rstd1"] = raw.layernorm_fwd(x, pending, ln1.params[0], ln1.params[1], ln1.epsilon,
                                                              p_pend, seed_pend)
            s["x"], s["h1"], s["p_in"], s["seed_in"], s["had_pending"] = x, h1, p_pend, seed_pend, pending is not None
            wqkv, bqkv, wo, bo = attn.params
            qkv = gemm(h1, wqkv, bias=bqkv)
            a, lse = raw.attn_fwd(qkv, B, S, attn.num_heads, attn.head_dim, attn.is_causal, attn.attn_scale)
            y1 = gemm(a, wo, bias=bo)
            p1 = drop1.dropout_rate if drop1.training else 0.0
            seed1 = drop1.step_seed(ctx)
            x1, h2, s["mean2"], s["rstd2"] = raw.layernorm_fwd(x, y1, ln2.params[0], ln2.params[1], ln2.epsilon, p1, seed1)
            z = torch.empty(x.shape[0], fc1.output_features, dtype=x.dtype, device=x.device)
            gact = gemm(h2, fc1.params[0], bias=fc1.params[1], gelu=True, save_preact=z)
            y2 = gemm(gact, fc2.params[0], bias=fc2.params[1])
            # recompute_qkv: the packed projection (3 x the residual stream per block) is not kept for the backward
            # pass but computed again there from the saved layer-norm output
            s.update(qkv=None if attn.recompute_qkv else qkv, a=a, lse=lse, x1=x1, h2=h2, z=z, g=gact, p1=p1, seed1=seed1)
            saved.append(s)
            x, pending = x1, y2
            p_pend = drop2.dropout_rate if drop2.training else 0.0
            seed_pend = drop2.step_seed(ctx)
        ctx["saved"], ctx["dims"] = saved, (B, S, E)
        ctx["tail"] = (p_pend, seed_pend)
        if self.final is not None:
            ln = self.final.layer
            xf, hf, mean, rstd = raw.layernorm_fwd(x, pending, ln.params[0], ln.params[1], ln.epsilon, p_pend, seed_pend)
            ctx["final"] = (xf, mean, rstd)
            out = hf
        else:
            out = raw.binary(x, raw.dropout(pending, p_pend, seed_pend), "add")
        vals[id(self.out_node)] = out.reshape(B, S, E)

    def backward(self, gvals, ctx, no_grad_nodes):
        g = gvals.pop(id(self.out_node), None)
        if g is None:
            return
        B, S, E = ctx["dims"]
        g = _flat2d(g).contiguous()
        p_pend, seed_pend = ctx["tail"]
        if self.final is not None:
            ln = self.final.layer
            xf, mean, rstd = ctx["final"]
            # the layer-norm backward kernels also sum the columns of the ddelta they emit: that is the bias gradient
            # of the dense layer in front of the norm (fc2 of the last block here)
            dres, dpend = raw.layernorm_bwd(g, xf, mean, rstd, ln.params[0], None, True, p_pend, seed_pend,
                                            ln.grads[0], ln.grads[1], dbias=self.blocks[-1][7].layer.grads[1])
            bias_done = True
        else:
            dres, dpend = g, raw.dropout(g, p_pend, seed_pend)
            bias_done = False
        for bi in reversed(range(len(self.blocks))):
            es, s = self.blocks[bi], ctx["saved"][bi]
            ln1, attn, _, _, ln2, fc1, _, fc2, _, _ = (e.layer for e in es)
            # fc2
            gemm(dpend, s["g"], a_t=True, b_t=True, out=fc2.grads[0], atomic=True)
            if not bias_done:
                raw.colsum_accum(dpend, fc2.grads[1])
            dz = gemm(dpend, fc2.params[0], b_t=True, dgelu_of=s["z"])
            # fc1
            gemm(dz, s["h2"], a_t=True, b_t=True, out=fc1.grads[0], atomic=True)
            raw.colsum_accum(dz, fc1.grads[1])
            dh2 = gemm(dz, fc1.params[0], b_t=True)
            # LN2 + residual + dropout
            dx1, dy1 = raw.layernorm_bwd(dh2, s["x1"], s["mean2"], s["rstd2"], ln2.params[0], dres, True, s["p1"],
                                         s["seed1"], ln2.grads[0], ln2.grads[1], dbias=attn.grads[3])
            # attention
            wqkv, bqkv, wo, bo = attn.params
            gemm(dy1, s["a"], a_t=True, b_t=True, out=attn.grads[2], atomic=True)
            da = gemm(dy1, wo, b_t=True)
            qkv = s["qkv"] if s["qkv"] is not None else gemm(s["h1"], wqkv, bias=bqkv)
            dqkv = raw.attn_bwd(qkv, s["a"], da, s["lse"], B, S, attn.num_heads, attn.head_dim, attn.is_causal,
                                attn.attn_scale)
            gemm(dqkv, s["h1"], a_t=True, b_t=True, out=attn.grads[0], atomic=True)
            raw.colsum_accum(dqkv, attn.grads[1])
            dh1 = gemm(dqkv, wqkv, b_t=True)
            # LN1 (+ the previous block's trailing residual add + dropout)
            bias_done = bool(s["had_pending"]) and bi > 0
            dres, dpend = raw.layernorm_bwd(dh1, s["x"], s["mean1"], s["rstd1"], ln1.params[0], dx1, s["had_pending"],
                                            s["p_in"], s["seed_in"], ln1.grads[0], ln1.grads[1],
                                            dbias=self.blocks[bi - 1][7].layer.grads[1] if bias_done else None)
            if self.g.grad_hook is not None:  # this block and everything after it in the flat buffer is final
                self.g.grad_hook(self._block_floor(self.g, es))
        if id(self.in_node) not in no_grad_nodes:
            _accum(gvals, self.in_node, dres.reshape(B, S, E))
