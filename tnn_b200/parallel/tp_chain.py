"""Tensor-parallel execution of a run of transformer blocks (see :mod:`tnn_b200.parallel.tp`).

Rows of the residual stream are split over the tensor-parallel ranks (sequence parallelism): the
layernorm / residual / dropout kernels work on ``M/tp`` rows, the attention and MLP GEMMs on all
``M`` rows but ``1/tp`` of the heads / hidden width. Per block and direction there are two
all-gather->GEMM and two GEMM->reduce-scatter hand-offs; the rows travel inside the layer-norm kernels and the
GEMM epilogues (pushed with peer stores), so no stand-alone collective or copy kernel is issued.
"""
from __future__ import annotations

from typing import List

import torch

from ..nn.graph import Graph, _EmbedSegment, _GPTChain, _Segment, _accum, _flat2d
from ..ops import raw
from ..ops.gemm import gemm
from .tp import CommContext, GatherSite, ScatterSite, _reinit_shards


class _TPGPTChain(_Segment):
    def __init__(self, chain: _GPTChain, cc: CommContext, ring: int = 1, in_is_shard: bool = False):
        self.start, self.end = chain.start, chain.end
        self.blocks, self.final = chain.blocks, chain.final
        self.in_node, self.out_node = chain.in_node, chain.out_node
        self.cc = cc
        # One set of symmetric buffers per micro-batch that can be in flight (pipeline stages keep the
        # gathered activations of a micro-batch until its backward pass).
        self.ring = max(1, ring)
        self.site_ring = {}
        # True when the chain starts at a pipeline-stage boundary: the input is already this rank's rows
        self.in_is_shard = in_is_shard

    def _make_sites(self, M: int, E: int):
        cc = self.cc
        # pass counters of this set of sites: one per direction, bumped at the start of every pass
        cf, cb = cc.new_pass_counter(), cc.new_pass_counter()
        sites = []
        for es in self.blocks:
            fc1 = es[5].layer
            F = fc1.output_features // cc.tp
            sites.append({
                "g1": GatherSite(cc, M, E, cf), "g2": GatherSite(cc, M, E, cf),          # forward: LN1 / LN2 outputs
                "gb1": GatherSite(cc, M, E, cb), "gb2": GatherSite(cc, M, E, cb),        # backward: dY of out-proj / fc2
                "s_out": ScatterSite(cc, M, E, cf), "s_fc2": ScatterSite(cc, M, E, cf),  # forward reduce-scatters
                "s_qkv": ScatterSite(cc, M, E, cb), "s_fc1": ScatterSite(cc, M, E, cb),  # backward reduce-scatters
                "F": F, "pass_f": cf, "pass_b": cb,
            })
        return sites

    def _ln_into(self, site: GatherSite, x, pending, pend_site, ln, p, seed):
        """Layer norm of ``x + dropout(pending)`` straight into this rank's rows of a gather site; on the fused
        path the kernel also adds the peers' share of ``pending`` and delivers the result to the peers."""
        tgt = site.mine()
        xo, h, mean, rstd = raw.layernorm_fwd(x, pending, ln.params[0], ln.params[1], ln.epsilon, p, seed, h_out=tgt,
                                              tp_pull=pend_site.pull_args() if pend_site is not None else None,
                                              tp_push=site.push_args())
        if h.data_ptr() != tgt.data_ptr():
            tgt.copy_(h)
        return xo, mean, rstd

    def forward(self, vals, ctx):
        cc = self.cc
        x3 = vals[id(self.in_node)]
        E = x3.shape[-1]
        rows_in = x3.numel() // E
        M = rows_in * cc.tp if self.in_is_shard else rows_in
        S = cc.seq_len or x3.shape[1]
        B = M // S
        if M % (128 * cc.tp):
            raise ValueError(f"tensor parallelism needs batch*seq ({M}) to be a multiple of {128 * cc.tp}")
        slot = int(ctx.get("_pid", 0)) % self.ring
        if slot not in self.site_ring or self.site_ring[slot][0] != M:
            self.site_ring[slot] = (M, self._make_sites(M, E))
        sites = ctx["sites"] = self.site_ring[slot][1]
        Ms = M // cc.tp
        sites[0]["pass_f"].add_(1)  # new pass number for every hand-off of this pass
        x = _flat2d(x3).contiguous() if self.in_is_shard else _flat2d(x3)[cc.idx * Ms:(cc.idx + 1) * Ms].contiguous()
        pending, pend_site, p_pend, seed_pend = None, None, 0.0, 0
        saved = []
        for es, st in zip(self.blocks, sites):
            ln1, attn, drop1, _, ln2, fc1, _, fc2, drop2, _ = (e.layer for e in es)
            s = {}
            x, s["mean1"], s["rstd1"] = self._ln_into(st["g1"], x, pending, pend_site, ln1, p_pend, seed_pend)
            s["x"], s["p_in"], s["seed_in"], s["had_pending"] = x, p_pend, seed_pend, pending is not None
            wqkv, bqkv, wo, bo = attn.params
            qkv = st["g1"].gemm(wqkv, bias=bqkv)                                  # [M, 3E/tp]
            heads = attn.num_heads // cc.tp
            a, lse = raw.attn_fwd(qkv, B, S, heads, attn.head_dim, attn.is_causal, attn.attn_scale)
            y1 = st["s_out"].gemm(a, wo, bias=bo)                                 # [Ms, E]
            p1 = drop1.dropout_rate if drop1.training else 0.0
            seed1 = drop1.step_seed(ctx)
            x1, s["mean2"], s["rstd2"] = self._ln_into(st["g2"], x, y1, st["s_out"], ln2, p1, seed1)
            z = torch.empty(M, st["F"], dtype=x.dtype, device=x.device)
            gact = st["g2"].gemm(fc1.params[0], bias=fc1.params[1], gelu_preact=z)  # [M, 4E/tp]
            y2 = st["s_fc2"].gemm(gact, fc2.params[0], bias=fc2.params[1])        # [Ms, E]
            s.update(qkv=None if attn.recompute_qkv else qkv, a=a, lse=lse, x1=x1, z=z, g=gact, p1=p1, seed1=seed1, heads=heads)
            saved.append(s)
            x, pending, pend_site = x1, y2, st["s_fc2"]
            p_pend = drop2.dropout_rate if drop2.training else 0.0
            seed_pend = drop2.step_seed(ctx)
        ctx["saved"], ctx["dims"], ctx["tail"] = saved, (B, S, E), (p_pend, seed_pend)
        if self.final is not None:
            ln = self.final.layer
            xf, hf, mean, rstd = raw.layernorm_fwd(x, pending, ln.params[0], ln.params[1], ln.epsilon, p_pend, seed_pend,
                                                   tp_pull=pend_site.pull_args() if pend_site is not None else None)
            ctx["final"] = (xf, mean, rstd)
            out = hf
        else:
            if pend_site is not None:
                pending = pend_site.resolve(pending)
            out = raw.binary(x, raw.dropout(pending, p_pend, seed_pend), "add")
        # downstream layers (the vocabulary head) see only this rank's rows
        vals[id(self.out_node)] = out.reshape(1, Ms, E)

    def backward(self, gvals, ctx, no_grad_nodes):
        g = gvals.pop(id(self.out_node), None)
        if g is None:
            return
        cc = self.cc
        B, S, E = ctx["dims"]
        M = B * S
        Ms = M // cc.tp
        g = _flat2d(g).contiguous()
        p_pend, seed_pend = ctx["tail"]
        sites = ctx["sites"]
        sites[0]["pass_b"].add_(1)
        last = sites[-1]
        if self.final is not None:
            ln = self.final.layer
            xf, mean, rstd = ctx["final"]
            dres, dpend = raw.layernorm_bwd(g, xf, mean, rstd, ln.params[0], None, True, p_pend, seed_pend, ln.grads[0],
                                            ln.grads[1], ddelta_out=last["gb2"].mine() if g.is_cuda else None,
                                            tp_push=last["gb2"].push_args() if g.is_cuda else None,
                                            dbias=self.blocks[-1][7].layer.grads[1])
            bias_done = True   # the norm's backward kernel summed the columns of the ddelta it emitted
        else:
            dres, dpend = g, raw.dropout(g, p_pend, seed_pend)
            bias_done = False
        for bi in reversed(range(len(self.blocks))):
            es, s, st = self.blocks[bi], ctx["saved"][bi], sites[bi]
            ln1, attn, _, _, ln2, fc1, _, fc2, _, _ = (e.layer for e in es)
            wqkv, bqkv, wo, bo = attn.params
            # ---- fc2 (row parallel): gather dY, dgrad with GELU' ----
            tgt = st["gb2"].mine()
            if dpend.data_ptr() != tgt.data_ptr():  # not written in place (and delivered) by a layer-norm backward
                st["gb2"].push(dpend)
            if not bias_done:
                raw.colsum_accum(tgt, fc2.grads[1])
            dz = st["gb2"].gemm(fc2.params[0], b_t=True, dgelu_of=s["z"])          # [M, 4E/tp]
            gemm(st["gb2"].buf, s["g"], a_t=True, b_t=True, out=fc2.grads[0], atomic=True)
            # ---- fc1 (column parallel) ----
            gemm(dz, st["g2"].buf, a_t=True, b_t=True, out=fc1.grads[0], atomic=True)
            raw.colsum_accum(dz, fc1.grads[1])
            dh2 = st["s_fc1"].gemm(dz, fc1.params[0], b_t=True)                    # [Ms, E]
            # ---- LN2 + residual + dropout ----
            dx1, dy1 = raw.layernorm_bwd(dh2, s["x1"], s["mean2"], s["rstd2"], ln2.params[0], dres, True, s["p1"], s["seed1"],
                                         ln2.grads[0], ln2.grads[1], ddelta_out=st["gb1"].mine() if dh2.is_cuda else None,
                                         tp_pull=st["s_fc1"].pull_args(), tp_push=st["gb1"].push_args() if dh2.is_cuda else None,
                                         dbias=attn.grads[3])
            tgt = st["gb1"].mine()
            if dy1.data_ptr() != tgt.data_ptr():
                st["gb1"].push(dy1)
            # ---- attention output projection (row parallel) ----
            da = st["gb1"].gemm(wo, b_t=True)                                      # [M, E/tp]
            gemm(st["gb1"].buf, s["a"], a_t=True, b_t=True, out=attn.grads[2], atomic=True)
            # recompute_qkv: the gathered layer-norm output is still complete in the site's buffer, a plain GEMM redoes it
            qkv = s["qkv"] if s["qkv"] is not None else gemm(st["g1"].buf, wqkv, bias=bqkv)
            dqkv = raw.attn_bwd(qkv, s["a"], da, s["lse"], B, S, s["heads"], attn.head_dim, attn.is_causal, attn.attn_scale)
            # ---- QKV projection (column parallel) ----
            gemm(dqkv, st["g1"].buf, a_t=True, b_t=True, out=attn.grads[0], atomic=True)
            raw.colsum_accum(dqkv, attn.grads[1])
            dh1 = st["s_qkv"].gemm(dqkv, wqkv, b_t=True)                           # [Ms, E]
            # ---- LN1 (+ the previous block's trailing residual add + dropout) ----
            prev = sites[bi - 1]["gb2"] if (bi > 0 and dh1.is_cuda and s["had_pending"]) else None
            bias_done = bool(s["had_pending"]) and bi > 0
            dres, dpend = raw.layernorm_bwd(dh1, s["x"], s["mean1"], s["rstd1"], ln1.params[0], dx1, s["had_pending"],
                                            s["p_in"], s["seed_in"], ln1.grads[0], ln1.grads[1],
                                            ddelta_out=prev.mine() if prev is not None else None,
                                            tp_pull=st["s_qkv"].pull_args(), tp_push=prev.push_args() if prev is not None else None,
                                            dbias=self.blocks[bi - 1][7].layer.grads[1] if bias_done else None)
        if self.in_is_shard:
            if id(self.in_node) not in no_grad_nodes:
                _accum(gvals, self.in_node, dres.reshape(1, Ms, E))
        elif id(self.in_node) not in no_grad_nodes:
            full = torch.zeros(M, E, dtype=dres.dtype, device=dres.device)
            full[cc.idx * Ms:(cc.idx + 1) * Ms] = dres
            _accum(gvals, self.in_node, full.reshape(B, S, E))


def install_tp_segments(graph: Graph, topo, heap, fused: bool = True, ring: int = 1) -> None:
    """Swap every fused GPT chain of a compiled graph for its tensor-parallel version and give the
    shards of each tensor-parallel rank their own random initialisation."""
    cc = CommContext(topo, heap, fused, graph.device)
    n = 0
    for k, seg in enumerate(graph.segments):
        if isinstance(seg, _GPTChain):
            graph.segments[k] = _TPGPTChain(seg, cc, ring, id(seg.in_node) in {id(n) for n in graph.input_nodes})
            n += 1
    if n == 0:
        raise ValueError("no transformer block chain found for tensor parallelism")
    _reinit_shards(graph, topo)
    graph.tp_context = cc
