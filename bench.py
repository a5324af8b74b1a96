#!/usr/bin/env python
"""Headline benchmark: GPT-2 small pre-training throughput (tokens/s) on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

The step is the full training step of the flagship configuration: GPT-2 small (12 layers, d=768,
12 heads, context 1024, vocabulary 50257, tanh-GELU, pre-LN, dropout 0.1, untied biased head),
bf16 compute with fp32 master weights, AdamW, 8 sequences of 1024 tokens per GPU (global batch 64
at 8 GPUs, weak scaling), synthetic uniform token ids, random-init weights. With more than one
GPU the layout is TP=2 x DP=N/2. The same invocation then measures ResNet-50 images/s (256 images per GPU, data
parallel) under the same rules and reports it as the ``resnet50`` sub-record of the line; ``--model resnet50`` runs
that configuration alone.

Two numbers are reported in one JSON line: ``value`` times K steps on the device (CUDA events,
max over ranks) with the batch already resident, ``e2e`` times the same K steps through
``Trainer.train_step`` including the pinned host->device upload of every batch and a device->host
read of every loss. ``--impl reference`` times the reference's own code instead (see
baseline/README.md for what can be built offline).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gpt2_small", choices=["gpt2_small", "gpt2_medium", "resnet50", "wrn16_8"])
    ap.add_argument("--per-gpu-batch", type=int, default=0)
    ap.add_argument("--parallelism", default="", help="override, e.g. dp8 or tp2dp4")
    ap.add_argument("--no-graph", action="store_true", help="do not capture the step in a CUDA graph")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(s) > 2 + i and s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


BASELINE_PUBLISHED = None  # the reference publishes no throughput numbers


def model_setup(args):
    if args.model.startswith("gpt2"):
        per_gpu = args.per_gpu_batch or 8
        return {"zoo": args.model, "per_gpu_batch": per_gpu, "seq_len": 1024, "unit": "tokens/s", "metric": "tokens_per_sec",
                "items_per_sample": 1024, "optimizer": {"type": "adamw", "learning_rate": 3e-4, "beta1": 0.9, "beta2": 0.95,
                                                        "epsilon": 1e-8, "weight_decay": 0.1}}
    if args.model == "resnet50":
        per_gpu = args.per_gpu_batch or 256
        return {"zoo": "imagenet_resnet50", "per_gpu_batch": per_gpu, "seq_len": None, "unit": "images/s",
                "metric": "images_per_sec", "items_per_sample": 1, "optimizer": {"type": "sgd", "learning_rate": 0.01, "momentum": 0.9}}
    per_gpu = args.per_gpu_batch or 128
    return {"zoo": "cifar100_wrn16_8", "per_gpu_batch": per_gpu, "seq_len": None, "unit": "images/s", "metric": "images_per_sec",
            "items_per_sample": 1, "optimizer": {"type": "sgd", "learning_rate": 0.1, "momentum": 0.9}}


def run_ours(args):
    import torch
    import torch.distributed as dist

    from tnn_b200.data.loaders import SyntheticLoader
    from tnn_b200.models import zoo
    from tnn_b200.ops.gemm import LAUNCHES
    from tnn_b200.utils.config import TrainingConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    ms = model_setup(args)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(layout, sample_clocks, ms=ms):
        """Build the trainer for one layout, warm up, time K resident steps on the device and K end-to-end steps."""
        cfg = TrainingConfig.from_dict({"model_name": ms["zoo"], "batch_size": ms["per_gpu_batch"], "device_type": "CUDA",
                                        "optimizer": ms["optimizer"], "scheduler": {"type": "no_op"},
                                        "loss": {"type": "logsoftmax_crossentropy"}, "seed": 0})
        is_lm = ms["seq_len"] is not None
        if world > 1:
            from tnn_b200.parallel.runtime import ParallelTrainer
            trainer = ParallelTrainer(cfg, layout=layout, log=False)
        else:
            from tnn_b200.trainer import Trainer
            trainer = Trainer(cfg, device=dev, log=False)
        lb = trainer.local_batch if world > 1 else ms["per_gpu_batch"]
        seed = 1234 + getattr(trainer, "data_rank", rank)
        if is_lm:
            loader = SyntheticLoader((ms["seq_len"],), 50257, lb, 10 ** 9, tokens=True, seed=seed)
        else:
            classes = 1000 if ms["zoo"] == "imagenet_resnet50" else 100
            # images are produced in the io dtype (bf16), as the reference's loaders emit `io_dtype` floats
            loader = SyntheticLoader(zoo.INPUT_SHAPES[ms["zoo"]], classes, lb, 10 ** 9, seed=seed, dtype=torch.bfloat16)
        batches = iter(loader)
        # ---- warm-up (also captures the CUDA graph) ----
        data, labels = next(batches)
        if not args.no_graph:
            trainer.enable_cuda_graph(data, labels)
        for _ in range(max(3, args.warmup)):
            data, labels = next(batches)
            loss = trainer.train_step(data, labels)
        barrier()
        first_loss = float(loss.item())
        # ---- device-timed region: K steps, batch resident, no host sync in between ----
        sampler = ClockSampler(local) if sample_clocks else None
        if sampler:
            sampler.start()
        time.sleep(0.3)
        n0 = LAUNCHES["count"]
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            loss = trainer.step_resident()
        e1.record()
        barrier()
        dev_ms = e0.elapsed_time(e1)
        launches = (LAUNCHES["count"] - n0) if trainer.launches_per_step == 0 else trainer.launches_per_step * args.steps
        # ---- end-to-end region: fresh pinned batch uploaded and loss read back every step ----
        barrier()
        t0 = time.perf_counter()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record()
        last = 0.0
        # every step's batch goes host -> device from pinned memory inside the timed region; the copy of step k+1 is
        # started (Trainer.prefetch, copy stream) right after step k has been launched, so it overlaps step k's compute
        nxt = next(batches)
        for i in range(args.steps):
            data, labels = nxt
            loss = trainer.train_step(data, labels)
            if i + 1 < args.steps:
                nxt = next(batches)
                trainer.prefetch(*nxt)
            last = float(loss.item())
        e3.record()
        barrier()
        e2e_ms = max(e2.elapsed_time(e3), (time.perf_counter() - t0) * 1e3)
        clocks = sampler.stop() if sampler else {}
        if world > 1:
            t = torch.tensor([dev_ms, e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dev_ms, e2e_ms = float(t[0]), float(t[1])
            if sampler:
                clocks = merge_clocks(clocks, world)
        from tnn_b200.ops import _lib
        _lib.check_status(dev)
        global_batch = trainer.global_batch if world > 1 else ms["per_gpu_batch"]
        items = global_batch * ms["items_per_sample"]
        res = {"layout": layout, "global_batch": global_batch, "dev_ms": dev_ms, "e2e_ms": e2e_ms,
               "value": items * args.steps / (dev_ms / 1e3), "e2e": items * args.steps / (e2e_ms / 1e3),
               "h2d": int(data.numel() * data.element_size() + labels.numel() * labels.element_size()), "launches": int(launches),
               "first_loss": first_loss, "last_loss": last, "clocks": clocks}
        trainer.close()
        del trainer
        torch.cuda.empty_cache()
        barrier()
        return res

    def measure_pipeline(layout, sample_clocks):
        """Pipeline layouts (``pp4tp2`` ...): 1F1B over the partitioner's stages, 8 micro-batches per step, stage
        send / recv on NCCL point-to-point; after the timed steps every stage writes its TNNG file and reads it back."""
        import tempfile

        from tnn_b200.nn.graph import Graph
        from tnn_b200.parallel.pp import PipelineTrainer
        from tnn_b200.parallel.runtime import parse_layout

        n_stages = parse_layout(layout)["pp"]
        micro = 8
        pcfg = TrainingConfig.from_dict({"model_name": ms["zoo"], "batch_size": ms["per_gpu_batch"] * n_stages, "device_type": "CUDA",
                                         "optimizer": ms["optimizer"], "scheduler": {"type": "no_op"},
                                         "loss": {"type": "logsoftmax_crossentropy"}, "seed": 0,
                                         "parallel": {"microbatches": micro}})
        trainer = PipelineTrainer(pcfg, layout)
        lb = trainer.local_batch
        loader = SyntheticLoader((ms["seq_len"],), 50257, lb, 10 ** 9, tokens=True, seed=1234 + trainer.data_rank)
        batches = iter(loader)
        loss = None
        for _ in range(max(3, args.warmup)):
            data, labels = next(batches)
            loss = trainer.train_step(data, labels)
        barrier()
        first_loss = float(loss.item()) if loss is not None else None
        sampler = ClockSampler(local) if sample_clocks else None
        if sampler:
            sampler.start()
        time.sleep(0.3)
        d_res, l_res = data.to(dev), labels.to(dev)
        n0 = LAUNCHES["count"]
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            loss = trainer.train_step(d_res, l_res)
        e1.record()
        barrier()
        dev_ms = e0.elapsed_time(e1)
        launches = LAUNCHES["count"] - n0
        barrier()
        t0 = time.perf_counter()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record()
        last = None
        for _ in range(args.steps):
            data, labels = next(batches)
            loss = trainer.train_step(data, labels)
            if loss is not None:
                last = float(loss.item())
        e3.record()
        barrier()
        e2e_ms = max(e2.elapsed_time(e3), (time.perf_counter() - t0) * 1e3)
        clocks = sampler.stop() if sampler else {}
        t = torch.tensor([dev_ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])
        if sampler:
            clocks = merge_clocks(clocks, world)
        from tnn_b200.ops import _lib
        _lib.check_status(dev)
        # ---- checkpoint round trip: one TNNG file per stage (tensor-parallel shards gathered), read back ----
        folder = [tempfile.mkdtemp(prefix="tnnb_bench_ckpt_") if rank == 0 else None]
        dist.broadcast_object_list(folder, src=0)
        t1 = time.perf_counter()
        name = trainer.save_stage(os.path.join(folder[0], "gpt2"))
        barrier()
        save_s = time.perf_counter() - t1
        ck = {"stage": trainer.topo.pp_idx, "ok": None}
        if trainer.topo.dp_idx == 0 and trainer.topo.tp_idx == 0:
            t2 = time.perf_counter()
            g2 = Graph.load_state(name, device="cpu")
            n_loaded = g2.num_parameters()
            n_stage = trainer.stage.num_parameters()
            # replicated parameters count once, sharded ones tp times
            ck = {"stage": trainer.topo.pp_idx, "bytes": os.path.getsize(name), "params": n_loaded, "load_s": round(time.perf_counter() - t2, 2),
                  "ok": bool(torch.isfinite(g2.params_flat).all()) and n_stage <= n_loaded <= n_stage * trainer.topo.tp}
            os.remove(name)
        allck, alll = [None] * world, [None] * world
        dist.all_gather_object(allck, ck)
        dist.all_gather_object(alll, (first_loss, last))
        stages = sorted((c for c in allck if c.get("ok") is not None), key=lambda c: c["stage"])
        losses = [x for x in alll if x[0] is not None][0]
        if rank == 0:
            try:
                os.rmdir(folder[0])
            except OSError:
                pass
        items = trainer.global_batch * ms["items_per_sample"]
        res = {"layout": layout, "global_batch": trainer.global_batch, "dev_ms": dev_ms, "e2e_ms": e2e_ms,
               "value": items * args.steps / (dev_ms / 1e3), "e2e": items * args.steps / (e2e_ms / 1e3),
               "h2d": int(data.numel() * data.element_size() + labels.numel() * labels.element_size()), "launches": int(launches),
               "first_loss": losses[0], "last_loss": losses[1], "clocks": clocks,
               "checkpoint": {"format": "TNNG, one file per stage", "save_s": round(save_s, 2), "stages": stages,
                              "round_trip_ok": all(c["ok"] for c in stages) and len(stages) == trainer.topo.pp},
               "microbatches": micro}
        trainer.close()
        del trainer
        torch.cuda.empty_cache()
        barrier()
        return res

    from tnn_b200.parallel.runtime import default_layout
    layout = args.parallelism or (named_layout(world, ms["zoo"]) if world > 1 else "single")
    if layout.startswith("pp"):
        r = measure_pipeline(layout, True)
        args.no_graph = True
    else:
        r = measure(layout, True)
    # The other half of the headline metric: ResNet-50 images/s (bottleneck blocks [3,4,6,3], 256 images of
    # 224 x 224 x 3 per GPU, bf16, SGD momentum 0.9, data parallel with the fused reduce + update kernel), measured in
    # the same invocation with the same rules. TNNB_BENCH_RESNET=0 leaves it out.
    resnet = None
    if args.model == "gpt2_small" and not args.parallelism and os.environ.get("TNNB_BENCH_RESNET", "1") != "0":
        rargs = argparse.Namespace(**{**vars(args), "model": "resnet50", "per_gpu_batch": 0})
        rms = model_setup(rargs)
        rl = f"dp{world}" if world > 1 else "single"
        try:
            rr = measure(rl, True, rms)
            resnet = {"metric": rms["metric"], "value": round(rr["value"], 1), "unit": rms["unit"], "ms_per_step": round(rr["dev_ms"] / args.steps, 3),
                      "steps": args.steps, "warmup": max(3, args.warmup), "dtype": "bf16",
                      "config": {"model": "resnet50", "global_batch": rr["global_batch"], "per_gpu_batch": rms["per_gpu_batch"],
                                 "image": "224x224x3 NHWC, N(0,1) pixels, labels uniform in [0,1000)", "parallelism": rl,
                                 "optimizer": "sgd momentum 0.9", "cuda_graph": not args.no_graph},
                      "e2e": {"value": round(rr["e2e"], 1), "unit": rms["unit"], "ms_per_step": round(rr["e2e_ms"] / args.steps, 3),
                              "h2d_bytes_per_step": rr["h2d"], "d2h_bytes_per_step": 4},
                      "gpu_launches": rr["launches"], "clocks": rr["clocks"],
                      "loss_first": round(rr["first_loss"], 4), "loss_last": round(rr["last_loss"], 4)}
        except Exception as e:  # the headline line must still be printed
            resnet = {"error": f"{type(e).__name__}: {e}"[:300]}
    alt = None
    dp_layout = default_layout(world, ms["zoo"])
    if world > 1 and not args.parallelism and layout != dp_layout and not layout.startswith("pp"):
        alt = measure(dp_layout, False)  # the same job as pure data parallelism, for comparison

    out = {
        "metric": ms["metric"], "value": round(r["value"], 1), "unit": ms["unit"], "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": round(r["dev_ms"] / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": (r["value"] / BASELINE_PUBLISHED) if BASELINE_PUBLISHED else None, "dtype": "bf16",
        "data": "synthetic (uniform random token ids / N(0,1) images, random-init weights)",
        "config": {"model": args.model, "global_batch": r["global_batch"], "seq_len": ms["seq_len"], "parallelism": layout,
                   "per_gpu_batch": ms["per_gpu_batch"], "optimizer": ms["optimizer"]["type"], "cuda_graph": not args.no_graph,
                   "l2": "working set (weights + activations, > 2 GB per step) far exceeds the 126 MB L2; no flush needed"},
        "clocks": r["clocks"],
        "e2e": {"value": round(r["e2e"], 1), "unit": ms["unit"], "ms_per_step": round(r["e2e_ms"] / args.steps, 3),
                "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": 4},
        "gpu_launches": r["launches"], "loss_first": round(r["first_loss"], 4), "loss_last": round(r["last_loss"], 4), "impl": "ours",
    }
    if "checkpoint" in r:
        out["checkpoint"] = r["checkpoint"]
        out["config"]["microbatches"] = r["microbatches"]
        out["config"]["schedule"] = "1F1B"
    if resnet is not None:
        out["resnet50"] = resnet
    if alt is not None:
        out["alt"] = {"parallelism": alt["layout"], "value": round(alt["value"], 1), "ms_per_step": round(alt["dev_ms"] / args.steps, 3),
                      "e2e_value": round(alt["e2e"], 1), "note": "same model, batch and steps as pure data parallelism (fused reduce + AdamW + broadcast kernel)"}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def merge_clocks(mine: dict, world: int) -> dict:
    """Every rank sampled its own GPU: report the slowest median SM clock, the union of the throttle reasons and the
    per-rank medians (a step that ends in a cross-rank barrier runs at the pace of the slowest GPU)."""
    import torch.distributed as dist

    allc = [None] * world
    dist.all_gather_object(allc, mine)
    med = [c.get("sm_mhz") for c in allc]
    known = [m for m in med if m is not None]
    reasons = sorted({r for c in allc for r in c.get("reasons", [])})
    return {"sm_mhz": min(known) if known else None, "sm_max_mhz": max((c.get("sm_max_mhz") or 0) for c in allc) or None,
            "reasons": reasons, "samples": sum(c.get("samples", 0) for c in allc), "sm_mhz_per_rank": med}


def named_layout(world: int, zoo_name: str) -> str:
    """The layout the benchmark configuration names: GPT-2 runs tensor-parallel pairs (fused all-gather->GEMM and
    GEMM->reduce-scatter) combined with data parallelism; the CNNs are data parallel."""
    if zoo_name == "gpt2_medium" and world == 8:
        return "pp4tp2"  # 1F1B over four partitioner stages, each a tensor-parallel pair
    if "gpt2" in zoo_name and world % 2 == 0:
        return "tp2" if world == 2 else f"tp2dp{world // 2}"
    return f"dp{world}"


def main():
    args = parse_args()
    if args.impl == "reference":
        from baseline.reference_arm import run_reference
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
