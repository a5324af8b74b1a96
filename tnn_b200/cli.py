"""Command line: ``python -m tnn_b200 <command>``.

    train     --config x.json [--layout dp8|tp2dp4|pp2 ...]   single device, or one rank of a torchrun job
    infer     --config x.json                                  validation loss / accuracy of model_path or a fresh model
    generate  --model gpt2_small|--model-path f.tnng --vocab vocab.bin [--tokens train.bin]
    tcp-worker      [port] [--host H] [--gpu]                  one pipeline stage served over TCP
    tcp-coordinator --config x.json                            partition a model, deploy it to TCP workers, train
    info                                                       devices, build status, registered models and layers

These are the counterparts of the reference's ``trainer``, ``inferencer`` and ``gpt2_inference`` binaries
(examples/trainer.cpp:15-85, examples/inferencer.cpp:12-70, examples/gpt2_inference.cpp:16-114) and of its
``tcp_coordinator`` / ``tcp_worker`` pair (examples/tcp_coordinator.cpp:27-128, examples/tcp_worker.cpp:39-141).
Inside one NVSwitch box the parallel path is ``train`` under ``torchrun`` with a ``--layout`` (one process per GPU,
no coordinator process); the TCP pair is for stages on other hosts.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _load_cfg(path: str):
    from .utils.config import TrainingConfig

    cfg = TrainingConfig.load_from_json(path)
    print(json.dumps(cfg.to_dict(), indent=2, default=str))
    return cfg


def cmd_train(a) -> int:
    cfg = _load_cfg(a.config)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        import torch.distributed as dist

        local = int(os.environ.get("LOCAL_RANK", "0"))
        on_gpu = cfg.device_type.upper() == "CUDA" and torch.cuda.is_available()
        if on_gpu:
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
        from .parallel.runtime import default_layout, parse_layout

        layout = a.layout or cfg.parallel.layout or default_layout(world, cfg.model_name)
        try:
            if parse_layout(layout)["pp"] > 1:
                from .parallel.pp import PipelineTrainer

                t = PipelineTrainer(cfg, layout, fused=on_gpu)
            else:
                from .parallel.runtime import ParallelTrainer

                t = ParallelTrainer(cfg, layout=layout, fused=on_gpu)
            res = t.fit()
            if dist.get_rank() == 0:
                print(json.dumps(res))
            t.close()
        finally:
            dist.destroy_process_group()
        return 0
    from .trainer import train_model

    print(json.dumps(train_model(cfg)))
    return 0


def cmd_infer(a) -> int:
    from .inference import evaluate
    from .trainer import Trainer

    cfg = _load_cfg(a.config)
    t = Trainer(cfg, log=False)
    res = evaluate(t, max_batches=a.max_batches)
    print(f"Validation Loss: {res['loss']:.6f}, Accuracy: {res['accuracy_pct']:.2f}%")
    t.close()
    return 0


def cmd_generate(a) -> int:
    from .data.tokenizer import Tokenizer
    from .inference import greedy_generate, model_seq_len
    from .models import zoo
    from .nn.graph import Graph

    dev = torch.device("cuda" if (a.device.upper() == "CUDA" and torch.cuda.is_available()) else "cpu")
    if a.model_path:
        g = Graph.load_state(a.model_path, device=dev)
    else:
        g = zoo.create(a.model).compile(device=dev, seed=a.seed)
    tok = Tokenizer(a.vocab) if a.vocab else None
    if a.prompt_ids:
        prompt = [int(t) for t in a.prompt_ids.split(",")]
    elif a.tokens:
        import numpy as np

        data = np.memmap(a.tokens, dtype=np.uint16, mode="r")
        start = int(torch.randint(0, max(1, len(data) - a.prompt_len), (1,), generator=torch.Generator().manual_seed(a.seed)))
        prompt = [int(t) for t in data[start:start + a.prompt_len]]
    else:
        prompt = [50256]
    show = (lambda ids: tok.decode(ids)) if tok else (lambda ids: " ".join(map(str, ids)))
    print("[PROMPT]:", show(prompt))
    print("[GENERATED]: ", end="", flush=True)
    out = greedy_generate(g, prompt, a.num_tokens, eos=a.eos, seq_len=a.seq_len or model_seq_len(g),
                          on_token=lambda t: print(show([t]), end=" " if not tok else "", flush=True))
    print("\n\n[FULL TEXT]:\n" + show(out))
    return 0


def cmd_tcp_worker(a) -> int:
    """One pipeline stage behind a TCP endpoint (reference: examples/tcp_worker.cpp:39-141)."""
    from .parallel.tcp_transport import main as tcp_main

    dev = "cuda" if (a.gpu and torch.cuda.is_available()) else "cpu"
    return tcp_main(["worker", "--host", a.host, "--port", str(a.port), "--device", dev, "--sockets", str(a.sockets),
                     "--max-packet", str(a.max_packet)])


def cmd_tcp_coordinator(a) -> int:
    """Pipeline training driven from this process over TCP (reference: examples/tcp_coordinator.cpp:27-128 with the keys
    of configs/tcp_config.json): stage i goes to ``worker_endpoints[i]``; when ``local_worker_port`` is set, the last
    stage runs on a thread of this process behind that port."""
    import threading
    import time

    from .data.loaders import create_loaders
    from .models import zoo
    from .parallel.tcp_transport import TcpStageServer, tcp_coordinator

    cfg = _load_cfg(a.config)
    endpoints = [f"{w.get('host', '127.0.0.1')}:{int(w['port'])}" for w in cfg.worker_endpoints]
    local = None
    if cfg.local_worker_port:
        dev = "cuda" if (cfg.device_type.upper() == "CUDA" and torch.cuda.is_available()) else "cpu"
        srv = TcpStageServer(cfg.local_worker_host or cfg.host, cfg.local_worker_port, dev, cfg.skts_per_endpoint, cfg.max_packet_size)
        local = threading.Thread(target=srv.serve, daemon=True)
        local.start()
        endpoints.append(srv.name)
    ratios = list(cfg.partition_ratios or cfg.parallel.partition_ratios) or [1.0] * len(endpoints)
    if len(ratios) != len(endpoints):
        raise SystemExit(f"{len(ratios)} partition ratios for {len(endpoints)} workers")
    graph = zoo.create(cfg.model_name)
    co = tcp_coordinator(graph, ratios, endpoints, cfg.optimizer, cfg.scheduler, cfg.loss, cfg.num_microbatches,
                         cfg.host, cfg.port, cfg.skts_per_endpoint, cfg.max_packet_size)
    train, val = create_loaders(cfg.dataset_name, cfg.dataset_path, cfg.batch_size, cfg.seed,
                              cfg.prefetch_depth if cfg.prefetch_data else 0, cfg.model_name)
    co.broadcast("TRAIN_MODE", expect="MODE_CHANGED")
    steps = cfg.max_steps if cfg.max_steps and cfg.max_steps > 0 else cfg.epochs * train.batches_per_epoch()
    it, done, loss = iter(train), 0, float("nan")
    t0 = time.perf_counter()
    while done < steps:
        try:
            data, labels = next(it)
        except StopIteration:
            it = iter(train)
            continue
        loss = co.train_batch(data, labels)
        done += 1
        if done % max(1, cfg.progress_print_interval) == 0 or done == steps:
            print(f"step {done}/{steps} loss {loss:.4f} ({(time.perf_counter() - t0) / done * 1e3:.1f} ms/step)", flush=True)
    val_res = co.evaluate(val, max_batches=a.val_batches) if a.val_batches else {}
    if val_res:
        print(f"validation: loss {val_res['loss']:.4f} accuracy {val_res['accuracy_pct']:.2f} % over {val_res['batches']} batches", flush=True)
    if cfg.snapshot_dir:
        os.makedirs(cfg.snapshot_dir, exist_ok=True)
        from .parallel.stage_worker import simple_message
        for i, name in enumerate(co.names):  # each worker writes its own stage, on its own host
            co.post(name, simple_message("SAVE_TO_FILE", text=os.path.join(cfg.snapshot_dir, f"{cfg.model_name}_stage{i}.tnng")))
        co.broadcast("PRINT_LR", expect="LR_PRINTED")  # answered after the save
    co.shutdown()
    stats = co.transport.stats()
    co.transport.close()
    if local is not None:
        local.join(timeout=30)
    print(json.dumps({"steps": done, "final_loss": loss, "seconds": round(time.perf_counter() - t0, 3),
                      **{"val_" + k: v for k, v in val_res.items()}, **stats}))
    return 0


def cmd_info(a) -> int:
    from . import _build
    from .host import H
    from .models import zoo
    from .nn.layers import LAYER_REGISTRY

    print("kernel library :", _build.kernels_path(), "(present)" if os.path.exists(_build.kernels_path()) else "(not built)")
    print("hardware       :", json.dumps(H.hardware_info()))
    print("cuda devices   :", [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())])
    print("models         :", ", ".join(sorted(zoo.available_models())))
    print("layer types    :", ", ".join(sorted(LAYER_REGISTRY)))
    return 0


def main(argv=None) -> int:
    from .utils.env import EnvLoader, default_device_type
    EnvLoader("./.env")  # optional KEY=value file in the working directory, exported to the environment
    ap = argparse.ArgumentParser(prog="tnn_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("train", help="train from a JSON config (epoch or step mode)")
    p.add_argument("--config", "-c", required=True)
    p.add_argument("--layout", default="", help="parallel layout when launched under torchrun, e.g. dp8, tp2dp4, pp2")
    p = sub.add_parser("infer", help="validation loss / accuracy")
    p.add_argument("--config", "-c", required=True)
    p.add_argument("--max-batches", type=int, default=None)
    p = sub.add_parser("generate", help="greedy decoding with a GPT-2 style model")
    p.add_argument("--model", default="gpt2_small")
    p.add_argument("--model-path", default="")
    p.add_argument("--vocab", default="")
    p.add_argument("--tokens", default="", help="uint16 token file to cut the prompt from")
    p.add_argument("--prompt-ids", default="", help="comma separated token ids")
    p.add_argument("--prompt-len", type=int, default=30)
    p.add_argument("--num-tokens", type=int, default=50)
    p.add_argument("--seq-len", type=int, default=0)
    p.add_argument("--eos", type=int, default=50256)
    p.add_argument("--device", default=default_device_type(), help="CPU or CUDA (default: $DEVICE_TYPE, else CUDA when present)")
    p.add_argument("--seed", type=int, default=0)
    p = sub.add_parser("tcp-worker", help="serve one pipeline stage over TCP until the coordinator shuts it down")
    p.add_argument("port", type=int, nargs="?", default=0)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--gpu", action="store_true")
    p.add_argument("--sockets", type=int, default=4)
    p.add_argument("--max-packet", type=int, default=4 << 20)
    p = sub.add_parser("tcp-coordinator", help="partition a model and train it on TCP workers (keys of the reference's tcp_config.json)")
    p.add_argument("--config", "-c", required=True)
    p.add_argument("--val-batches", type=int, default=4, help="validation batches after training (0 = none)")
    sub.add_parser("info", help="build and device information")
    a = ap.parse_args(argv)
    return {"train": cmd_train, "infer": cmd_infer, "generate": cmd_generate, "info": cmd_info,
            "tcp-worker": cmd_tcp_worker, "tcp-coordinator": cmd_tcp_coordinator}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
