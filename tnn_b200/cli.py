"""Command line: ``python -m tnn_b200 <command>``.

    train     --config x.json [--layout dp8|tp2dp4|pp2 ...]   single device, or one rank of a torchrun job
    infer     --config x.json                                  validation loss / accuracy of model_path or a fresh model
    generate  --model gpt2_small|--model-path f.tnng --vocab vocab.bin [--tokens train.bin]
    info                                                       devices, build status, registered models and layers

These are the counterparts of the reference's ``trainer``, ``inferencer`` and ``gpt2_inference`` binaries
(examples/trainer.cpp:15-85, examples/inferencer.cpp:12-70, examples/gpt2_inference.cpp:16-114); its
``tcp_coordinator`` / ``tcp_worker`` pair is replaced by launching ``train`` under ``torchrun`` with a
``--layout`` (one process per GPU, no coordinator process).
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
    sub.add_parser("info", help="build and device information")
    a = ap.parse_args(argv)
    return {"train": cmd_train, "infer": cmd_infer, "generate": cmd_generate, "info": cmd_info}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
