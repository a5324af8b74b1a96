"""Command line, examples and inference helpers on CPU."""
import importlib.util
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_graph_builder_example_trains_small_cnn():
    """The small CNN of the builder-API example (conv3x3-32 / ReLU / pool / conv3x3-64 / ... / dense-10, assembled with
    ``g.input``, layer calls, ``node + node`` and ``set_output``) learns a separable synthetic problem on CPU."""
    ex = _load(os.path.join(ROOT, "examples", "graph_api_mnist.py"), "graph_api_mnist")
    first, last = ex.main(steps=30, batch=16, device="cpu")
    assert last < 0.3 * first


def test_greedy_generate_slides_window_and_stops_at_eos():
    from tnn_b200.inference import greedy_generate, model_seq_len
    from tnn_b200.models import zoo

    g = zoo.gpt2(64, 1, 1, "tiny", seq_len=16, vocab=37, drop=0.0).compile(device="cpu", seed=1)
    assert model_seq_len(g) == 16
    out = greedy_generate(g, [1, 2, 3], num_new=20, eos=None)
    assert len(out) == 23 and all(0 <= t < 37 for t in out)
    # deterministic, and identical to a manual argmax of the padded forward pass
    x = torch.zeros(1, 16, dtype=torch.long)
    x[0, :3] = torch.tensor([1, 2, 3])
    g.set_training(False)
    logits = g.forward({"input": x})["output"][0, 2]
    assert out[3] == int(torch.argmax(logits))
    # eos stops generation right after it appears
    stop = out[3]
    assert greedy_generate(g, [1, 2, 3], num_new=20, eos=stop) == [1, 2, 3, stop]


def test_cli_train_and_infer_smoke(tmp_path):
    cfg = json.load(open(os.path.join(ROOT, "configs", "smoke_synthetic.json")))
    cfg.update(max_steps=3, snapshot_dir=str(tmp_path / "snap"))
    cfg["log_mode"]["log_dir"] = str(tmp_path / "logs")
    path = tmp_path / "cfg.json"
    path.write_text("// comments are allowed\n" + json.dumps(cfg))
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "tnn_b200", "train", "--config", str(path)], capture_output=True, text=True, env=env,
                       cwd=str(tmp_path), timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert "loss" in res
    r = subprocess.run([sys.executable, "-m", "tnn_b200", "infer", "--config", str(path), "--max-batches", "1"], capture_output=True,
                       text=True, env=env, cwd=str(tmp_path), timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "Validation Loss:" in r.stdout


def test_every_config_file_parses():
    from tnn_b200.utils.config import TrainingConfig

    for name in sorted(os.listdir(os.path.join(ROOT, "configs"))):
        if name.endswith(".json"):
            cfg = TrainingConfig.load_from_json(os.path.join(ROOT, "configs", name))
            assert cfg.batch_size > 0 and cfg.model_name


def test_layer_profiler_records_compute_events_and_log_lines(tmp_path):
    from tnn_b200.models import zoo
    from tnn_b200.trainer import Trainer
    from tnn_b200.utils.config import TrainingConfig

    zoo.register_model("tiny_prof", lambda: zoo.gpt2(64, 1, 2, "t", seq_len=16, vocab=37, drop=0.0))
    cfg = TrainingConfig.from_dict({"model_name": "tiny_prof", "batch_size": 2, "device_type": "CPU", "profiler_type": "CUMULATIVE",
                                    "optimizer": {"type": "sgd", "learning_rate": 0.01}})
    t = Trainer(cfg, log=False)
    seq = torch.randint(0, 37, (2, 17))
    for _ in range(2):
        t.train_step(seq[:, :-1].contiguous(), seq[:, 1:].contiguous())
    lp = t.layer_profiler
    names = {n for (n, _ph) in lp.totals}
    assert any("block_0" in n for n in names) and all(calls == 2 for _, calls in lp.totals.values())   # cumulative over 2 steps
    assert {ph for (_n, ph) in lp.totals} == {"forward", "backward"}
    table = lp.table()
    assert "fwd ms" in table and "total" in table
    log = lp.write_log(str(tmp_path / "profiler.log"))
    first = open(log).readline()
    assert first.startswith("Event: ") and "Type: COMPUTE" in first and "Duration:" in first
    from tnn_b200.utils.profiling import merge_across_ranks
    assert len(merge_across_ranks(lp)) == len(lp.profiler)      # single process: nothing to merge
    t.close()


def test_env_file_rules(tmp_path, monkeypatch):
    from tnn_b200.utils.env import EnvLoader, augmentation_enabled, default_device_type, from_str

    p = tmp_path / ".env"
    p.write_text("# comment\n\nDEVICE_TYPE = CPU   # trailing comment\nNAME=\"quoted # kept\"\nN=0x10\nRATE='0.5'\n"
                 "BAD KEY=1\nNOEQUALS\nAUGMENTATION=yes\n")
    for k in ("DEVICE_TYPE", "NAME", "N", "RATE", "AUGMENTATION", "BAD KEY"):
        monkeypatch.delenv(k, raising=False)
    env = EnvLoader(str(p))
    assert env.loaded and env.vars == {"DEVICE_TYPE": "CPU", "NAME": "quoted # kept", "N": "0x10", "RATE": "0.5", "AUGMENTATION": "yes"}
    import os
    assert os.environ["NAME"] == "quoted # kept"
    assert env.get("N", 0) == 16 and env.get("RATE", 0.0) == 0.5 and env.get("MISSING", 7) == 7
    assert default_device_type() == "CPU" and augmentation_enabled()
    assert from_str("TRUE", bool) and not from_str("off", bool)
    assert not EnvLoader(str(tmp_path / "nope.env")).loaded
    for k in env.vars:
        monkeypatch.delenv(k, raising=False)
