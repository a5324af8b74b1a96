"""Telemetry sampler (against a fake NVML reader: it only ever reads) and the profiler timeline export."""
import csv
import json

import torch


class FakeReader:
    """Stands in for NVML: counters that grow by a known amount per sample."""

    def __init__(self):
        self.n = 0
        self.closed = False

    def sample(self):
        self.n += 1
        return {"gpu_util_pct": 90 + self.n, "mem_util_pct": 40, "mem_used_mib": 1000 * self.n, "sm_mhz": 1965, "mem_mhz": 3996,
                "power_w": 700.5, "temp_c": 55, "clock_event_reasons": 4, "nvlink_tx_kib": 1_000_000 * self.n,
                "nvlink_rx_kib": 2_000_000 * self.n}

    def close(self):
        self.closed = True


def test_monitor_writes_rows_and_rates(tmp_path):
    from tnn_b200.utils import monitor

    t = [100.0]
    path = str(tmp_path / "logs" / "telemetry.csv")
    rd = FakeReader()
    n = monitor.run(path, gpu=3, interval=1.0, duration=2.0, reader=rd, clock=lambda: t[0], sleep=lambda s: t.__setitem__(0, t[0] + s))
    assert n == 3 and rd.closed
    rows = list(csv.DictReader(open(path)))
    assert [r["gpu"] for r in rows] == ["3"] * 3 and rows[0]["nvlink_tx_gbs"] == ""
    # 1e6 KiB per second = 1.024 GB/s; twice that on the receive side
    assert abs(float(rows[1]["nvlink_tx_gbs"]) - 1.024) < 1e-6 and abs(float(rows[2]["nvlink_rx_gbs"]) - 2.048) < 1e-6
    assert rows[2]["sm_mhz"] == "1965" and rows[2]["clock_event_reasons"] == "4"
    # a second run appends without repeating the header
    monitor.run(path, gpu=3, interval=1.0, duration=0.0, reader=FakeReader(), clock=lambda: t[0], sleep=lambda s: None)
    assert len(list(csv.DictReader(open(path)))) == 4


def test_profile_timeline_from_layer_profiler(tmp_path):
    from tnn_b200.models import zoo
    from tnn_b200.utils import profile_timeline
    from tnn_b200.utils.profiling import LayerProfiler

    g = zoo.create("mnist_cnn").compile(device="cpu", seed=0)
    prof = LayerProfiler(torch.device("cpu"), source="rank0")
    g.profiler = prof
    g.train()
    prof.begin_step()
    y = g(torch.rand(2, 28, 28, 1))
    g.backward({"output": torch.ones_like(y)})
    prof.end_step()
    log = prof.write_log(str(tmp_path / "profiler.log"))
    # plus a line in the reference coordinator's shape (no event name in front)
    with open(log, "a") as f:
        f.write("[info] Source: worker1, Type: COMMUNICATION, Start: 1.500 ms, End: 2.750 ms, Duration: 1.250 ms\n")
    ev = profile_timeline.parse_log(log)
    assert set(ev) == {"rank0", "worker1"} and "COMPUTE" in ev["rank0"]
    assert ev["worker1"]["COMMUNICATION"] == [("COMMUNICATION", 1.5, 1.25)]
    names = {n for n, _, _ in ev["rank0"]["COMPUTE"]}
    assert any(n.endswith(":forward") for n in names) and any(n.endswith(":backward") for n in names)
    out = str(tmp_path / "trace.json")
    assert profile_timeline.main([log, "--trace", out]) == 0
    tr = json.load(open(out))["traceEvents"]
    assert sum(1 for e in tr if e["ph"] == "X") == sum(len(v) for s in ev.values() for v in s.values())
    assert {e["args"]["name"] for e in tr if e["ph"] == "M" and e["name"] == "process_name"} == {"rank0", "worker1"}


def test_compare_logs_throughput_and_loss(tmp_path):
    """Two log dialects (this framework's batch CSV, the reference PyTorch trainer's phase-tagged log), the
    reference's throughput and TFLOP/s arithmetic, rolling-mean loss, and the merged per-step series."""
    import csv
    import json as _json

    from tnn_b200.utils import compare_logs as cl
    from tnn_b200.utils.csv_logger import CsvLogger

    lg = CsvLogger(str(tmp_path), "resnet50")
    for i in range(10):
        lg.log_train_step(epoch=0, step=i, batch_loss=2.0 - 0.1 * i, avg_loss=2.0, accuracy_pct=10.0 + i, time_ms=50.0 if i else 500.0)
    lg.close()
    ours = lg.paths["batch"]
    theirs = tmp_path / "torch.csv"
    with open(theirs, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["phase", "epoch", "step", "batch_loss", "avg_loss", "accuracy_percent", "batch_total_time", "batch_size"])
        for i in range(6):
            w.writerow(["train_batch", 0, i, 3.0, 3.0, 5.0, 0.2, 64])
        w.writerow(["validation", 0, 0, "", "", "", "", ""])
        w.writerow(["train_batch", 0, 6, "broken", "", "", "", ""])
    a = cl.summarize(ours, 256, gflop_per_sample=cl.GFLOP_PER_SAMPLE["resnet50"], skip=1, smooth=3)
    assert a["steps"] == 10 and a["median_ms"] == 50.0 and a["throughput"] == 5120.0
    assert abs(a["tflops"] - 256 * 12.3 / 0.05 / 1e3) < 0.01
    assert abs(a["final_loss_smoothed"] - (1.3 + 1.2 + 1.1) / 3) < 1e-4 and a["first_loss"] == 2.0
    b = cl.summarize(str(theirs), 128)  # the file's own batch_size column wins; seconds become milliseconds
    assert b["steps"] == 6 and b["batch_size"] == 64 and b["median_ms"] == 200.0 and b["throughput"] == 320.0
    assert cl.rolling_mean([1, 2, 3, 4], 2) == [1.0, 1.5, 2.5, 3.5]
    out = tmp_path / "series.csv"
    assert cl.main([ours, str(theirs), "--batch-size", "256", "--model", "resnet50", "--skip", "1", "--series-csv", str(out)]) == 0
    rows = list(csv.reader(open(out)))
    assert len(rows) == 11 and rows[0][0] == "global_step" and rows[7][3] == "" and float(rows[1][1]) == 2.0
    # language-model form: tokens per second
    c = cl.summarize(ours, 8, samples_per_item=1024, gflop_per_sample=cl.GFLOP_PER_SAMPLE["gpt2_small"], skip=1)
    assert c["throughput"] == 8 * 1024 / 0.05 and _json.dumps(c)
