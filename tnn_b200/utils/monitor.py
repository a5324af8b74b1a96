"""GPU / NVLink / NIC telemetry sampler that appends one CSV row per interval.

    python -m tnn_b200.utils.monitor --csv logs/telemetry.csv --gpu 0 --interval 1.0 [--iface eth0] [--duration 60]

The B200 counterpart of the reference's ``torch/monitor_net_gpu.py`` (NIC and RDMA byte counters from sysfs plus
``nvidia-smi`` utilisation, written to CSV while a distributed run is going on). On one NVSwitch box the traffic that
matters is on NVLink, so the sampler reads the per-GPU NVLink transmit / receive byte counters through NVML
(``nvidia_ml_py``) when the driver exposes them, next to SM / memory utilisation, clocks, power, temperature, memory
in use and the clock-event reasons; the network-interface columns are kept for runs that do use a NIC. It only reads
- it never changes a setting of the GPU. ``nvidia-smi`` is the fallback when NVML cannot be loaded.
"""
from __future__ import annotations

import argparse
import csv
import os
import signal
import subprocess
import time
from typing import Dict, Optional

_STOP = False


def _handle(signum, frame):
    global _STOP
    _STOP = True


def read_int(path: str) -> Optional[int]:
    try:
        with open(path) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return None


def read_net_counters(iface: str) -> Dict[str, Optional[int]]:
    base = f"/sys/class/net/{iface}/statistics"
    return {"net_rx_bytes": read_int(f"{base}/rx_bytes"), "net_tx_bytes": read_int(f"{base}/tx_bytes")}


class NvmlReader:
    """Reads one GPU through NVML; every field that the driver refuses is reported as empty."""

    def __init__(self, index: int):
        import pynvml  # provided by nvidia_ml_py

        self.nv = pynvml
        pynvml.nvmlInit()
        self.h = pynvml.nvmlDeviceGetHandleByIndex(index)

    def _try(self, fn, *a):
        try:
            return fn(self.h, *a)
        except Exception:
            return None

    def sample(self) -> Dict[str, object]:
        nv = self.nv
        util = self._try(nv.nvmlDeviceGetUtilizationRates)
        mem = self._try(nv.nvmlDeviceGetMemoryInfo)
        power = self._try(nv.nvmlDeviceGetPowerUsage)
        row = {
            "gpu_util_pct": getattr(util, "gpu", None), "mem_util_pct": getattr(util, "memory", None),
            "mem_used_mib": (mem.used >> 20) if mem else None,
            "sm_mhz": self._try(nv.nvmlDeviceGetClockInfo, nv.NVML_CLOCK_SM),
            "mem_mhz": self._try(nv.nvmlDeviceGetClockInfo, nv.NVML_CLOCK_MEM),
            "power_w": round(power / 1000.0, 1) if power is not None else None,
            "temp_c": self._try(nv.nvmlDeviceGetTemperature, nv.NVML_TEMPERATURE_GPU),
            "clock_event_reasons": self._try(nv.nvmlDeviceGetCurrentClocksEventReasons)
            if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") else self._try(nv.nvmlDeviceGetCurrentClocksThrottleReasons),
        }
        tx = rx = None
        fid_tx = getattr(nv, "NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX", None)
        fid_rx = getattr(nv, "NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX", None)
        if fid_tx is not None and fid_rx is not None:
            try:
                vals = nv.nvmlDeviceGetFieldValues(self.h, [fid_tx, fid_rx])
                tx, rx = (int(v.value.ullVal) if v.nvmlReturn == 0 else None for v in vals)  # KiB since driver load
            except Exception:
                pass
        row["nvlink_tx_kib"], row["nvlink_rx_kib"] = tx, rx
        return row

    def close(self):
        try:
            self.nv.nvmlShutdown()
        except Exception:
            pass


def smi_sample(index: int) -> Dict[str, object]:
    q = "utilization.gpu,utilization.memory,memory.used,clocks.sm,clocks.mem,power.draw,temperature.gpu"
    try:
        out = subprocess.run(["nvidia-smi", "-i", str(index), f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=10).stdout.strip().split(",")
        vals = [x.strip() for x in out]
        keys = ["gpu_util_pct", "mem_util_pct", "mem_used_mib", "sm_mhz", "mem_mhz", "power_w", "temp_c"]
        return dict(zip(keys, vals))
    except Exception:
        return {}


FIELDS = ["timestamp", "elapsed_s", "gpu", "gpu_util_pct", "mem_util_pct", "mem_used_mib", "sm_mhz", "mem_mhz", "power_w", "temp_c",
          "clock_event_reasons", "nvlink_tx_kib", "nvlink_rx_kib", "nvlink_tx_gbs", "nvlink_rx_gbs", "net_rx_bytes", "net_tx_bytes",
          "net_rx_mbs", "net_tx_mbs"]


def run(csv_path: str, gpu: int, interval: float, iface: Optional[str] = None, duration: Optional[float] = None,
        reader=None, clock=time.time, sleep=time.sleep) -> int:
    """Sampling loop; ``reader`` (an object with ``sample()``) can be injected, which is how the tests fake NVML."""
    os.makedirs(os.path.dirname(os.path.abspath(csv_path)), exist_ok=True)
    if reader is None:
        try:
            reader = NvmlReader(gpu)
        except Exception:
            reader = None
    new = not os.path.exists(csv_path)
    rows = 0
    t0 = clock()
    prev: Dict[str, object] = {}
    prev_t = t0
    with open(csv_path, "a", newline="") as f:
        w = csv.DictWriter(f, fieldnames=FIELDS)
        if new:
            w.writeheader()
        while not _STOP:
            now = clock()
            row: Dict[str, object] = {"timestamp": round(now, 3), "elapsed_s": round(now - t0, 3), "gpu": gpu}
            row.update(reader.sample() if reader is not None else smi_sample(gpu))
            if iface:
                row.update(read_net_counters(iface))
            dt = now - prev_t
            if prev and dt > 0:  # rates from counter differences
                for key, out, scale in (("nvlink_tx_kib", "nvlink_tx_gbs", 1024 / 1e9), ("nvlink_rx_kib", "nvlink_rx_gbs", 1024 / 1e9),
                                        ("net_rx_bytes", "net_rx_mbs", 1e-6), ("net_tx_bytes", "net_tx_mbs", 1e-6)):
                    a, b = prev.get(key), row.get(key)
                    if isinstance(a, int) and isinstance(b, int):
                        row[out] = round((b - a) * scale / dt, 3)
            w.writerow({k: ("" if row.get(k) is None else row.get(k)) for k in FIELDS})
            f.flush()
            rows += 1
            prev, prev_t = row, now
            if duration is not None and now - t0 >= duration:
                break
            sleep(interval)
    if reader is not None and hasattr(reader, "close"):
        reader.close()
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--csv", required=True)
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--interval", type=float, default=1.0)
    ap.add_argument("--iface", default=None, help="network interface whose byte counters to record")
    ap.add_argument("--duration", type=float, default=None, help="stop after this many seconds (default: until SIGINT / SIGTERM)")
    a = ap.parse_args(argv)
    if a.iface and not os.path.exists(f"/sys/class/net/{a.iface}"):
        raise SystemExit(f"no such network interface: {a.iface}")
    signal.signal(signal.SIGINT, _handle)
    signal.signal(signal.SIGTERM, _handle)
    n = run(a.csv, a.gpu, a.interval, a.iface, a.duration)
    print(f"{n} samples -> {a.csv}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
