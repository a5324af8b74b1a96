"""List the devices the framework can run on, the way the reference's device-manager demo does
(examples/device_manager_example.cpp; devices keyed "CPU:0", "CUDA:i" in src/device/device_manager.cpp:22-62), and
move a tensor across them. Device, stream and memory management belong to PyTorch here; the host runtime adds
the hardware summary and rank pinning (``H.hardware_info``, ``H.pin_rank``)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.host import H  # noqa: E402


def devices():
    out = {"CPU:0": torch.device("cpu")}
    for i in range(torch.cuda.device_count()):
        out[f"CUDA:{i}"] = torch.device("cuda", i)
    return out


def main():
    info = H.hardware_info()
    print("host:", {k: info[k] for k in sorted(info)} if isinstance(info, dict) else info)
    devs = devices()
    for name, d in devs.items():
        if d.type == "cuda":
            p = torch.cuda.get_device_properties(d)
            free, total = torch.cuda.mem_get_info(d)
            print(f"{name}: {p.name}, sm_{p.major}{p.minor}, {p.multi_processor_count} SMs, {total >> 20} MiB ({free >> 20} free)")
        else:
            print(f"{name}: {os.cpu_count()} logical cores, {torch.get_num_threads()} compute threads")
    x = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    for name, d in devs.items():
        y = x.to(d)
        assert torch.equal(y.cpu(), x)
        print(f"copied a {tuple(x.shape)} tensor to {name} and back")
    return list(devs)


if __name__ == "__main__":
    main()
