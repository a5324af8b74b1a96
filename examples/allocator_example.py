"""Device inventory and the two sub-allocators of the host runtime.

``PoolAllocator`` is a size-bucketed free list over one slab (the symmetric heap of the parallel runtime
sub-allocates with it); ``DoubleEndedArena`` hands out blocks from either end of a slab and flips sides, which
lets consecutive layers' activations alternate ends without fragmenting the middle.
Reference: examples/device_manager_example.cpp, examples/test_del.cpp."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.host import H  # noqa: E402

print("host:", json.dumps(H.hardware_info()))
print("devices:", ["CPU:0"] + [f"CUDA:{i} {torch.cuda.get_device_name(i)}" for i in range(torch.cuda.device_count())])

pool = H.PoolAllocator(1 << 20, 256)
a, b = pool.allocate(1000), pool.allocate(5000)
pool.release(a)
c = pool.allocate(900)  # reuses the released bucket
print("pool offsets", a, b, c, "used", pool.used(), "peak", pool.peak())

arena = H.DoubleEndedArena(1 << 20, 256)
x = arena.allocate(4096)
arena.flip()
y = arena.allocate(4096)  # comes from the other end
print("arena offsets", x, y, "side", arena.side(), "used", arena.used())
arena.release(x)
arena.release(y)
print("free blocks after release:", arena.free_blocks())
