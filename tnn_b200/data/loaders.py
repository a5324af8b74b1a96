"""Data loaders. All emit channels-last float images (or int64 token ids) on the host plus
integer labels, like the reference loaders (include/data_loading/*.hpp). The file-backed ones run
in C++ (``host.H.Loader``) with a background prefetch thread; ``synthetic`` produces tensors of a
model's input shape in pinned host memory for benchmarks.
"""
from __future__ import annotations

import glob
import json
import os
from typing import Iterator, Optional, Tuple

import numpy as np
import torch

from ..host import H


class BaseLoader:
    """Iterator of ``(data, labels)`` host tensors; ``reset()`` starts a new (reshuffled) epoch."""

    def __len__(self) -> int:
        raise NotImplementedError

    def batches_per_epoch(self) -> int:
        raise NotImplementedError

    def reset(self) -> None:
        pass

    def next_batch(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        raise NotImplementedError

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        self.reset()
        while True:
            b = self.next_batch()
            if b is None:
                return
            yield b


class SyntheticLoader(BaseLoader):
    """Random tensors of a given shape: N(0,1) images (or uniform [0,1) with ``uniform=True``) with
    uniform integer labels, or uniform token ids with next-token labels. Batches are generated into
    a small ring of pinned buffers so that the host-to-device copy is a true pinned transfer."""

    def __init__(self, sample_shape, num_classes: int, batch_size: int, steps_per_epoch: int = 100, tokens: bool = False,
                 uniform: bool = False, seed: int = 0, pin: bool = True, ring: int = 4, dtype: torch.dtype = torch.float32):
        self.shape, self.num_classes, self.batch = tuple(sample_shape), int(num_classes), int(batch_size)
        self.steps, self.tokens, self.uniform = int(steps_per_epoch), tokens, uniform
        self.gen = torch.Generator().manual_seed(seed)
        pin = pin and torch.cuda.is_available()
        self.ring = []
        for _ in range(ring):
            if tokens:
                d = torch.empty((self.batch,) + self.shape, dtype=torch.int64)
                l = torch.empty((self.batch,) + self.shape, dtype=torch.int64)
            else:
                d = torch.empty((self.batch,) + self.shape, dtype=dtype)  # images in the model's io dtype, like the reference loaders
                l = torch.empty((self.batch,), dtype=torch.int64)
            self.ring.append((d.pin_memory() if pin else d, l.pin_memory() if pin else l))
        self.i = 0
        # the ring is filled once: generating tens of millions of random numbers per step on the host
        # would time the random generator, not the input pipeline
        for d, l in self.ring:
            self._fill(d, l)

    def _fill(self, d, l):
        if self.tokens:
            seq = torch.randint(0, self.num_classes, (self.batch, self.shape[0] + 1), generator=self.gen)
            d.copy_(seq[:, :-1])
            l.copy_(seq[:, 1:])
        else:
            d.copy_(torch.rand(d.shape, generator=self.gen) if self.uniform else torch.randn(d.shape, generator=self.gen))
            l.copy_(torch.randint(0, self.num_classes, (self.batch,), generator=self.gen))

    def __len__(self):
        return self.steps * self.batch

    def batches_per_epoch(self):
        return self.steps

    def reset(self):
        self.i = 0

    def next_batch(self):
        if self.i >= self.steps:
            return None
        d, l = self.ring[self.i % len(self.ring)]
        self.i += 1
        return d, l


class NativeLoader(BaseLoader):
    """Wraps a C++ ``Loader`` (CIFAR-10/100 binaries, MNIST CSV, uint16 token streams)."""

    def __init__(self, native, tokens: bool = False, transform=None):
        self.native, self.tokens, self.transform = native, tokens, transform

    def __len__(self):
        return len(self.native)

    def batches_per_epoch(self):
        return self.native.batches_per_epoch()

    def reset(self):
        self.native.reset()

    def next_batch(self):
        b = self.native.next()
        if b is None:
            return None
        data, labels = torch.from_numpy(b[0]), torch.from_numpy(b[1]).long()
        if self.tokens:
            data = data.long()
        elif self.transform is not None:
            data = self.transform(data)
        return data, labels


def _first_existing(folder, names):
    for n in names:
        p = os.path.join(folder, n)
        if os.path.exists(p):
            return p
    raise FileNotFoundError(f"none of {names} in {folder}")


def create_loaders(name: str, path: str, batch_size: int, seed: int = 0, prefetch_depth: int = 2, model_name: str = "",
                   augmentation=None, steps_per_epoch: int = 100):
    """``(train_loader, val_loader)`` for a dataset name of the reference's factory
    (src/data_loading/data_loading.cpp:38-124) or ``synthetic``."""
    from ..models.zoo import INPUT_SHAPES
    name = (name or "synthetic").lower()
    if name == "synthetic" or not path or not os.path.exists(path):
        if model_name and "gpt2" in model_name:
            mk = lambda s: SyntheticLoader((1024,), 50257, batch_size, steps_per_epoch, tokens=True, seed=s)
        else:
            shape = INPUT_SHAPES.get(model_name, (28, 28, 1))
            classes = {"mnist_cnn": 10, "imagenet_resnet50": 1000}.get(model_name, 10 if "cifar10_" in model_name else 100 if ("cifar100" in model_name or "imagenet100" in model_name) else 200)
            mk = lambda s: SyntheticLoader(shape, classes, batch_size, steps_per_epoch, seed=s)
        return mk(seed), mk(seed + 1)
    if name == "mnist":
        tr = _first_existing(path, ["train.csv", "mnist_train.csv"])
        te = _first_existing(path, ["test.csv", "mnist_test.csv"])
        return (NativeLoader(H.Loader.mnist_csv(tr, batch_size, True, seed, prefetch_depth), transform=augmentation),
                NativeLoader(H.Loader.mnist_csv(te, batch_size, False, seed, prefetch_depth)))
    if name == "cifar10":
        tr = sorted(glob.glob(os.path.join(path, "data_batch_*.bin")))
        te = [os.path.join(path, "test_batch.bin")]
        return (NativeLoader(H.Loader.cifar10(tr, batch_size, True, seed, prefetch_depth), transform=augmentation),
                NativeLoader(H.Loader.cifar10(te, batch_size, False, seed, prefetch_depth)))
    if name == "cifar100":
        return (NativeLoader(H.Loader.cifar100([os.path.join(path, "train.bin")], False, batch_size, True, seed, prefetch_depth),
                             transform=augmentation),
                NativeLoader(H.Loader.cifar100([os.path.join(path, "test.bin")], False, batch_size, False, seed, prefetch_depth)))
    if name == "open_webtext":
        return (NativeLoader(H.Loader.tokens(os.path.join(path, "train.bin"), 1024, batch_size, seed, prefetch_depth), tokens=True),
                NativeLoader(H.Loader.tokens(os.path.join(path, "val.bin"), 1024, batch_size, seed + 1, prefetch_depth), tokens=True))
    if name in ("tiny_imagenet", "imagenet100"):
        from .image_folder import create_image_folder_loaders
        return create_image_folder_loaders(name, path, batch_size, seed, augmentation)
    raise ValueError(f"unknown dataset {name!r}")
