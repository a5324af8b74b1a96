"""Directory-of-JPEG datasets: Tiny-ImageNet (``wnids.txt``, ``train/<wnid>/images``,
``val/val_annotations.txt``) and ImageNet-100 (``Labels.json`` + class folders, resize-256 /
center-crop-224 for validation, random-resized-crop for training, mean/std normalisation) -
reference: include/data_loading/{tiny_imagenet,imagenet100}_data_loader.hpp. Decoding uses PIL
when it is importable; without it these loaders raise at construction."""
from __future__ import annotations

import json
import os
import random
from typing import List, Tuple

import numpy as np
import torch

from .loaders import BaseLoader

MEAN = np.array([0.485, 0.456, 0.406], dtype=np.float32)
STD = np.array([0.229, 0.224, 0.225], dtype=np.float32)


def _pil():
    try:
        from PIL import Image
        return Image
    except Exception as e:  # pragma: no cover
        raise RuntimeError("image-folder datasets need Pillow to decode JPEG files") from e


class ImageFolderLoader(BaseLoader):
    def __init__(self, items: List[Tuple[str, int]], batch: int, side: int, train: bool, seed: int, normalize: bool,
                 augmentation=None):
        self.items, self.batch, self.side, self.train = items, batch, side, train
        self.rng = random.Random(seed)
        self.normalize, self.aug = normalize, augmentation
        self.Image = _pil()
        self.order = list(range(len(items)))
        self.cur = 0

    def __len__(self):
        return len(self.items)

    def batches_per_epoch(self):
        return len(self.items) // self.batch

    def reset(self):
        if self.train:
            self.rng.shuffle(self.order)
        self.cur = 0

    def _load(self, path):
        im = self.Image.open(path).convert("RGB")
        s = self.side
        if s >= 224:
            if self.train:
                w, h = im.size
                area = w * h * self.rng.uniform(0.08, 1.0)
                ar = self.rng.uniform(3 / 4, 4 / 3)
                cw, ch = min(w, int(round((area * ar) ** 0.5))), min(h, int(round((area / ar) ** 0.5)))
                x0, y0 = self.rng.randint(0, w - cw), self.rng.randint(0, h - ch)
                im = im.crop((x0, y0, x0 + cw, y0 + ch)).resize((s, s))
                if self.rng.random() < 0.5:
                    im = im.transpose(self.Image.FLIP_LEFT_RIGHT)
            else:
                w, h = im.size
                sc = 256 / min(w, h)
                im = im.resize((max(s, int(w * sc)), max(s, int(h * sc))))
                w, h = im.size
                im = im.crop(((w - s) // 2, (h - s) // 2, (w - s) // 2 + s, (h - s) // 2 + s))
        elif im.size != (s, s):
            im = im.resize((s, s))
        a = np.asarray(im, dtype=np.float32) / 255.0
        if self.normalize:
            a = (a - MEAN) / STD
        return a

    def next_batch(self):
        if self.cur + self.batch > len(self.order):
            return None
        idx = self.order[self.cur:self.cur + self.batch]
        self.cur += self.batch
        data = torch.from_numpy(np.stack([self._load(self.items[i][0]) for i in idx]))
        labels = torch.tensor([self.items[i][1] for i in idx], dtype=torch.int64)
        if self.aug is not None and self.train:
            data = self.aug(data)
        return data, labels


def create_image_folder_loaders(name, path, batch, seed, augmentation):
    if name == "tiny_imagenet":
        wnids = [l.strip() for l in open(os.path.join(path, "wnids.txt")) if l.strip()]
        cls = {w: i for i, w in enumerate(wnids)}
        train = []
        for w in wnids:
            d = os.path.join(path, "train", w, "images")
            train += [(os.path.join(d, f), cls[w]) for f in sorted(os.listdir(d))] if os.path.isdir(d) else []
        val = []
        ann = os.path.join(path, "val", "val_annotations.txt")
        if os.path.exists(ann):
            for l in open(ann):
                parts = l.split("\t")
                if len(parts) >= 2 and parts[1] in cls:
                    val.append((os.path.join(path, "val", "images", parts[0]), cls[parts[1]]))
        return (ImageFolderLoader(train, batch, 64, True, seed, False, augmentation),
                ImageFolderLoader(val, batch, 64, False, seed, False))
    if augmentation is None:
        # the reference switches its ImageNet-100 augmentation (flip, brightness, contrast, saturation) on with the
        # AUGMENTATION / tunx_AUGMENTATION environment variable (src/data_loading/data_loading.cpp:93-124)
        from ..utils.env import augmentation_enabled
        if augmentation_enabled():
            from .augmentation import AugmentationBuilder
            augmentation = AugmentationBuilder(seed).horizontal_flip(0.5).brightness(0.5, 0.2).contrast(0.5, 0.2).saturation(0.5, 0.2).build()
    labels = json.load(open(os.path.join(path, "Labels.json")))
    cls = {w: i for i, w in enumerate(sorted(labels))}
    train, val = [], []
    for sub in sorted(os.listdir(path)):
        d = os.path.join(path, sub)
        if not os.path.isdir(d):
            continue
        for w in sorted(os.listdir(d)):
            if w in cls and os.path.isdir(os.path.join(d, w)):
                items = [(os.path.join(d, w, f), cls[w]) for f in sorted(os.listdir(os.path.join(d, w)))]
                (val if sub.startswith("val") else train).extend(items)
    return (ImageFolderLoader(train, batch, 224, True, seed, True, augmentation),
            ImageFolderLoader(val, batch, 224, False, seed, True))
