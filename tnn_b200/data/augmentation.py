"""Batch augmentations on NHWC float tensors with a builder, mirroring the reference's set
(include/data_augmentation/augmentation.hpp:108 and siblings): horizontal / vertical flip,
rotation, brightness, contrast, saturation, gaussian noise, random crop, random-resized crop,
resize-center-crop, cutout, normalize. Each op has a probability ``p`` and draws per-sample."""
from __future__ import annotations

import math
from typing import Callable, List, Sequence

import torch
import torch.nn.functional as F


class Augmentation:
    def __init__(self, p: float = 1.0):
        self.p = p

    def pick(self, n, gen):
        return torch.rand(n, generator=gen) < self.p

    def __call__(self, x: torch.Tensor, gen: torch.Generator) -> torch.Tensor:
        raise NotImplementedError


class HorizontalFlip(Augmentation):
    def __call__(self, x, gen):
        m = self.pick(x.shape[0], gen)
        x = x.clone()
        x[m] = x[m].flip(2)
        return x


class VerticalFlip(Augmentation):
    def __call__(self, x, gen):
        m = self.pick(x.shape[0], gen)
        x = x.clone()
        x[m] = x[m].flip(1)
        return x


class Rotation(Augmentation):
    def __init__(self, p=0.5, max_degrees=15.0):
        super().__init__(p)
        self.deg = max_degrees

    def __call__(self, x, gen):
        n = x.shape[0]
        ang = (torch.rand(n, generator=gen) * 2 - 1) * math.radians(self.deg) * self.pick(n, gen)
        c, s = torch.cos(ang), torch.sin(ang)
        theta = torch.stack([torch.stack([c, -s, torch.zeros(n)], 1), torch.stack([s, c, torch.zeros(n)], 1)], 1)
        nchw = x.permute(0, 3, 1, 2)
        grid = F.affine_grid(theta, list(nchw.shape), align_corners=False)
        return F.grid_sample(nchw, grid, padding_mode="zeros", align_corners=False).permute(0, 2, 3, 1).contiguous()


class Brightness(Augmentation):
    def __init__(self, p=0.5, delta=0.2):
        super().__init__(p)
        self.delta = delta

    def __call__(self, x, gen):
        n = x.shape[0]
        f = 1 + (torch.rand(n, generator=gen) * 2 - 1) * self.delta * self.pick(n, gen)
        return x * f.view(n, 1, 1, 1)


class Contrast(Augmentation):
    def __init__(self, p=0.5, delta=0.2):
        super().__init__(p)
        self.delta = delta

    def __call__(self, x, gen):
        n = x.shape[0]
        f = (1 + (torch.rand(n, generator=gen) * 2 - 1) * self.delta * self.pick(n, gen)).view(n, 1, 1, 1)
        mean = x.mean((1, 2, 3), keepdim=True)
        return (x - mean) * f + mean


class Saturation(Augmentation):
    def __init__(self, p=0.5, delta=0.2):
        super().__init__(p)
        self.delta = delta

    def __call__(self, x, gen):
        if x.shape[-1] != 3:
            return x
        n = x.shape[0]
        f = (1 + (torch.rand(n, generator=gen) * 2 - 1) * self.delta * self.pick(n, gen)).view(n, 1, 1, 1)
        gray = (x * torch.tensor([0.299, 0.587, 0.114])).sum(-1, keepdim=True)
        return (x - gray) * f + gray


class GaussianNoise(Augmentation):
    def __init__(self, p=0.5, std=0.05):
        super().__init__(p)
        self.std = std

    def __call__(self, x, gen):
        m = self.pick(x.shape[0], gen).view(-1, 1, 1, 1)
        return x + torch.randn(x.shape, generator=gen) * self.std * m


class RandomCrop(Augmentation):
    def __init__(self, p=1.0, padding=4):
        super().__init__(p)
        self.pad = padding

    def __call__(self, x, gen):
        n, h, w, _ = x.shape
        xp = F.pad(x, (0, 0, self.pad, self.pad, self.pad, self.pad))
        out = x.clone()
        m = self.pick(n, gen)
        for i in range(n):
            if m[i]:
                dy, dx = (int(torch.randint(0, 2 * self.pad + 1, (1,), generator=gen)) for _ in range(2))
                out[i] = xp[i, dy:dy + h, dx:dx + w]
        return out


class RandomResizedCrop(Augmentation):
    def __init__(self, p=1.0, scale=(0.08, 1.0), ratio=(3 / 4, 4 / 3)):
        super().__init__(p)
        self.scale, self.ratio = scale, ratio

    def __call__(self, x, gen):
        n, h, w, _ = x.shape
        out = x.clone()
        m = self.pick(n, gen)
        for i in range(n):
            if not m[i]:
                continue
            area = h * w * float(torch.empty(1).uniform_(*self.scale, generator=gen))
            ar = float(torch.empty(1).uniform_(*self.ratio, generator=gen))
            cw, ch = max(1, min(w, int(round((area * ar) ** 0.5)))), max(1, min(h, int(round((area / ar) ** 0.5))))
            x0 = int(torch.randint(0, w - cw + 1, (1,), generator=gen))
            y0 = int(torch.randint(0, h - ch + 1, (1,), generator=gen))
            crop = x[i:i + 1, y0:y0 + ch, x0:x0 + cw].permute(0, 3, 1, 2)
            out[i] = F.interpolate(crop, size=(h, w), mode="bilinear", align_corners=False)[0].permute(1, 2, 0)
        return out


class ResizeCenterCrop(Augmentation):
    def __init__(self, resize: int, crop: int):
        super().__init__(1.0)
        self.resize, self.crop = resize, crop

    def __call__(self, x, gen):
        nchw = F.interpolate(x.permute(0, 3, 1, 2), size=(self.resize, self.resize), mode="bilinear", align_corners=False)
        o = (self.resize - self.crop) // 2
        return nchw[:, :, o:o + self.crop, o:o + self.crop].permute(0, 2, 3, 1).contiguous()


class Cutout(Augmentation):
    def __init__(self, p=0.5, size=8):
        super().__init__(p)
        self.size = size

    def __call__(self, x, gen):
        n, h, w, _ = x.shape
        out = x.clone()
        m = self.pick(n, gen)
        for i in range(n):
            if m[i]:
                cy, cx = int(torch.randint(0, h, (1,), generator=gen)), int(torch.randint(0, w, (1,), generator=gen))
                out[i, max(0, cy - self.size // 2):cy + self.size // 2, max(0, cx - self.size // 2):cx + self.size // 2] = 0
        return out


class Normalize(Augmentation):
    def __init__(self, mean: Sequence[float], std: Sequence[float]):
        super().__init__(1.0)
        self.mean, self.std = torch.tensor(mean), torch.tensor(std)

    def __call__(self, x, gen):
        return (x - self.mean) / self.std


class AugmentationPipeline:
    def __init__(self, ops: List[Augmentation], seed: int = 0):
        self.ops, self.gen = ops, torch.Generator().manual_seed(seed)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        for op in self.ops:
            x = op(x, self.gen)
        return x


class AugmentationBuilder:
    """``AugmentationBuilder().horizontal_flip(0.5).random_crop(1.0, 4).normalize(m, s).build()``"""

    def __init__(self, seed: int = 0):
        self.ops: List[Augmentation] = []
        self.seed = seed

    def _add(self, op):
        self.ops.append(op)
        return self

    def horizontal_flip(self, p=0.5): return self._add(HorizontalFlip(p))
    def vertical_flip(self, p=0.5): return self._add(VerticalFlip(p))
    def rotation(self, p=0.5, max_degrees=15.0): return self._add(Rotation(p, max_degrees))
    def brightness(self, p=0.5, delta=0.2): return self._add(Brightness(p, delta))
    def contrast(self, p=0.5, delta=0.2): return self._add(Contrast(p, delta))
    def saturation(self, p=0.5, delta=0.2): return self._add(Saturation(p, delta))
    def gaussian_noise(self, p=0.5, std=0.05): return self._add(GaussianNoise(p, std))
    def random_crop(self, p=1.0, padding=4): return self._add(RandomCrop(p, padding))
    def random_resized_crop(self, p=1.0, scale=(0.08, 1.0), ratio=(3 / 4, 4 / 3)): return self._add(RandomResizedCrop(p, scale, ratio))
    def resize_center_crop(self, resize, crop): return self._add(ResizeCenterCrop(resize, crop))
    def cutout(self, p=0.5, size=8): return self._add(Cutout(p, size))
    def normalize(self, mean, std): return self._add(Normalize(mean, std))

    def build(self) -> AugmentationPipeline:
        return AugmentationPipeline(list(self.ops), self.seed)
