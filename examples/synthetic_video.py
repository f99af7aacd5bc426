"""Seeded synthetic videos standing in for the real footage the reference was demonstrated on
(static camera, few moving objects). One generator, parameterised per benchmark configuration.

A video is a static smooth-noise background in [0,1] plus moving textured objects plus
per-frame Gaussian noise; everything derives from ``seed`` so that runs are reproducible on
any machine. Frames are float32 N,3,H,W in [0,1].
"""
import math

import torch


def _background(gen, h, w):
    low = torch.rand(1, 3, max(h // 16, 2), max(w // 16, 2), generator=gen)
    bg = torch.nn.functional.interpolate(low, size=(h, w), mode="bilinear", align_corners=False)[0]
    bg = (bg - bg.min()) / (bg.max() - bg.min() + 1e-12)
    return bg


class MovingObjectsVideo:
    """Rectangles (textured patches) or Gaussian blobs moving with integer velocities and
    reflecting at the borders."""

    def __init__(self, seed, h, w, n_objects=3, obj_h=40, obj_w=40, vmin=2, vmax=4, sigma=0.005, kind="rect",
                 blob_sigma=12.0, blob_amp=0.8):
        self.h, self.w, self.sigma, self.kind = h, w, sigma, kind
        self.seed = seed
        gen = torch.Generator().manual_seed(seed)
        self.bg = _background(gen, h, w)
        self.objs = []
        for i in range(n_objects):
            og = torch.Generator().manual_seed(seed * 1000 + 17 * (i + 1))
            if kind == "rect":
                tex = torch.rand(3, obj_h, obj_w, generator=og)
                alpha = torch.ones(1, obj_h, obj_w)
            else:
                r = int(3 * blob_sigma)
                ys = torch.arange(-r, r + 1).float()
                gy, gx = torch.meshgrid(ys, ys, indexing="ij")
                alpha = (blob_amp * torch.exp(-(gy * gy + gx * gx) / (2 * blob_sigma ** 2)))[None]
                tex = torch.rand(3, 1, 1, generator=og).expand(3, 2 * r + 1, 2 * r + 1)
            oh, ow = tex.shape[1:]
            y = int(torch.randint(0, max(h - oh, 1), (1,), generator=og))
            x = int(torch.randint(0, max(w - ow, 1), (1,), generator=og))
            vy = int(torch.randint(vmin, vmax + 1, (1,), generator=og)) * (1 if torch.rand(1, generator=og) < 0.5 else -1)
            vx = int(torch.randint(vmin, vmax + 1, (1,), generator=og)) * (1 if torch.rand(1, generator=og) < 0.5 else -1)
            self.objs.append([tex, alpha, y, x, vy, vx])

    def _reflect(self, p, v, size, limit):
        p += v
        if p < 0:
            p, v = -p, -v
        if p + size > limit:
            p, v = 2 * (limit - size) - p, -v
        return max(min(p, limit - size), 0), v

    def frame(self, t):
        """Frame ``t`` (frames must be requested in increasing order starting at 0)."""
        img = self.bg.clone()
        for o in self.objs:
            tex, alpha, y, x, vy, vx = o
            oh, ow = tex.shape[1:]
            if t > 0:
                y, vy = self._reflect(y, vy, oh, self.h)
                x, vx = self._reflect(x, vx, ow, self.w)
                o[2:] = [y, x, vy, vx]
            img[:, y:y + oh, x:x + ow] = img[:, y:y + oh, x:x + ow] * (1 - alpha) + tex * alpha
        if self.sigma > 0:
            ng = torch.Generator().manual_seed(self.seed * 100003 + t)
            img = img + self.sigma * torch.randn(img.shape, generator=ng)
        return img.clamp_(0, 1)

    def frames(self, n):
        return torch.stack([self.frame(t) for t in range(n)])


class StickFigureVideo:
    """An articulated figure of 14 Gaussian-blurred limb segments whose joint angles follow
    seeded sinusoids, over a static background."""

    def __init__(self, seed, h, w, sigma=0.003, width=4.0):
        self.h, self.w, self.sigma, self.width, self.seed = h, w, sigma, width, seed
        gen = torch.Generator().manual_seed(seed)
        self.bg = _background(gen, h, w) * 0.6
        self.phase = torch.rand(14, generator=gen) * 2 * math.pi
        self.freq = 0.15 + 0.2 * torch.rand(14, generator=gen)
        self.base = torch.tensor([90, 90, 200, 340, 200, 340, 250, 290, 250, 290, 270, 270, 180, 0], dtype=torch.float32)
        self.length = torch.tensor([0.16, 0.1, 0.12, 0.12, 0.1, 0.1, 0.15, 0.15, 0.14, 0.14, 0.05, 0.05, 0.06, 0.06]) * h
        # parent joint of each segment (-1: anchored at the hip), a fixed 14-segment skeleton
        self.parent = [-1, 0, 1, 1, 2, 3, -1, -1, 6, 7, 8, 9, 1, 1]
        ys, xs = torch.meshgrid(torch.arange(h).float(), torch.arange(w).float(), indexing="ij")
        self.ys, self.xs = ys, xs
        self.colour = torch.rand(14, 3, generator=gen)

    def frame(self, t):
        hip = torch.tensor([self.h * 0.55 + 4 * math.sin(0.2 * t), self.w * 0.5 + 0.6 * t % (self.w * 0.2)])
        ends, img = [], self.bg.clone()
        for s in range(14):
            a = math.radians(float(self.base[s]) + 25 * math.sin(float(self.freq[s]) * t + float(self.phase[s])))
            start = hip if self.parent[s] < 0 else ends[self.parent[s]]
            end = start + self.length[s] * torch.tensor([-math.sin(a), math.cos(a)])
            ends.append(end)
            d = end - start
            tt = (((self.ys - start[0]) * d[0] + (self.xs - start[1]) * d[1]) / (d.dot(d) + 1e-6)).clamp(0, 1)
            dist2 = (self.ys - (start[0] + tt * d[0])) ** 2 + (self.xs - (start[1] + tt * d[1])) ** 2
            alpha = torch.exp(-dist2 / (2 * (self.width / 2) ** 2))[None]
            img = img * (1 - alpha) + self.colour[s][:, None, None] * alpha
        if self.sigma > 0:
            ng = torch.Generator().manual_seed(self.seed * 100003 + t)
            img = img + self.sigma * torch.randn(img.shape, generator=ng)
        return img.clamp_(0, 1)

    def frames(self, n):
        return torch.stack([self.frame(t) for t in range(n)])


def make_video(config, seed):
    """Video source of a benchmark configuration: 'mobilenet' (224x224, 3 rectangles 40x40),
    'resnet50' (512x512, 5 blobs), 'hrnet' (256x256 stick figure), 'centernet' (544x960, 20
    rectangles 80x30)."""
    if config == "mobilenet":
        return MovingObjectsVideo(seed, 224, 224, 3, 40, 40, 2, 4, 0.005, "rect")
    if config == "resnet50":
        return MovingObjectsVideo(seed, 512, 512, 5, 0, 0, 2, 4, 0.003, "blob")
    if config == "hrnet":
        return StickFigureVideo(seed, 256, 256)
    if config == "centernet":
        return MovingObjectsVideo(seed, 544, 960, 20, 80, 30, 1, 3, 0.003, "rect")
    raise ValueError(config)
