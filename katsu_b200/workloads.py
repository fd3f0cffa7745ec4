"""The five named workloads (shapes, distributions, seeds) as data.

Each conv entry: x [N,C,H,W], w [K,C,R,S], stride, padding; values are drawn by
katsu_b200.synth with the seeds listed here so that every run, every rank and
the CPU baseline see identical inputs.  "N(0, v)" is a variance (He init:
std = sqrt(2 / fan_in)).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

from . import synth


@dataclass(frozen=True)
class ConvSpec:
    name: str
    n: int
    c: int
    h: int
    w: int
    k: int
    r: int
    s: int
    stride: int
    pad: int
    x_dist: tuple  # ("uniform", lo, hi) or ("normal", std)
    w_dist: tuple
    x_seed: int
    w_seed: int

    @property
    def oh(self):
        return (self.h + 2 * self.pad - self.r) // self.stride + 1

    @property
    def ow(self):
        return (self.w + 2 * self.pad - self.s) // self.stride + 1

    @property
    def x_shape(self):
        return [self.n, self.c, self.h, self.w]

    @property
    def w_shape(self):
        return [self.k, self.c, self.r, self.s]

    @property
    def y_shape(self):
        return [self.n, self.k, self.oh, self.ow]

    def with_batch(self, n: int) -> "ConvSpec":
        return ConvSpec(**{**self.__dict__, "n": n})

    # dense multiply-add count of one pass (padding taps included)
    @property
    def macs(self):
        return self.n * self.k * self.oh * self.ow * self.c * self.r * self.s

    @property
    def flops_fwd_bwd(self):
        return 6 * self.macs

    # compulsory traffic at the reference's function boundaries:
    # forward reads x, w and writes y; backward reads g, x, w and writes dx, dw
    @property
    def algorithmic_bytes(self):
        x = self.n * self.c * self.h * self.w
        w = self.k * self.c * self.r * self.s
        y = self.n * self.k * self.oh * self.ow
        return 4 * (2 * y + 3 * x + 3 * w)


def _draw(dist, seed, count):
    if dist[0] == "uniform":
        return synth.uniform(seed, count, dist[1], dist[2])
    if dist[0] == "normal":
        return synth.normal(seed, count, dist[1])
    raise ValueError(dist)


def conv_inputs(spec: ConvSpec, first_image: int = 0, images: int | None = None):
    """(x, w) as flat f32 arrays.  `first_image`/`images` select a batch shard
    without generating the rest (both streams are counter based)."""
    images = spec.n - first_image if images is None else images
    per_image = spec.c * spec.h * spec.w
    if spec.x_dist[0] == "uniform":
        x = synth.uniform(spec.x_seed, images * per_image, spec.x_dist[1], spec.x_dist[2], offset=first_image * per_image)
    else:
        x = synth.normal(spec.x_seed, images * per_image, spec.x_dist[1], offset=first_image * per_image)
    w = _draw(spec.w_dist, spec.w_seed, spec.k * spec.c * spec.r * spec.s)
    return x, w


def he_std(fan_in: int) -> float:
    return math.sqrt(2.0 / fan_in)


CONV = {
    # Katsu's RGB example shape as it runs on the CPU today, seed 0
    "rgb_example": ConvSpec("rgb_example", 1, 3, 224, 224, 8, 3, 3, 1, 1,
                            ("uniform", -1.0, 1.0), ("uniform", -0.5, 0.5), 0, 0 + 100),
    # batched low-channel stem: the benchmark's headline workload
    "stem_256x3x224": ConvSpec("stem_256x3x224", 256, 3, 224, 224, 64, 3, 3, 1, 1,
                               ("uniform", -1.0, 1.0), ("normal", he_std(27)), 2, 102),
    # wide-channel conv (tensor-core shape)
    "wide_128x256x56": ConvSpec("wide_128x256x56", 128, 256, 56, 56, 256, 3, 3, 1, 1,
                                ("normal", 1.0), ("normal", he_std(2304)), 3, 103),
    # strided downsampling conv
    "down_128x128x112_s2": ConvSpec("down_128x128x112_s2", 128, 128, 112, 112, 256, 3, 3, 2, 1,
                                    ("normal", 1.0), ("normal", he_std(1152)), 4, 104),
    # the two convs of the small CNN
    "cnn_conv1": ConvSpec("cnn_conv1", 512, 3, 64, 64, 32, 3, 3, 1, 1,
                          ("uniform", -1.0, 1.0), ("normal", he_std(27)), 5, 105),
    "cnn_conv2": ConvSpec("cnn_conv2", 512, 32, 64, 64, 64, 3, 3, 2, 1,
                          ("normal", 1.0), ("normal", he_std(288)), 6, 106),
}

# Small CNN: conv1 -> conv2 -> reshape [N, 65536] -> matmul W_fc [65536, 10] -> add const [N, 10] -> sum(out*out)
CNN = {
    "batch": 512,
    "fc_in": 64 * 32 * 32,
    "fc_out": 10,
    "fc_seed": 107,
    "const_seed": 205,
}


def cnn_fc_weights():
    return synth.normal(CNN["fc_seed"], CNN["fc_in"] * CNN["fc_out"], math.sqrt(1.0 / CNN["fc_in"]))


def cnn_constant(first_image: int = 0, images: int | None = None):
    images = CNN["batch"] - first_image if images is None else images
    full = synth.uniform(CNN["const_seed"], CNN["batch"] * CNN["fc_out"], -0.1, 0.1)
    return full[first_image * CNN["fc_out"]:(first_image + images) * CNN["fc_out"]].copy()
