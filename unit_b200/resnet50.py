"""ResNet-50 (v1b stride placement) convolution layer table and synthetic inputs.

Shapes are the ones the reference logged for this network (its
``cpu-shapes.log`` resnet50_v1b rows): a 7x7/2 stem on 3 channels, then four
bottleneck stages of widths 64/128/256/512 at 56/28/14/7 pixels, each block a
1x1 reduce, a 3x3 (stride 2 on the first 3x3 of stages 2-4) and a 1x1 expand,
plus the four 1x1 projection shortcuts.  ``count`` is how often a shape occurs:
53 convolutions in total.

The value distributions stand in for the calibrated ImageNet models the
reference ran: post-ReLU u8 activations (half zeros, the rest uniform in
[1, 255]), s8 weights round(N(0, 32)) clipped to [-128, 127], s32 bias uniform
in [-2^15, 2^15), requantisation shift 8.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

import numpy as np


@dataclass(frozen=True)
class ConvLayer:
    name: str
    c_in: int      # logical input channels
    hw: int        # input height = width
    c_out: int
    k: int
    stride: int
    pad: int
    count: int
    proj: bool = False

    @property
    def c_block(self) -> int:
        return 16 if self.c_in % 16 == 0 else 4

    @property
    def c_in_stored(self) -> int:
        return (self.c_in + self.c_block - 1) // self.c_block * self.c_block

    @property
    def out_hw(self) -> int:
        return (self.hw + 2 * self.pad - self.k) // self.stride + 1

    def ops(self, batch: int) -> float:
        """2 x MACs with logical channels, every tap counted."""
        return 2.0 * batch * self.out_hw ** 2 * self.c_out * self.c_in * self.k ** 2

    def bytes(self, batch: int, out_bytes: int = 1, bias: bool = True) -> float:
        """Each tensor once in its boundary layout: activations, weights, output, bias."""
        x = batch * self.c_in_stored * self.hw ** 2
        w = self.c_out * self.c_in_stored * self.k ** 2
        o = batch * self.c_out * self.out_hw ** 2 * out_bytes
        return float(x + w + o + (4 * self.c_out if bias else 0))


LAYERS: List[ConvLayer] = [
    ConvLayer('stem_7x7s2_3_64', 3, 224, 64, 7, 2, 3, 1),
    ConvLayer('s1_1x1_64_64', 64, 56, 64, 1, 1, 0, 1),
    ConvLayer('s1_1x1_256_64', 256, 56, 64, 1, 1, 0, 2),
    ConvLayer('s1_3x3_64_64', 64, 56, 64, 3, 1, 1, 3),
    ConvLayer('s1_1x1_64_256', 64, 56, 256, 1, 1, 0, 3),
    ConvLayer('s1_proj_64_256', 64, 56, 256, 1, 1, 0, 1, True),
    ConvLayer('s2_1x1_256_128', 256, 56, 128, 1, 1, 0, 1),
    ConvLayer('s2_3x3s2_128_128', 128, 56, 128, 3, 2, 1, 1),
    ConvLayer('s2_1x1_512_128', 512, 28, 128, 1, 1, 0, 3),
    ConvLayer('s2_3x3_128_128', 128, 28, 128, 3, 1, 1, 3),
    ConvLayer('s2_1x1_128_512', 128, 28, 512, 1, 1, 0, 4),
    ConvLayer('s2_proj_s2_256_512', 256, 56, 512, 1, 2, 0, 1, True),
    ConvLayer('s3_1x1_512_256', 512, 28, 256, 1, 1, 0, 1),
    ConvLayer('s3_3x3s2_256_256', 256, 28, 256, 3, 2, 1, 1),
    ConvLayer('s3_1x1_1024_256', 1024, 14, 256, 1, 1, 0, 5),
    ConvLayer('s3_3x3_256_256', 256, 14, 256, 3, 1, 1, 5),
    ConvLayer('s3_1x1_256_1024', 256, 14, 1024, 1, 1, 0, 6),
    ConvLayer('s3_proj_s2_512_1024', 512, 28, 1024, 1, 2, 0, 1, True),
    ConvLayer('s4_1x1_1024_512', 1024, 14, 512, 1, 1, 0, 1),
    ConvLayer('s4_3x3s2_512_512', 512, 14, 512, 3, 2, 1, 1),
    ConvLayer('s4_1x1_2048_512', 2048, 7, 512, 1, 1, 0, 2),
    ConvLayer('s4_3x3_512_512', 512, 7, 512, 3, 1, 1, 2),
    ConvLayer('s4_1x1_512_2048', 512, 7, 2048, 1, 1, 0, 3),
    ConvLayer('s4_proj_s2_1024_2048', 1024, 14, 2048, 1, 2, 0, 1, True),
]


def sweep_ops(batch: int) -> float:
    return sum(l.ops(batch) * l.count for l in LAYERS)


def sweep_bytes(batch: int) -> float:
    return sum(l.bytes(batch) * l.count for l in LAYERS)


def synth_activations(rng: np.random.Generator, shape: Tuple[int, ...]) -> np.ndarray:
    """Post-ReLU u8: Bernoulli(0.5) x U[1, 255]."""
    v = rng.integers(1, 256, size=shape, dtype=np.uint8)
    return v * rng.integers(0, 2, size=shape, dtype=np.uint8)


def synth_weights(rng: np.random.Generator, shape: Tuple[int, ...]) -> np.ndarray:
    return np.clip(np.rint(rng.normal(0.0, 32.0, size=shape)), -128, 127).astype(np.int8)


def synth_bias(rng: np.random.Generator, n: int) -> np.ndarray:
    return rng.integers(-2 ** 15, 2 ** 15, size=n, dtype=np.int32)


def layer_seed(config: int, layer_index: int, what: int) -> int:
    """Seeds 1000*config + 10*layer + {0: activations, 1: weights, 2: bias}."""
    return 1000 * config + 10 * layer_index + what


def make_layer_inputs(layer: ConvLayer, layer_index: int, batch: int, config: int = 3):
    """Blocked-layout host arrays (x, w, bias) for one layer, seeded."""
    cb = layer.c_block
    cs = layer.c_in_stored
    x = synth_activations(np.random.default_rng(layer_seed(config, layer_index, 0)),
                          (batch, cs // cb, layer.hw, layer.hw, cb))
    w = synth_weights(np.random.default_rng(layer_seed(config, layer_index, 1)),
                      (layer.c_out // 16, cs // cb, layer.k, layer.k, cb // 4, 16, 4))
    if cs != layer.c_in:  # stored padding channels carry zeros
        x[..., layer.c_in:] = 0
        wv = w.reshape(layer.c_out // 16, cs // cb, layer.k, layer.k, cb // 4, 16, 4)
        for m in range(cb // 4):
            for r in range(4):
                if m * 4 + r >= layer.c_in:
                    wv[:, :, :, :, m, :, r] = 0
    b = synth_bias(np.random.default_rng(layer_seed(config, layer_index, 2)), layer.c_out)
    return x, w, b
