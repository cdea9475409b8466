"""Parameter layouts and seeded synthetic inputs of the two CNN benchmark configs
(LeNet-5 on 28x28, the VGG-style net on 64x64), shared by the trace generator, the
tests and bench.py so that all of them drive the same step programs with the same data."""
from __future__ import annotations

import numpy as np

from . import synth

LENET_SHAPES = [(6, 1, 5, 5), (6,), (16, 6, 5, 5), (16,), (400, 120), (120,), (120, 84), (84,), (84, 10), (10,)]
LENET_FAN_IN = [25, 25, 150, 150, 400, 400, 120, 120, 84, 84]
LENET_NAMES = ["W1", "b1", "W2", "b2", "W3", "b3", "W4", "b4", "W5", "b5"]

VGG_CHAN = (3, 64, 64, 128, 128, 256, 256)      # input channels, then the six conv widths (three blocks of two)


def lenet_params(seed=synth.SEED_BASE + 4):
    return [synth.kaiming_uniform(seed, 10 + i, int(np.prod(s)), f) for i, (s, f) in enumerate(zip(LENET_SHAPES, LENET_FAN_IN))]


def lenet_inputs(B, steps, seed=synth.SEED_BASE + 4):
    return synth.uniform(seed, 0, steps * B * 784), synth.labels(seed, 1, steps * B, 10), lenet_params(seed)


def vgg_shapes(chan=VGG_CHAN, H=64, classes=100):
    shapes, names = [], []
    for l in range(6):
        shapes += [(chan[l + 1], chan[l], 3, 3), (chan[l + 1],), (chan[l + 1],)]
        names += [f"W{l}", f"gamma{l}", f"beta{l}"]
    F = chan[6] * (H // 8) ** 2
    return shapes + [(F, classes), (classes,)], names + ["Wl", "bl"]


def vgg_params(H=64, classes=100, chan=VGG_CHAN, seed=synth.SEED_BASE + 5):
    shapes, names = vgg_shapes(chan, H, classes)
    ps = []
    for i, (s, n) in enumerate(zip(shapes, names)):
        k = int(np.prod(s))
        if n.startswith("gamma"):
            ps.append(np.float32(1) + np.float32(0.1) * synth.uniform(seed, 10 + i, k))
        elif n.startswith("beta") or n == "bl":
            ps.append(np.float32(0.1) * synth.uniform(seed, 10 + i, k))
        else:
            ps.append(synth.kaiming_uniform(seed, 10 + i, k, int(np.prod(s[1:])) if len(s) == 4 else s[0]))
    return ps


def vgg_inputs(B, steps, H=64, classes=100, chan=VGG_CHAN, seed=synth.SEED_BASE + 5):
    x = synth.normal(seed, 0, steps * B * chan[0] * H * H)
    return x, synth.labels(seed, 1, steps * B, classes), vgg_params(H, classes, chan, seed)


def onehot(labels, classes):
    o = np.zeros((labels.size, classes), dtype=np.float32)
    o[np.arange(labels.size), labels] = 1.0
    return o.ravel()
