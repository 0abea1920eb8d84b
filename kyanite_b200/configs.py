"""Builders for the benchmark workloads: synthetic graphs with the shapes of the configurations the
executor is measured on, random-initialised from a seed (no trained weights are involved), and
their seeded synthetic inputs.

Every builder returns `(graph, make_inputs)` where `make_inputs(batch_size, seed)` yields the list
of host arrays for one evaluation.
"""
from __future__ import annotations

import math
from typing import Callable, List, Tuple

import numpy as np

from .graph import BATCH, DType, Graph, Value, shape

Inputs = Callable[[int, int], List[np.ndarray]]


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


class _Seeds:
    def __init__(self, first: int):
        self.next = first

    def take(self) -> int:
        s = self.next
        self.next += 1
        return s


def _linear(g: Graph, x: Value, w: np.ndarray, b: np.ndarray) -> Value:
    """`linear` + bias as the builder emits them: permute + matmul + broadcast add."""
    y = g.linear(x, g.constant_tensor(w.astype(np.float32)))
    return g.add(y, g.constant_tensor(b.astype(np.float32).reshape(1, -1)))


def mlp() -> Tuple[Graph, Inputs]:
    """f32 MLP 16 -> 32 -> 32 -> 4 with ReLU and a final softmax; weights U(-1/4, 1/4),
    biases 0.01 * N(0, 1)."""
    g = Graph()
    x = g.input(shape(BATCH, 16))
    seeds = _Seeds(2)
    dims = [(16, 32), (32, 32), (32, 4)]
    ws = [_rng(seeds.take()).uniform(-0.25, 0.25, (o, i)) for i, o in dims]
    bs = [0.01 * _rng(seeds.take()).standard_normal(o) for _, o in dims]
    cur = x
    for k, (w, b) in enumerate(zip(ws, bs)):
        cur = _linear(g, cur, w, b)
        if k < 2:
            cur = g.relu(cur)
    g.output(g.softmax(cur, 1))

    def make_inputs(batch_size: int, seed: int = 1):
        return [_rng(seed).standard_normal((batch_size, 16)).astype(np.float32)]

    return g, make_inputs


def resnet_tower(channels: int = 128, blocks: int = 16, board: int = 8, in_planes: int = 21,
                 policy_channels: int = 73, value_channels: int = 32, value_hidden: int = 256,
                 seed: int = 10) -> Tuple[Graph, Inputs]:
    """ResNet-style board-game tower, f32.  Stem conv3x3 + bias + ReLU; `blocks` residual blocks of
    conv3x3 + bias, ReLU, conv3x3 + bias, + residual, ReLU (batch-norm already folded into the
    bias); policy head conv1x1 -> flatten -> softmax; value head conv1x1 -> flatten -> linear + ReLU
    -> linear -> softmax.  Kaiming-normal weights; the second convolution of every block is scaled by
    1/sqrt(2 * blocks), standing in for the folded batch-norm gain, so that activations stay O(1)
    through the residual stream instead of doubling in variance per block."""
    g = Graph()
    seeds = _Seeds(seed)

    def conv_w(cout, cin, k, gain=1.0):
        std = gain * math.sqrt(2.0 / (cin * k * k))
        return (_rng(seeds.take()).standard_normal((cout, cin, k, k)) * std).astype(np.float32)

    def bias(c):
        return (0.1 * _rng(seeds.take()).standard_normal((1, c, 1, 1))).astype(np.float32)

    def conv_bias(x, cout, cin, k, gain=1.0):
        y = g.conv(x, g.constant_tensor(conv_w(cout, cin, k, gain)), 1, 1, k // 2, k // 2)
        return g.add(y, g.constant_tensor(bias(cout)))

    x = g.input(shape(BATCH, in_planes, board, board))
    cur = g.relu(conv_bias(x, channels, in_planes, 3))
    for _ in range(blocks):
        y = g.relu(conv_bias(cur, channels, channels, 3))
        y = conv_bias(y, channels, channels, 3, gain=1.0 / math.sqrt(2.0 * blocks))
        cur = g.relu(g.add(y, cur))

    policy = conv_bias(cur, policy_channels, channels, 1)
    policy = g.softmax(g.flatten(policy, 1), 1)

    value = conv_bias(cur, value_channels, channels, 1)
    value = g.flatten(value, 1)
    flat = value_channels * board * board
    w1 = _rng(seeds.take()).standard_normal((value_hidden, flat)) * math.sqrt(2.0 / flat)
    b1 = 0.1 * _rng(seeds.take()).standard_normal(value_hidden)
    w2 = _rng(seeds.take()).standard_normal((3, value_hidden)) * math.sqrt(2.0 / value_hidden)
    b2 = 0.1 * _rng(seeds.take()).standard_normal(3)
    value = g.relu(_linear(g, value, w1, b1))
    value = g.softmax(_linear(g, value, w2, b2), 1)

    g.output_all([policy, value])

    def make_inputs(batch_size: int, seed: int = 1):
        planes = _rng(seed).random((batch_size, in_planes, board, board)) < 0.1
        return [planes.astype(np.float32)]

    return g, make_inputs


def resnet_tower_flops(batch: int, channels: int = 128, blocks: int = 16, board: int = 8, in_planes: int = 21,
                       policy_channels: int = 73, value_channels: int = 32, value_hidden: int = 256) -> float:
    """2*M*N*K over every conv and matmul of `resnet_tower` (padding taps included)."""
    px = batch * board * board
    f = 2.0 * px * channels * in_planes * 9
    f += blocks * 2 * (2.0 * px * channels * channels * 9)
    f += 2.0 * px * policy_channels * channels + 2.0 * px * value_channels * channels
    f += 2.0 * batch * value_hidden * value_channels * board * board + 2.0 * batch * 3 * value_hidden
    return f
