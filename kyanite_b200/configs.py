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


# --------------------------------------------------------------------------------------
# transformer-shaped workloads
# --------------------------------------------------------------------------------------
def _normal(seeds: _Seeds, shape_, std=0.02) -> np.ndarray:
    # drawn directly in f32: the diffusion-shaped graph has 860 M weights
    out = _rng(seeds.take()).standard_normal(shape_, dtype=np.float32)
    out *= np.float32(std)
    return out


def _dense(g: Graph, seeds: _Seeds, x: Value, n_in: int, n_out: int, bias: bool = True) -> Value:
    """x [rows, n_in] -> [rows, n_out] with an [n_out, n_in] weight, N(0, 0.02)."""
    y = g.linear(x, g.constant_tensor(_normal(seeds, (n_out, n_in))))
    if bias:
        y = g.add(y, g.constant_tensor(_normal(seeds, (1, n_out))))
    return y


def _gelu(g: Graph, x: Value) -> Value:
    """x * 0.5 * (1 + erf(x / sqrt(2)))"""
    from .graph import UnaryOp
    inner = g.unary(UnaryOp.ERF, g.mul(x, g.scalar(1.0 / math.sqrt(2.0))))
    return g.mul(g.mul(x, g.scalar(0.5)), g.add(inner, g.scalar(1.0)))


def _layernorm_affine(g: Graph, x: Value, axis: int, eps: float, gamma: np.ndarray, beta: np.ndarray) -> Value:
    y = g.layernorm(x, axis, eps)
    return g.add(g.mul(y, g.constant_tensor(gamma)), g.constant_tensor(beta))


def _attention(g: Graph, q: Value, k: Value, v: Value, rows_q, rows_kv, heads: int, head_dim: int, batch,
               mask: Value = None, dtype: DType = DType.F32) -> Value:
    """q [B*Sq, h*d], k/v [B*Skv, h*d] -> [B*Sq, h*d]; scores are materialised (the IR has no attention op)."""
    sq, skv = rows_q, rows_kv

    def split(x, s):
        x = g.view(x, shape(batch, s, heads, head_dim))
        x = g.permute(x, [0, 2, 1, 3])
        return g.view(x, shape(batch * heads, s, head_dim))

    qh, kh, vh = split(q, sq), split(k, skv), split(v, skv)
    scores = g.batched_mat_mul(qh, g.permute(kh, [0, 2, 1]))
    scores = g.mul(scores, g.scalar(1.0 / math.sqrt(head_dim), dtype))
    if mask is not None:
        scores = g.add(scores, mask)
    probs = g.softmax(scores, 2)
    ctx = g.batched_mat_mul(probs, vh)
    ctx = g.view(ctx, shape(batch, heads, sq, head_dim))
    ctx = g.permute(ctx, [0, 2, 1, 3])
    return g.view(ctx, shape(batch * sq, heads * head_dim))


def bert_encoder(layers: int = 12, hidden: int = 768, heads: int = 12, ffn: int = 3072, vocab: int = 30522,
                 seq: int = 512, eps: float = 1e-12, seed: int = 10, taps: list = None) -> Tuple[Graph, Inputs]:
    """BERT-base-shaped encoder, f32, post-LayerNorm, learned positions, GELU via erf; weights N(0, 0.02),
    gamma 1, beta 0.  Input: token ids [B, seq] (i32).  `taps`, if given, receives (name, value) for the
    embedding output and every layer's output, for layer-wise checks."""
    g = Graph()
    seeds = _Seeds(seed)
    head_dim = hidden // heads
    ids = g.input(shape(BATCH, seq), DType.I32)
    table = g.constant_tensor(_normal(seeds, (vocab, hidden)))
    x = g.gather(table, 0, g.flatten(ids, 0))                         # [B*seq, hidden]
    x = g.view(x, shape(BATCH, seq, hidden))
    x = g.add(x, g.constant_tensor(_normal(seeds, (1, seq, hidden))))
    ones, zeros = np.ones((1, 1, hidden), np.float32), np.zeros((1, 1, hidden), np.float32)
    x = _layernorm_affine(g, x, 2, eps, ones, zeros)
    if taps is not None:
        taps.append(("embedding", x))
    rows = BATCH * seq
    for li in range(layers):
        x2 = g.view(x, shape(rows, hidden))
        q = _dense(g, seeds, x2, hidden, hidden)
        k = _dense(g, seeds, x2, hidden, hidden)
        v = _dense(g, seeds, x2, hidden, hidden)
        ctx = _attention(g, q, k, v, seq, seq, heads, head_dim, BATCH)
        att = _dense(g, seeds, ctx, hidden, hidden)
        x = _layernorm_affine(g, g.add(g.view(att, shape(BATCH, seq, hidden)), x), 2, eps, ones, zeros)
        x2 = g.view(x, shape(rows, hidden))
        h = _gelu(g, _dense(g, seeds, x2, hidden, ffn))
        y = _dense(g, seeds, h, ffn, hidden)
        x = _layernorm_affine(g, g.add(g.view(y, shape(BATCH, seq, hidden)), x), 2, eps, ones, zeros)
        if taps is not None:
            taps.append((f"layer{li}", x))
    g.output(x)

    def make_inputs(batch_size: int, seed: int = 1):
        return [_rng(seed).integers(0, vocab, (batch_size, seq)).astype(np.int32)]

    return g, make_inputs


def llama_weights(layers: int, d_model: int, heads: int, ffn: int, vocab: int, seed: int = 10,
                  head_slice: slice = None, ffn_slice: slice = None, vocab_slice: slice = None,
                  draw_slices_only: bool = False) -> dict:
    """The decoder's weights, N(0, 0.02) (norm gains 1 + N(0, 0.02)), drawn in a fixed order so that every
    builder of the same model (whole, or one tensor-parallel rank's slice) sees the same numbers.

    With slices given (a tensor-parallel rank), the split matrices are returned already cut: W_q/W_k/W_v rows
    and W_o columns of the heads in `head_slice`, gate/up rows and down columns of `ffn_slice`, lm-head rows of
    `vocab_slice`.  Each matrix is still drawn whole and then cut, so the numbers equal the unpartitioned
    model's, but only the slice is kept in memory.  `draw_slices_only` draws just the slice's worth of numbers
    instead (8x less work for 8 ranks; the numbers then differ from the whole model's: for timing runs)."""
    seeds = _Seeds(seed)
    hd = d_model // heads
    cols = slice(head_slice.start * hd, head_slice.stop * hd) if head_slice is not None else None

    def matrix(rows_n, cols_n, row_slice=None, col_slice=None):
        if draw_slices_only:
            r = rows_n if row_slice is None else row_slice.stop - row_slice.start
            c = cols_n if col_slice is None else col_slice.stop - col_slice.start
            return _normal(seeds, (r, c))
        m = _normal(seeds, (rows_n, cols_n))
        if row_slice is not None:
            m = np.ascontiguousarray(m[row_slice])
        if col_slice is not None:
            m = np.ascontiguousarray(m[:, col_slice])
        return m

    w = {"table": _normal(seeds, (vocab, d_model)), "layers": [], "sliced": head_slice is not None or ffn_slice is not None}
    for _ in range(layers):
        layer = {}
        layer["norm1"] = np.ones((1, 1, d_model), np.float32) + _normal(seeds, (1, 1, d_model))
        for name in ("wq", "wk", "wv"):
            layer[name] = matrix(d_model, d_model, row_slice=cols)
        layer["wo"] = matrix(d_model, d_model, col_slice=cols)
        layer["norm2"] = np.ones((1, 1, d_model), np.float32) + _normal(seeds, (1, 1, d_model))
        layer["gate"] = matrix(ffn, d_model, row_slice=ffn_slice)
        layer["up"] = matrix(ffn, d_model, row_slice=ffn_slice)
        layer["down"] = matrix(d_model, ffn, col_slice=ffn_slice)
        w["layers"].append(layer)
    w["norm_f"] = np.ones((1, 1, d_model), np.float32) + _normal(seeds, (1, 1, d_model))
    w["lm_head"] = matrix(vocab, d_model, row_slice=vocab_slice)
    return w


def rope_tables(seq: int, head_dim: int, rope_base: float):
    """cos / sin tables [1, seq, 1, head_dim] of the half-split rotary embedding."""
    inv_freq = rope_base ** (-np.arange(0, head_dim, 2, dtype=np.float64) / head_dim)
    ang = np.arange(seq, dtype=np.float64)[:, None] * inv_freq[None, :]            # [seq, hd/2]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], 1).astype(np.float32).reshape(1, seq, 1, head_dim)
    sin = np.concatenate([np.sin(ang), np.sin(ang)], 1).astype(np.float32).reshape(1, seq, 1, head_dim)
    return cos, sin


class LlamaBlocks:
    """The pieces of the LLaMA-shaped decoder as graph fragments, shared by `llama_decoder` and by the
    tensor-parallel builder (kyanite_b200/tensor_parallel.py), which uses them on weight slices."""

    def __init__(self, g: Graph, d_model: int, head_dim: int, seq: int, eps: float, rope_base: float,
                 dtype: DType = DType.F32):
        """`dtype`: the storage type of activations and weights, F32 or F16.  With F16 every value of the graph is
        f16 except inside RMSNorm, whose statistics are computed on f32 casts (as half-precision decoders do) and
        whose result is cast back."""
        self.g, self.d_model, self.hd, self.seq, self.eps, self.dtype = g, d_model, head_dim, seq, eps, dtype
        cos, sin = rope_tables(seq, head_dim, rope_base)
        self.cos, self.sin = g.constant_tensor(cos.astype(dtype.np)), g.constant_tensor(sin.astype(dtype.np))
        self.mask = g.constant_tensor(np.triu(np.full((seq, seq), -np.inf, dtype.np), 1).reshape(1, seq, seq))
        self.rows = BATCH * seq

    def linear(self, x: Value, w: np.ndarray) -> Value:
        return self.g.linear(x, self.g.constant_tensor(np.ascontiguousarray(w, dtype=self.dtype.np)))

    def rmsnorm(self, t: Value, gain: np.ndarray) -> Value:
        """t [B, seq, d_model]: composed from pow / mean / sqrt / div (the IR has no RMSNorm)."""
        from .graph import BinaryOp, ReduceOp, UnaryOp
        g = self.g
        if self.dtype != DType.F32:
            t = g.value_cast(t, DType.F32)
        ms = g.view(g.reduce(g.pow(t, g.scalar(2.0)), [2], ReduceOp.MEAN), shape(BATCH, self.seq, 1))
        rms = g.unary(UnaryOp.SQRT, g.add(ms, g.scalar(self.eps)))
        out = g.mul(g.binary(BinaryOp.DIV, t, rms), g.constant_tensor(gain))
        return out if self.dtype == DType.F32 else g.value_cast(out, self.dtype)

    def rope(self, t: Value, heads: int) -> Value:
        """t [B*seq, heads*hd] -> rotated, same shape (half-split: pairs (i, i + hd/2))."""
        from .graph import SliceRange, UnaryOp
        g, hd = self.g, self.hd
        t4 = g.view(t, shape(BATCH, self.seq, heads, hd))
        lo = g.slice(t4, 3, SliceRange(0, hd // 2))
        hi = g.slice(t4, 3, SliceRange(hd // 2, hd))
        rot = g.concat([g.unary(UnaryOp.NEG, hi), lo], 3)
        out = g.add(g.mul(t4, self.cos), g.mul(rot, self.sin))
        return g.view(out, shape(self.rows, heads * hd))

    def attention_partial(self, x: Value, layer: dict, head_slice: slice, heads: int) -> Value:
        """Pre-norm causal self-attention over the heads in `head_slice`, projected by the matching
        columns of W_o: [B, seq, d_model].  With all heads this is the whole attention output; with a
        slice, the slices of all ranks sum to it (column-parallel Q/K/V, row-parallel O)."""
        g, hd = self.g, self.hd
        cols = slice(head_slice.start * hd, head_slice.stop * hd)
        if layer["wq"].shape[0] == heads * hd:      # weights that `llama_weights` already cut for this rank
            cols = slice(None)
        h = g.view(self.rmsnorm(x, layer["norm1"]), shape(self.rows, self.d_model))
        q = self.rope(self.linear(h, layer["wq"][cols]), heads)
        k = self.rope(self.linear(h, layer["wk"][cols]), heads)
        v = self.linear(h, layer["wv"][cols])
        ctx = _attention(g, q, k, v, self.seq, self.seq, heads, hd, BATCH, mask=self.mask, dtype=self.dtype)
        return g.view(self.linear(ctx, layer["wo"][:, cols]), shape(BATCH, self.seq, self.d_model))

    def ffn_partial(self, x: Value, layer: dict, ffn_slice: slice) -> Value:
        """Pre-norm SwiGLU feed-forward over the hidden units in `ffn_slice`: [B, seq, d_model]
        (column-parallel gate/up, row-parallel down)."""
        g = self.g
        if layer["gate"].shape[0] == ffn_slice.stop - ffn_slice.start:   # already cut for this rank
            ffn_slice = slice(None)
        h = g.view(self.rmsnorm(x, layer["norm2"]), shape(self.rows, self.d_model))
        gate = self.linear(h, layer["gate"][ffn_slice])
        up = self.linear(h, layer["up"][ffn_slice])
        act = g.mul(g.mul(gate, g.sigmoid(gate)), up)
        return g.view(self.linear(act, layer["down"][:, ffn_slice]), shape(BATCH, self.seq, self.d_model))

    def logits(self, x: Value, gain: np.ndarray, lm_head: np.ndarray) -> Value:
        h = self.g.view(self.rmsnorm(x, gain), shape(self.rows, self.d_model))
        return self.g.view(self.linear(h, lm_head), shape(BATCH, self.seq, lm_head.shape[0]))


def llama_decoder(layers: int = 32, d_model: int = 4096, heads: int = 32, ffn: int = 11008, vocab: int = 32000,
                  seq: int = 2048, eps: float = 1e-6, rope_base: float = 10000.0, seed: int = 10,
                  dtype: DType = DType.F32, taps: list = None) -> Tuple[Graph, Inputs]:
    """LLaMA-shaped decoder prefill: RMSNorm composed from pow / mean / sqrt / div, rotary embedding from
    constant cos/sin tables with half-split slices, additive causal mask, SwiGLU, tied-shape lm head.
    Input: token ids [B, seq] (i32).  `dtype` F32, or F16 for half storage with f32 accumulation (weights,
    activations and logits f16; see `LlamaBlocks`).  `taps` receives (name, value) for the embedding and every
    block's output."""
    g = Graph()
    w = llama_weights(layers, d_model, heads, ffn, vocab, seed)
    blocks = LlamaBlocks(g, d_model, d_model // heads, seq, eps, rope_base, dtype)
    ids = g.input(shape(BATCH, seq), DType.I32)
    x = g.view(g.gather(g.constant_tensor(w["table"].astype(dtype.np)), 0, g.flatten(ids, 0)), shape(BATCH, seq, d_model))
    if taps is not None:
        taps.append(("embedding", x))
    for li, layer in enumerate(w["layers"]):
        x = g.add(x, blocks.attention_partial(x, layer, slice(0, heads), heads))
        if taps is not None:
            taps.append((f"layer{li}.attention", x))
        x = g.add(x, blocks.ffn_partial(x, layer, slice(0, ffn)))
        if taps is not None:
            taps.append((f"layer{li}.ffn", x))
    g.output(blocks.logits(x, w["norm_f"], w["lm_head"]))

    def make_inputs(batch_size: int, seed: int = 1):
        return [_rng(seed).integers(0, vocab, (batch_size, seq)).astype(np.int32)]

    return g, make_inputs


# --------------------------------------------------------------------------------------
# diffusion-UNet-shaped workload
# --------------------------------------------------------------------------------------
def unet_step(levels=(320, 640, 1280, 1280), res_blocks: int = 2, attention_levels=(0, 1, 2), heads: int = 8,
              latent_channels: int = 4, size: int = 64, ctx_len: int = 77, ctx_dim: int = 768, groups: int = 32,
              seed: int = 10, taps: list = None) -> Tuple[Graph, Inputs]:
    """One denoising step of a latent-diffusion-shaped UNet, f32.  The concrete layout (this file is
    its definition): sinusoidal timestep embedding of dim levels[0] -> two linears with SiLU; conv-in;
    per level `res_blocks` x [ResBlock (+ transformer block on attention levels)] then a stride-2
    conv down (except the last level); middle ResBlock - transformer - ResBlock; up path mirrors it with
    skip concatenation (res_blocks + 1 blocks per level) and nearest x2 upsampling + conv; GroupNorm
    (as view + layernorm + affine), SiLU, conv-out.  Transformer block: self-attention, cross-attention
    on the text context, GEGLU feed-forward, each with pre-LayerNorm and a residual.  Weights N(0, 0.02).
    Inputs: latent [B, C, size, size], timestep [1], context [B, ctx_len, ctx_dim].  `taps`, if given, receives
    (name, value) for the output of every block (ResBlock, transformer, down- and up-sampling convolution),
    for layer-wise checks."""
    from .graph import SliceRange, UnaryOp
    g = Graph()
    seeds = _Seeds(seed)
    ch0 = levels[0]
    temb_dim = 4 * ch0

    latent = g.input(shape(BATCH, latent_channels, size, size))
    timestep = g.input(shape(1))
    context = g.input(shape(BATCH, ctx_len, ctx_dim))

    def silu(t):
        return g.mul(t, g.sigmoid(t))

    def conv(t, cin, cout, k, stride=1):
        w = g.constant_tensor(_normal(seeds, (cout, cin, k, k)))
        b = g.constant_tensor(_normal(seeds, (1, cout, 1, 1)))
        return g.add(g.conv(t, w, stride, stride, k // 2, k // 2), b)

    def group_norm(t, c, hw):
        n = g.view(t, shape(BATCH, groups, (c // groups) * hw * hw))
        n = g.view(g.layernorm(n, 2, 1e-5), shape(BATCH, c, hw, hw))
        gamma = g.constant_tensor(np.ones((1, c, 1, 1), np.float32) + _normal(seeds, (1, c, 1, 1)))
        beta = g.constant_tensor(_normal(seeds, (1, c, 1, 1)))
        return g.add(g.mul(n, gamma), beta)

    # timestep embedding
    half = ch0 // 2
    freqs = np.exp(-math.log(10000.0) * np.arange(half, dtype=np.float64) / half).astype(np.float32)
    args = g.mul(g.view(timestep, shape(1, 1)), g.constant_tensor(freqs.reshape(1, half)))
    emb = g.concat([g.unary(UnaryOp.COS, args), g.unary(UnaryOp.SIN, args)], 1)          # [1, ch0]
    temb = _dense(g, seeds, silu(_dense(g, seeds, emb, ch0, temb_dim)), temb_dim, temb_dim)
    temb_act = silu(temb)

    def res_block(t, cin, cout, hw):
        h = conv(silu(group_norm(t, cin, hw)), cin, cout, 3)
        te = g.view(_dense(g, seeds, temb_act, temb_dim, cout), shape(1, cout, 1, 1))
        h = g.add(h, te)
        h = conv(silu(group_norm(h, cout, hw)), cout, cout, 3)
        skip = t if cin == cout else conv(t, cin, cout, 1)
        return g.add(h, skip)

    ctx_rows = g.view(context, shape(BATCH * ctx_len, ctx_dim))

    def layer_norm(t, c):
        gamma = np.ones((1, 1, c), np.float32)
        return _layernorm_affine(g, t, 2, 1e-5, gamma, np.zeros((1, 1, c), np.float32))

    def transformer(t, c, hw):
        tokens = hw * hw
        hd = c // heads
        h = conv(group_norm(t, c, hw), c, c, 1)
        x = g.view(g.permute(h, [0, 2, 3, 1]), shape(BATCH, tokens, c))
        # self-attention
        n = g.view(layer_norm(x, c), shape(BATCH * tokens, c))
        q = _dense(g, seeds, n, c, c, bias=False)
        k = _dense(g, seeds, n, c, c, bias=False)
        v = _dense(g, seeds, n, c, c, bias=False)
        a = _dense(g, seeds, _attention(g, q, k, v, tokens, tokens, heads, hd, BATCH), c, c)
        x = g.add(x, g.view(a, shape(BATCH, tokens, c)))
        # cross-attention on the text context
        n = g.view(layer_norm(x, c), shape(BATCH * tokens, c))
        q = _dense(g, seeds, n, c, c, bias=False)
        k = _dense(g, seeds, ctx_rows, ctx_dim, c, bias=False)
        v = _dense(g, seeds, ctx_rows, ctx_dim, c, bias=False)
        a = _dense(g, seeds, _attention(g, q, k, v, tokens, ctx_len, heads, hd, BATCH), c, c)
        x = g.add(x, g.view(a, shape(BATCH, tokens, c)))
        # GEGLU feed-forward
        n = g.view(layer_norm(x, c), shape(BATCH * tokens, c))
        proj = _dense(g, seeds, n, c, 8 * c)
        val = g.slice(proj, 1, SliceRange(0, 4 * c))
        gate = g.slice(proj, 1, SliceRange(4 * c, 8 * c))
        ff = _dense(g, seeds, g.mul(val, _gelu(g, gate)), 4 * c, c)
        x = g.add(x, g.view(ff, shape(BATCH, tokens, c)))
        back = g.permute(g.view(x, shape(BATCH, hw, hw, c)), [0, 3, 1, 2])
        return g.add(conv(back, c, c, 1), t)

    def tap(name, v):
        if taps is not None:
            taps.append((name, v))
        return v

    # down path
    cur = tap("conv_in", conv(latent, latent_channels, ch0, 3))
    hw = size
    skips = [(cur, ch0)]
    c_prev = ch0
    for li, c in enumerate(levels):
        for bi in range(res_blocks):
            cur = tap(f"down{li}.res{bi}", res_block(cur, c_prev, c, hw))
            c_prev = c
            if li in attention_levels:
                cur = tap(f"down{li}.attn{bi}", transformer(cur, c, hw))
            skips.append((cur, c))
        if li != len(levels) - 1:
            cur = tap(f"down{li}.downsample", conv(cur, c, c, 3, stride=2))
            hw //= 2
            skips.append((cur, c))
    # middle
    cur = tap("mid.res0", res_block(cur, c_prev, c_prev, hw))
    cur = tap("mid.attn", transformer(cur, c_prev, hw))
    cur = tap("mid.res1", res_block(cur, c_prev, c_prev, hw))
    # up path
    for li in reversed(range(len(levels))):
        c = levels[li]
        for bi in range(res_blocks + 1):
            skip, cs = skips.pop()
            cur = tap(f"up{li}.res{bi}", res_block(g.concat([cur, skip], 1), c_prev + cs, c, hw))
            c_prev = c
            if li in attention_levels:
                cur = tap(f"up{li}.attn{bi}", transformer(cur, c, hw))
        if li != 0:
            cur = g.repeat_interleave(g.repeat_interleave(cur, 2, 2), 3, 2)
            hw *= 2
            cur = tap(f"up{li}.upsample", conv(cur, c, c, 3))
    out = conv(silu(group_norm(cur, c_prev, hw)), c_prev, latent_channels, 3)
    g.output(out)

    def make_inputs(batch_size: int, seed: int = 1):
        r = _rng(seed)
        return [r.standard_normal((batch_size, latent_channels, size, size)).astype(np.float32),
                np.array([500.0], np.float32),
                _rng(seed + 1).standard_normal((batch_size, ctx_len, ctx_dim)).astype(np.float32)]

    return g, make_inputs
