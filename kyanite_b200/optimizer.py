"""Graph optimiser: rewrites a `Graph` into an equivalent, cheaper one before it is planned.

Mirrors `optimize_graph` of the reference (kn-graph/src/optimizer/mod.rs:26-47, core.rs, affine.rs).  Only
values reachable from the outputs are rebuilt (dead values disappear), inputs and outputs keep their order,
and four rewrites apply to f32 values, tried in this order for every value (core.rs:87-115):

1. layernorm: `(x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps)` spelled out with reduce / view /
   broadcast becomes one `layernorm` value (core.rs:117-236);
2. clamp: a chain of `min(., c)` / `max(., c)` with single-valued constants becomes one min and one max
   (core.rs:238-272);
3. affine: per-channel `+ - * /` by `[1, C, 1, 1]` constants around at most one stride-1,
   shape-preserving convolution with a constant filter are folded into the filter and one bias
   (core.rs:274-287, affine.rs) - this is what turns conv + batch-norm into conv + bias;
4. division by a constant becomes multiplication by its reciprocal (core.rs:289-311).

A chain is only followed through values that are hidden (neither input nor output) and used exactly once
(core.rs:313-337), so no shared intermediate is ever recomputed or lost.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np

from .graph import BinaryOp, DType, Graph, ONE, OpKind, ReduceOp, Size, UnaryOp, Value, ValueInfo

__all__ = ["OptimizerSettings", "optimize_graph"]


@dataclass(frozen=True)
class OptimizerSettings:
    """mod.rs:8-22, defaults mod.rs:49-58."""
    optimize: bool = True                   # False: return a copy of the graph untouched
    force_bias_through_conv: bool = False   # move a pre-conv bias behind a padded conv as a full-size bias map
    fuse_layernorm: bool = True
    div_to_mul: bool = True


class _Missing(Exception):
    """An operand of the value being rebuilt has no counterpart in the new graph yet."""

    def __init__(self, old: Value):
        self.old = old


def optimize_graph(graph: Graph, settings: OptimizerSettings = OptimizerSettings()) -> Graph:
    """Returns a new, independent graph that computes the same outputs."""
    if not settings.optimize:
        return _clone(graph)
    opt = _Optimizer(graph, settings)
    for old in graph.inputs:
        info = graph[old]
        opt.map[old.index] = opt.new.input(info.shape, info.dtype)
    for old in graph.outputs:
        opt.new.output(opt.visit_completely(old))
    return opt.new


def _clone(graph: Graph) -> Graph:
    """A value-for-value copy (every value, also unreachable ones, at the same index)."""
    new = Graph()
    for info in graph.values:
        if info.kind == OpKind.INPUT:
            new.input(info.shape, info.dtype)
        else:
            new._push(dataclasses.replace(info, non_output_uses=0))
    if len(new.values) != len(graph.values):
        raise AssertionError("clone merged values")
    for i, info in enumerate(graph.values):
        new.values[i].debug_id = info.debug_id
    for out in graph.outputs:
        new.output(new._v(out.index))
    return new


class _Optimizer:
    def __init__(self, old: Graph, settings: OptimizerSettings):
        self.old = old
        self.new = Graph()
        self.settings = settings
        self.map: Dict[int, Value] = {}

    # ------------------------------------------------------------------ traversal
    def visit_completely(self, start: Value) -> Value:
        stack = [start]
        while stack:
            cur = stack[-1]
            if cur.index in self.map:
                stack.pop()
                continue
            try:
                new = self.rebuild(cur)
            except _Missing as m:
                stack.append(m.old)
                continue
            if self.old[cur].shape != self.new[new].shape:
                raise AssertionError(f"optimiser changed the shape of {cur}")
            self.map[cur.index] = new
            stack.pop()
        return self.map[start.index]

    def visit(self, old: Value) -> Value:
        new = self.map.get(old.index)
        if new is None:
            raise _Missing(old)
        return new

    def rebuild(self, old: Value) -> Value:
        info = self.old[old]
        if self.settings.optimize and info.dtype == DType.F32:
            fused = self.try_fuse(old)
            if fused is not None:
                if info.debug_id:
                    self.new.set_debug_id(fused, info.debug_id)
                return fused
        # plain copy of the operation with its operands remapped
        operands = [self.visit(self.old._v(i)) for i in info.inputs]
        copy = dataclasses.replace(info, inputs=tuple(v.index for v in operands), non_output_uses=0)
        return self.new._push(copy)

    def try_fuse(self, old: Value) -> Optional[Value]:
        if self.settings.fuse_layernorm:
            r = self.try_fuse_layernorm(old)
            if r is not None:
                return r
        for rule in (self.try_fuse_clamp, self.try_fuse_conv_affine):
            r = rule(old)
            if r is not None:
                return r
        if self.settings.div_to_mul:
            return self.try_convert_div_to_mul(old)
        return None

    def follow_if(self, start: Value, step: Callable[[ValueInfo], Optional[Value]]) -> Optional[Value]:
        """Walks up from `start` while the current value is hidden with one use and `step` accepts its
        operation; returns where the walk stopped, or None if it never left `start`."""
        cur = start
        while self.old.is_hidden_with_uses(cur, 1):
            nxt = step(self.old[cur])
            if nxt is None:
                break
            cur = nxt
        return None if cur == start else cur

    # ------------------------------------------------------------------ 1. layernorm
    def try_fuse_layernorm(self, value: Value) -> Optional[Value]:
        g = self.old
        uses: Dict[int, int] = {}

        def info_of(index: int) -> ValueInfo:
            uses[index] = uses.get(index, 0) + 1
            return g.values[index]

        def binary(info: ValueInfo, op: BinaryOp) -> bool:
            return info.kind == OpKind.BINARY and info.binary_op == op

        top = g[value]
        if not binary(top, BinaryOp.DIV):
            return None
        zeroed0, std_broadcast = top.inputs
        zeroed = info_of(zeroed0)
        if not binary(zeroed, BinaryOp.SUB):
            return None
        input0, mean_broadcast = zeroed.inputs
        mb = info_of(mean_broadcast)
        if mb.kind != OpKind.BROADCAST:
            return None
        mv = info_of(mb.inputs[0])
        if mv.kind != OpKind.VIEW:
            return None
        mean = info_of(mv.inputs[0])
        if mean.kind != OpKind.REDUCE or mean.reduce_op != ReduceOp.MEAN:
            return None
        input1, axes0 = mean.inputs[0], mean.axes
        sb = info_of(std_broadcast)
        if sb.kind != OpKind.BROADCAST:
            return None
        std = info_of(sb.inputs[0])
        if std.kind != OpKind.UNARY or std.unary_op != UnaryOp.SQRT:
            return None
        stable_var = info_of(std.inputs[0])
        if not binary(stable_var, BinaryOp.ADD):
            return None
        var_view, const_eps = stable_var.inputs
        vv = info_of(var_view)
        if vv.kind != OpKind.VIEW:
            return None
        var = info_of(vv.inputs[0])
        if var.kind != OpKind.REDUCE or var.reduce_op != ReduceOp.MEAN:
            return None
        pow_, axes1 = var.inputs[0], var.axes
        pw = info_of(pow_)
        if not binary(pw, BinaryOp.POW):
            return None
        zeroed1, const_2 = pw.inputs
        info_of(zeroed1)        # the second use of the centred value
        if input0 != input1 or zeroed0 != zeroed1 or axes0 != axes1:
            return None
        # nothing inside the pattern may be visible outside it
        if any(not g.is_hidden_with_uses(g._v(i), n) for i, n in uses.items()):
            return None
        if len(axes0) != 1:
            return None
        eps = g.as_single_const(g._v(const_eps))
        if not isinstance(eps, np.float32):
            return None
        if not g.is_const_filled_with(g._v(const_2), np.float32(2.0)):
            return None
        return self.new.layernorm(self.visit(g._v(input0)), axes0[0], float(eps))

    # ------------------------------------------------------------------ 2. clamp
    def try_fuse_clamp(self, start: Value) -> Optional[Value]:
        g = self.old
        bounds = [np.float32(-np.inf), np.float32(np.inf)]      # running [max of lower, min of upper]

        def step(info: ValueInfo) -> Optional[Value]:
            if info.kind == OpKind.BINARY and info.binary_op in (BinaryOp.MIN, BinaryOp.MAX):
                c = g.as_single_const(g._v(info.inputs[1]))
                if isinstance(c, np.float32):
                    if info.binary_op == BinaryOp.MIN:
                        bounds[1] = np.fmin(bounds[1], c)
                    else:
                        bounds[0] = np.fmax(bounds[0], c)
                    return g._v(info.inputs[0])
            return None

        old_input = self.follow_if(start, step)
        if old_input is None:
            return None
        return self.new.clamp(self.visit(old_input), bounds[0], bounds[1])

    # ------------------------------------------------------------------ 3. affine around a convolution
    def try_fuse_conv_affine(self, start: Value) -> Optional[Value]:
        g = self.old
        out_shape = g[start].shape
        if len(out_shape) != 4 or not out_shape[1].is_fixed:
            return None
        group = _AffineGroup(out_shape[1].factor)

        def step(info: ValueInfo) -> Optional[Value]:
            if info.kind == OpKind.CONV:
                filt = g.as_const(g._v(info.inputs[1]))
                if filt is None or filt.dtype != np.float32 or group.conv is not None:
                    return None
                stride_y, stride_x, pad_y, pad_x = info.conv
                k_out, c_in, kh, kw = filt.shape
                keeps_spatial = 2 * pad_y == kh - 1 and 2 * pad_x == kw - 1
                if not keeps_spatial or stride_y != 1 or stride_x != 1:
                    return None
                in_shape = g.values[info.inputs[0]].shape
                group.set_conv(filt, pad_y, pad_x, in_shape)
                return g._v(info.inputs[0])
            if info.kind == OpKind.BINARY and info.binary_op in (BinaryOp.ADD, BinaryOp.SUB, BinaryOp.MUL, BinaryOp.DIV):
                right = g.values[info.inputs[1]]
                if right.kind != OpKind.BROADCAST:
                    return None
                inner = g._v(right.inputs[0])
                want = (ONE, Size(group.current_channels), ONE, ONE)
                if g[inner].shape != want:
                    return None
                data = g.as_const(inner)
                if data is None or data.dtype != np.float32:
                    return None
                data = data.reshape(-1)
                with np.errstate(all="ignore"):
                    if info.binary_op == BinaryOp.ADD:
                        group.push(False, data)
                    elif info.binary_op == BinaryOp.SUB:
                        group.push(False, -data)
                    elif info.binary_op == BinaryOp.MUL:
                        group.push(True, data)
                    else:
                        group.push(True, np.float32(1.0) / data)
                return g._v(info.inputs[0])
            return None

        old_input = self.follow_if(start, step)
        if old_input is None:
            return None
        return group.apply(self.settings, self.new, self.visit(old_input))

    # ------------------------------------------------------------------ 4. x / const -> x * (1 / const)
    def try_convert_div_to_mul(self, start: Value) -> Optional[Value]:
        info = self.old[start]
        if info.kind != OpKind.BINARY or info.binary_op != BinaryOp.DIV:
            return None
        right = self.old.as_const(self.old._v(info.inputs[1]))
        if right is None or right.dtype != np.float32:
            return None
        with np.errstate(all="ignore"):
            inverse = self.new.constant_tensor(np.float32(1.0) / right)
        return self.new.mul(self.visit(self.old._v(info.inputs[0])), inverse)


class _AffineGroup:
    """Per-channel scale/bias operations collected while walking UP from the last value of a chain: those
    seen before the convolution is met act on its output (`after`), the rest on its input (`before`)
    (affine.rs:115-165).  Both lists are stored in walk order, i.e. reversed execution order."""

    def __init__(self, out_channels: int):
        self.after_channels = out_channels
        self.current_channels = out_channels
        self.conv: Optional[Tuple[np.ndarray, int, int, tuple]] = None
        self.before_rev: List[Tuple[bool, np.ndarray]] = []
        self.after_rev: List[Tuple[bool, np.ndarray]] = []

    def set_conv(self, filt: np.ndarray, pad_y: int, pad_x: int, in_shape: tuple):
        self.conv = (filt, pad_y, pad_x, in_shape)
        self.current_channels = filt.shape[1]

    def push(self, is_scale: bool, data: np.ndarray):
        (self.before_rev if self.conv is not None else self.after_rev).append((is_scale, data))

    @staticmethod
    def _fold(ops_rev) -> Tuple[Optional[np.ndarray], Optional[np.ndarray]]:
        """Collapse a list of per-channel ops into (scale, bias) meaning `x * scale + bias`; None = no-op
        (affine.rs:354-388)."""
        scale = bias = None
        for is_scale, data in reversed(ops_rev):
            if is_scale:
                scale = data.copy() if scale is None else scale * data
                if bias is not None:
                    bias = bias * data
            else:
                bias = data.copy() if bias is None else bias + data
        return scale, bias

    @staticmethod
    def _apply_scale_bias(graph: Graph, x: Value, scale, bias) -> Value:
        if scale is not None:
            x = graph.binary(BinaryOp.MUL, x, graph.constant_tensor(scale.reshape(1, -1, 1, 1)))
        if bias is not None:
            x = graph.binary(BinaryOp.ADD, x, graph.constant_tensor(bias.reshape(1, -1, 1, 1)))
        return x

    def apply(self, settings: OptimizerSettings, graph: Graph, x: Value) -> Value:
        after_scale, after_bias = self._fold(self.after_rev)
        if self.conv is None:
            assert not self.before_rev
            return self._apply_scale_bias(graph, x, after_scale, after_bias)
        before_scale, before_bias = self._fold(self.before_rev)
        filt, pad_y, pad_x, in_shape = self.conv
        filt = filt.copy()
        k_out, c_in = filt.shape[:2]
        if after_scale is not None:
            filt *= after_scale.reshape(k_out, 1, 1, 1)
        bias_after = None if after_bias is None else after_bias.reshape(1, k_out, 1, 1)

        # a bias in front of the convolution can move behind it when its image under the convolution
        # is known: always if it is zero, as one value per output channel without padding, as a full
        # map when forced (affine.rs:263-308)
        moved: Optional[np.ndarray] = None
        stuck = False
        if before_bias is not None and np.any(before_bias != 0.0):
            if pad_y == 0 and pad_x == 0:
                moved = np.einsum("kc,c->k", filt.sum(axis=(2, 3), dtype=np.float32), before_bias).astype(np.float32)
                moved = moved.reshape(1, k_out, 1, 1)
            elif settings.force_bias_through_conv and all(d.is_fixed for d in in_shape[2:]):
                h, w = in_shape[2].factor, in_shape[3].factor
                moved = _convolve_constant(np.broadcast_to(before_bias.reshape(1, c_in, 1, 1), (1, c_in, h, w)),
                                           filt, pad_y, pad_x)
            else:
                stuck = True
        if stuck:
            x = self._apply_scale_bias(graph, x, before_scale, before_bias)
            x = graph.conv(x, graph.constant_tensor(filt), 1, 1, pad_y, pad_x)
            if bias_after is not None:
                x = graph.binary(BinaryOp.ADD, x, graph.constant_tensor(bias_after))
            return x
        total_bias = bias_after if moved is None else (moved if bias_after is None else moved + bias_after)
        if before_scale is not None:
            filt *= before_scale.reshape(1, c_in, 1, 1)
        x = graph.conv(x, graph.constant_tensor(filt), 1, 1, pad_y, pad_x)
        if total_bias is not None:
            x = graph.binary(BinaryOp.ADD, x, graph.constant_tensor(np.ascontiguousarray(total_bias, dtype=np.float32)))
        return x


def _convolve_constant(x: np.ndarray, filt: np.ndarray, pad_y: int, pad_x: int) -> np.ndarray:
    """Stride-1 zero-padded cross-correlation of a constant `[1, C, H, W]` map, f32."""
    _, c, h, w = x.shape
    k, _, kh, kw = filt.shape
    padded = np.zeros((c, h + 2 * pad_y, w + 2 * pad_x), np.float32)
    padded[:, pad_y:pad_y + h, pad_x:pad_x + w] = x[0]
    oh, ow = h + 2 * pad_y - kh + 1, w + 2 * pad_x - kw + 1
    out = np.zeros((k, oh, ow), np.float32)
    for dy in range(kh):
        for dx in range(kw):
            out += np.einsum("kc,chw->khw", filt[:, :, dy, dx], padded[:, dy:dy + oh, dx:dx + ow]).astype(np.float32)
    return out.reshape(1, k, oh, ow)
