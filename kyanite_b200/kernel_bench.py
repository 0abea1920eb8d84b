"""Per-kernel measurements at the sizes of the named workloads: each case is a one-operator graph (plus
the epilogue or scalar chain that fuses into it), run through `CudaExecutor`; every planned step is timed
with CUDA events (`kn_executor_time_step`, the step launched back to back) and reported as achieved GB/s
over its algorithmic bytes (memory-bound steps) or TFLOP/s over its FLOP (contractions).

    python -m kyanite_b200.kernel_bench                 # all cases, one JSON line per step
    python -m kyanite_b200.kernel_bench --case softmax  # one case (this is what the ncu captures run)

Working sets are several times the 126 MB L2, so back-to-back launches still stream from HBM.  Peaks come
from MEASURED_PEAKS.json at the repository root when present (copy bandwidth, bf16 GEMM burst; TF32 is
taken as half the bf16 figure, f16 operands as the bf16 figure itself), else the fallback 6650 GB/s / 1590 TFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import numpy as np

from .executor import MATH_TF32, CudaExecutor
from .graph import BATCH, BinaryOp, DType, Graph, ReduceOp, UnaryOp, shape


def _const(g, rng, *s, scale=0.02):
    return g.constant_tensor((rng.standard_normal(s) * scale).astype(np.float32))


def case_gelu(rng):
    """BERT feed-forward activation: bias + GELU(erf) over [16384, 3072] as one fused elementwise step."""
    g = Graph()
    x = g.input(shape(16384, 3072))
    y = g.add(x, _const(g, rng, 1, 3072))
    inner = g.unary(UnaryOp.ERF, g.mul(y, g.scalar(1.0 / math.sqrt(2.0))))
    g.output(g.mul(g.mul(y, g.scalar(0.5)), g.add(inner, g.scalar(1.0))))
    return g, 0, [rng.standard_normal((16384, 3072)).astype(np.float32)]


def case_residual_add(rng):
    """Residual add of two [16384, 3072] tensors."""
    g = Graph()
    a = g.input(shape(16384, 3072))
    b = g.input(shape(16384, 3072))
    g.output(g.add(a, b))
    return g, 0, [rng.standard_normal((16384, 3072)).astype(np.float32) for _ in range(2)]


def case_softmax(rng):
    """BERT attention probabilities: softmax(scores / 8) over [196608, 512] (32 x 12 heads x 512 queries)."""
    g = Graph()
    x = g.input(shape(196608, 512))
    g.output(g.softmax(g.mul(x, g.scalar(0.125)), 1))
    return g, 0, [rng.standard_normal((196608, 512)).astype(np.float32)]


def case_softmax_long(rng):
    """LLaMA prefill attention rows: softmax over [65536, 2048]."""
    g = Graph()
    x = g.input(shape(65536, 2048))
    g.output(g.softmax(x, 1))
    return g, 0, [rng.standard_normal((65536, 2048)).astype(np.float32)]


def case_layernorm(rng):
    """Post-LN with residual: layernorm(a + b) over [262144, 768] (16 BERT batches of 32 x 512 tokens)."""
    g = Graph()
    a = g.input(shape(262144, 768))
    b = g.input(shape(262144, 768))
    g.output(g.layernorm(g.add(a, b), 1, 1e-12))
    return g, 0, [rng.standard_normal((262144, 768)).astype(np.float32) for _ in range(2)]


def case_layernorm_group(rng):
    """A group norm of the UNet-shaped graph at batch 2, as the layernorm it is planned as: 64 rows (2 images x 32
    groups) of 81 920 elements.  21 MB in and out: the tensor stays in L2, the time is what counts (one CTA per row
    sweeping three times took 193 us)."""
    g = Graph()
    x = g.input(shape(64, 81920))
    g.output(g.layernorm(x, 1, 1e-5))
    return g, 0, [rng.standard_normal((64, 81920)).astype(np.float32)]


def case_reduce(rng):
    """RMSNorm statistic: mean of squares over the last axis of [65536, 4096]."""
    g = Graph()
    x = g.input(shape(65536, 4096))
    g.output(g.reduce(g.pow(x, g.scalar(2.0)), [1], ReduceOp.MEAN))
    return g, 0, [rng.standard_normal((65536, 4096)).astype(np.float32)]


def case_gather(rng):
    """Embedding lookup: 262144 token ids into a [30522, 768] table."""
    g = Graph()
    ids = g.input(shape(262144), DType.I32)
    g.output(g.gather(_const(g, rng, 30522, 768), 0, ids))
    return g, 0, [rng.integers(0, 30522, 262144).astype(np.int32)]


def case_permute_copy(rng):
    """Head split: [32, 512, 12, 64] -> [32, 12, 512, 64] materialised (a strided copy)."""
    g = Graph()
    x = g.input(shape(256, 512, 12, 64))
    y = g.permute(x, [0, 2, 1, 3])
    g.output(g.add(y, g.scalar(1.0)))
    return g, 0, [rng.standard_normal((256, 512, 12, 64)).astype(np.float32)]


def _linear_case(m, n, k, bias=True, relu=False, gelu=False):
    def build(rng):
        g = Graph()
        x = g.input(shape(m, k))
        y = g.linear(x, _const(g, rng, n, k))
        if bias:
            y = g.add(y, _const(g, rng, 1, n))
        if relu:
            y = g.relu(y)
        if gelu:
            gate = g.add(g.unary(UnaryOp.ERF, g.mul(y, g.scalar(1.0 / math.sqrt(2.0)))), g.scalar(1.0))
            y = g.mul(g.mul(y, g.scalar(0.5)), gate)
        g.output(y)
        return g, 0, [rng.standard_normal((m, k)).astype(np.float32)]
    build.__doc__ = (f"Linear layer [{m}, {k}] x [{k}, {n}]" + (" + bias" if bias else "") + (" + relu" if relu else "") +
                     (" + GELU(erf) in the epilogue" if gelu else ""))
    return build


def case_attention_scores(rng):
    """BERT attention scores: 384 x ([512, 64] . [64, 512])."""
    g = Graph()
    q = g.input(shape(384, 512, 64))
    k = g.input(shape(384, 512, 64))
    g.output(g.batched_mat_mul(q, g.permute(k, [0, 2, 1])))
    return g, 0, [rng.standard_normal((384, 512, 64)).astype(np.float32) for _ in range(2)]


def case_attention_softmax(rng):
    """BERT attention scores with their softmax: 384 x softmax([512, 64] . [64, 512] / 8), one fused step."""
    g = Graph()
    q = g.input(shape(384, 512, 64))
    k = g.input(shape(384, 512, 64))
    scores = g.mul(g.batched_mat_mul(q, g.permute(k, [0, 2, 1])), g.scalar(0.125))
    g.output(g.softmax(scores, 2))
    return g, 0, [rng.standard_normal((384, 512, 64)).astype(np.float32) for _ in range(2)]


def case_attention(rng):
    """BERT attention for 384 heads of 512 tokens: softmax([512, 64] . [64, 512] / 8) . [512, 64] as one fused step
    (V arrives as [384, 64, 512], keys contiguous, as the planner's transposing copy leaves it).  With KN_ATTN_TRACE=1
    in the environment the kernel's per-item phase clocks are printed at exit."""
    g = Graph()
    q = g.input(shape(384, 512, 64))
    k = g.input(shape(384, 512, 64))
    vt = g.input(shape(384, 64, 512))
    scores = g.mul(g.batched_mat_mul(q, g.permute(k, [0, 2, 1])), g.scalar(0.125))
    g.output(g.batched_mat_mul(g.softmax(scores, 2), g.permute(vt, [0, 2, 1])))
    r = [rng.standard_normal((384, 512, 64)).astype(np.float32) for _ in range(2)]
    return g, 0, r + [rng.standard_normal((384, 64, 512)).astype(np.float32)]


def case_conv_trunk(rng):
    """One trunk convolution of the tower on its own: 3x3, 128 -> 128, batch 256, 8x8, + bias + relu."""
    g = Graph()
    x = g.input(shape(BATCH, 128, 8, 8))
    y = g.add(g.conv(x, _const(g, rng, 128, 128, 3, 3), 1, 1, 1, 1), _const(g, rng, 1, 128, 1, 1))
    g.output(g.relu(y))
    return g, 256, [rng.standard_normal((256, 128, 8, 8)).astype(np.float32)]


def case_tower(rng):
    """The whole ResNet tower of the headline benchmark at batch 256: its trunk runs as one `ConvChain` step.
    With KN_CHAIN_TRACE=1 in the environment the kernel's per-layer phase clocks are printed at exit."""
    from .configs import resnet_tower
    g, make_inputs = resnet_tower()
    return g, 256, make_inputs(256, 3)


def case_conv_unet(rng):
    """UNet-sized convolution: 3x3, 320 -> 320, batch 8, 64x64, + bias."""
    g = Graph()
    x = g.input(shape(BATCH, 320, 64, 64))
    g.output(g.add(g.conv(x, _const(g, rng, 320, 320, 3, 3), 1, 1, 1, 1), _const(g, rng, 1, 320, 1, 1)))
    return g, 8, [rng.standard_normal((8, 320, 64, 64)).astype(np.float32)]


def _conv_case(n, c, h, w, k, r, stride, pad, doc):
    def build(rng):
        g = Graph()
        x = g.input(shape(BATCH, c, h, w))
        y = g.conv(x, _const(g, rng, k, c, r, r), stride, stride, pad, pad)
        g.output(g.add(y, _const(g, rng, 1, k, 1, 1)))
        return g, n, [rng.standard_normal((n, c, h, w)).astype(np.float32)]
    build.__doc__ = doc
    return build


def case_transpose(rng):
    """Value matrices of 384 attention heads made K-contiguous: [384, 512, 64] -> [384, 64, 512] (a transposing copy)."""
    g = Graph()
    x = g.input(shape(384, 512, 64))
    g.output(g.view(g.permute(x, [0, 2, 1]), shape(384 * 64 * 512)))
    return g, 0, [rng.standard_normal((384, 512, 64)).astype(np.float32)]


def _linear_f16_case(m, n, k):
    def build(rng):
        g = Graph()
        x = g.input(shape(m, k), DType.F16)
        w = g.constant_tensor((rng.standard_normal((n, k)) * 0.02).astype(np.float16))
        g.output(g.linear(x, w))
        return g, 0, [rng.standard_normal((m, k)).astype(np.float16)]
    build.__doc__ = f"Linear layer [{m}, {k}] x [{k}, {n}] in f16 storage, f32 accumulation (kind::f16 tensor cores)"
    return build


def case_softmax_f16_masked(rng):
    """LLaMA prefill attention probabilities in f16: softmax(scores / sqrt(128) + causal mask) over [32 x 2048, 2048]."""
    g = Graph()
    x = g.input(shape(32, 2048, 2048), DType.F16)
    mask = g.constant_tensor(np.triu(np.full((2048, 2048), -np.inf, np.float16), 1).reshape(1, 2048, 2048))
    g.output(g.softmax(g.add(g.mul(x, g.scalar(1.0 / math.sqrt(128.0), DType.F16)), mask), 2))
    return g, 0, [rng.standard_normal((32, 2048, 2048)).astype(np.float16)]


def case_rmsnorm_f16(rng):
    """LLaMA RMS norm in f16 storage, the pow / mean / sqrt / div / mul subgraph as one step: [16384, 4096]."""
    g = Graph()
    x = g.input(shape(16384, 4096), DType.F16)
    t = g.value_cast(x, DType.F32)
    ms = g.view(g.reduce(g.pow(t, g.scalar(2.0)), [1], ReduceOp.MEAN), shape(16384, 1))
    y = g.mul(g.binary(BinaryOp.DIV, t, g.unary(UnaryOp.SQRT, g.add(ms, g.scalar(1e-6)))),
              g.constant_tensor((1 + 0.02 * rng.standard_normal((1, 4096))).astype(np.float32)))
    g.output(g.value_cast(y, DType.F16))
    return g, 0, [rng.standard_normal((16384, 4096)).astype(np.float16)]


def case_swiglu_f16(rng):
    """LLaMA feed-forward gate in f16: gate * sigmoid(gate) * up over [8192, 11008]."""
    g = Graph()
    a = g.input(shape(8192, 11008), DType.F16)
    b = g.input(shape(8192, 11008), DType.F16)
    g.output(g.mul(g.mul(a, g.sigmoid(a)), b))
    return g, 0, [rng.standard_normal((8192, 11008)).astype(np.float16) for _ in range(2)]


def case_residual_add_f16(rng):
    """Residual add of two f16 [16384, 4096] tensors."""
    g = Graph()
    a = g.input(shape(16384, 4096), DType.F16)
    b = g.input(shape(16384, 4096), DType.F16)
    g.output(g.add(a, b))
    return g, 0, [rng.standard_normal((16384, 4096)).astype(np.float16) for _ in range(2)]


CASES = {
    "gelu": case_gelu,
    "residual_add": case_residual_add,
    "softmax": case_softmax,
    "softmax_long": case_softmax_long,
    "layernorm": case_layernorm,
    "layernorm_group": case_layernorm_group,
    "reduce": case_reduce,
    "gather": case_gather,
    "permute_copy": case_permute_copy,
    "linear_bert_qkv": _linear_case(16384, 768, 768),
    "linear_bert_ffn": _linear_case(16384, 3072, 768),
    "linear_bert_ffn_gelu": _linear_case(16384, 3072, 768, gelu=True),
    "linear_llama_proj": _linear_case(2048, 4096, 4096, bias=False),
    "linear_llama_ffn": _linear_case(2048, 11008, 4096, bias=False),
    "attention_scores": case_attention_scores,
    "attention_softmax": case_attention_softmax,
    "attention": case_attention,
    "tower": case_tower,
    "conv_trunk": case_conv_trunk,
    "conv_unet": case_conv_unet,
    "conv_unet_down": _conv_case(8, 320, 64, 64, 320, 3, 2, 1, "UNet downsampling convolution: 3x3 stride 2, 320 -> 320, batch 8, 64x64 (Im2col + matmul)"),
    "conv_unet_mid": _conv_case(2, 1280, 8, 8, 1280, 3, 1, 1, "UNet middle-block convolution: 3x3, 1280 -> 1280, batch 2, 8x8 (Im2col + split-K matmul)"),
    "conv_unet_pointwise": _conv_case(8, 320, 64, 64, 320, 1, 1, 0, "UNet 1x1 projection: 320 -> 320, batch 8, 64x64 (Im2col as transpose + matmul)"),
    "transpose": case_transpose,
    "linear_llama_proj_f16": _linear_f16_case(2048, 4096, 4096),
    "linear_llama_ffn_f16": _linear_f16_case(2048, 11008, 4096),
    "linear_llama_down_f16": _linear_f16_case(2048, 4096, 11008),
    "softmax_f16_masked": case_softmax_f16_masked,
    "rmsnorm_f16": case_rmsnorm_f16,
    "swiglu_f16": case_swiglu_f16,
    "residual_add_f16": case_residual_add_f16,
}


def _is_f16(name: str) -> bool:
    return "f16" in name


def load_peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"] / 2.0, "measured"
    return 6650.0, 1590.0 / 2.0, "fallback"


def run_case(name: str, launches: int, device: int):
    graph, batch, inputs = CASES[name](np.random.Generator(np.random.PCG64(1)))
    hbm, tf32, source = load_peaks()
    lines = []
    with CudaExecutor(device, graph, batch, math_mode=MATH_TF32) as ex:
        ex.evaluate(inputs)
        ex.set_profile(True)
        ex.run_async()
        steps = []
        for line in ex.last_profile().splitlines():
            parts = line.split()
            if parts and parts[0].isdigit():
                steps.append((int(parts[0]), parts[1], float(parts[3]), float(parts[4]), " ".join(parts[5:])))
        ex.set_profile(False)
        for idx, kind, alg_bytes, flops, desc in steps:
            us = ex.time_step(idx, launches)
            rec = {"case": name, "step": idx, "kind": kind, "desc": desc, "us": round(us, 2)}
            if flops > 0:
                # f16 operands: the dense f16 / bf16 rate (the measured bf16 GEMM figure); f32 storage: TF32, half of it
                peak = 2.0 * tf32 if _is_f16(name) else tf32
                rec.update(bound="tensor", achieved=round(flops / us / 1e6, 1), unit="TFLOP/s", peak=peak,
                           frac=round(flops / us / 1e6 / peak, 3))
            else:
                rec.update(bound="hbm", achieved=round(alg_bytes / us / 1e3, 1), unit="GB/s", peak=hbm,
                           frac=round(alg_bytes / us / 1e3 / hbm, 3), bytes=int(alg_bytes))
            rec["peak_source"] = source
            lines.append(rec)
    return lines


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kernel_bench", description=__doc__.splitlines()[0])
    ap.add_argument("--case", action="append", choices=sorted(CASES), help="case to run (repeatable); default all")
    ap.add_argument("--launches", type=int, default=20)
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    for name in args.case or list(CASES):
        for rec in run_case(name, args.launches, args.device):
            print(json.dumps(rec), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
