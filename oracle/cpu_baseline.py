"""CPU timing leg: the reference's W4A16 fallback arithmetic (Infer-engine/cuda/kernels.cu:1297-1318:
dequantise the WHOLE weight to bf16 on every call, then x @ W^T with fp32 accumulation, bf16 out)
restated with torch CPU ops on all host threads, for the four projections of one decoder layer.

TEST / BENCHMARK INFRASTRUCTURE ONLY ("port" baseline): the reference has no CPU implementation
of this path.  Used by bench.py's cpu_baseline leg and by `bench.py --impl reference`.
"""
from __future__ import annotations

import os
import time

import numpy as np
import torch

import fp4_oracle as o


def _dequant_bf16(pw, sw, g):
    """Vectorised a2 (kernels.cu:188-232) in torch: lut[nibble]*e4m3(scale)*global -> bf16."""
    lut = torch.from_numpy(o.E2M1_LUT)
    tab = torch.from_numpy(o.E4M3_TABLE)
    p = pw.to(torch.int64)
    q = torch.stack([p & 0xF, p >> 4], dim=-1).reshape(pw.shape[0], -1)
    w = lut[q] * tab[sw.to(torch.int64)].repeat_interleave(16, dim=1)
    return (w * g).to(torch.bfloat16)


def _linear(x_bf16, w):
    pw, sw, g = w
    wd = _dequant_bf16(pw, sw, g)                       # every call, as the reference does
    return (x_bf16.float() @ wd.float().T).to(torch.bfloat16)


def layer_proj_cpu(x_bf16, lw):
    """q|k|v, o + residual, gate|up + SiLU-gate, down + residual (attention stand-in = q slice)."""
    q = _linear(x_bf16, lw["q"])
    _linear(x_bf16, lw["k"])
    _linear(x_bf16, lw["v"])
    h1 = (_linear(q, lw["o"]).float() + x_bf16.float()).to(torch.bfloat16)
    g = _linear(h1, lw["gate"]).float()
    u = _linear(h1, lw["up"]).float()
    act = ((g * (1.0 / (1.0 + torch.exp(-g)))) * u).to(torch.bfloat16)
    return (_linear(act, lw["down"]).float() + h1.float()).to(torch.bfloat16)


def make_layer(hidden, ffn, kv, layer=0):
    shapes = [("q", hidden, hidden), ("k", kv, hidden), ("v", kv, hidden), ("o", hidden, hidden),
              ("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)]
    # same seeded weights as the GPU arm (the package's generator, run on the CPU)
    from glm_asr_stack_b200 import synth
    lw = {}
    for i, (n, N, K) in enumerate(shapes):
        t = synth.seeded_weight(N, K, 1000 * layer + i, device="cpu")
        lw[n] = (t.w_packed, t.w_scales, float(t.w_global_scale))
    return lw


def layer_flops(M, hidden, ffn, kv):
    return 2.0 * M * (hidden * (hidden + 2 * kv) + hidden * hidden + 2 * ffn * hidden + hidden * ffn)


def time_layer(M_sample, hidden=2048, ffn=6144, kv=512, steps=1, warmup=0):
    """Returns (seconds per step on the sample, threads used)."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    lw = make_layer(hidden, ffn, kv)
    x = torch.from_numpy(o.bf16_bits_to_f32(o.seeded_activation(M_sample, hidden, 1))).to(torch.bfloat16)
    for _ in range(warmup):
        layer_proj_cpu(x, lw)
    t0 = time.perf_counter()
    for _ in range(steps):
        layer_proj_cpu(x, lw)
    return (time.perf_counter() - t0) / max(steps, 1), threads
