"""Seeded synthetic FP4 weights and activations with the shapes of the benchmark
configurations (no checkpoint can be downloaded here).

The weight quantiser is builder-defined -- the reference only ever loads pre-quantised
checkpoints -- and uses the rounding rules of the reference's activation quantiser
(Infer-engine/cuda/nvfp4_cutlass.cu:45-86): g = amax(W)/(6*448); per 16-K block
s = e4m3(amax_blk/(6 g)); q = e2m1(w/(float(s) g)), round-to-nearest-even, saturating;
even k in the low nibble.  Runs on whatever device the input lives on.
"""
from __future__ import annotations

import math

import torch

from .ops import Fp4Tensor

# round-to-nearest-even thresholds between the e2m1 magnitudes {0,.5,1,1.5,2,3,4,6}: a value v
# maps to the number of thresholds strictly below it.  Ties go to the even code, so the
# thresholds of odd->even upward ties (0.75, 1.75, 3.5) are nudged one ulp down.
_E2M1_EDGES = [0.25, math.nextafter(0.75, 0.0), 1.25, math.nextafter(1.75, 0.0), 2.5, math.nextafter(3.5, 0.0), 5.0]


def e2m1_encode(y: torch.Tensor) -> torch.Tensor:
    edges = torch.tensor(_E2M1_EDGES, dtype=torch.float64, device=y.device)
    code = torch.bucketize(y.abs().double(), edges, right=False).to(torch.uint8)
    return code | (torch.signbit(y).to(torch.uint8) << 3)


def quantize_weight(w: torch.Tensor):
    """fp32 [N, K] -> (packed u8 [N, K/2], scales u8 [N, K/16], global fp32)."""
    w = w.float()
    N, K = w.shape
    assert K % 16 == 0
    g = (w.abs().max() / (6.0 * 448.0)).float()
    if float(g) == 0.0:
        g = torch.ones((), device=w.device)
    wb = w.view(N, K // 16, 16)
    amax = wb.abs().amax(dim=-1)
    s8 = (amax / (6.0 * g)).float().to(torch.float8_e4m3fn)
    s = s8.float()
    denom = (s * g).unsqueeze(-1)
    y = torch.where(denom > 0, wb / denom, torch.zeros_like(wb))
    q = e2m1_encode(y).view(N, K)
    packed = (q[:, 0::2] & 0xF) | ((q[:, 1::2] & 0xF) << 4)
    return packed.contiguous(), s8.view(torch.uint8).contiguous(), float(g)


def seeded_weight(N: int, K: int, seed: int, device="cuda") -> Fp4Tensor:
    """W ~ N(0, 0.02), quantised; generated on the CPU generator so every device sees the same bits."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.randn((N, K), generator=gen, dtype=torch.float32) * 0.02
    w = w.to(device)
    packed, scales, g = quantize_weight(w)
    return Fp4Tensor(packed, scales, g)


def seeded_weight_fast(N: int, K: int, seed: int, device="cuda") -> Fp4Tensor:
    """Same distribution, generated with the device's own generator (much faster for the 1.4 G
    weights of a 28-layer decoder; bits differ from seeded_weight)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    w = torch.randn((N, K), generator=gen, dtype=torch.float32, device=device) * 0.02
    packed, scales, g = quantize_weight(w)
    return Fp4Tensor(packed, scales, g)


def seeded_activation(M: int, K: int, seed: int, device="cuda") -> torch.Tensor:
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn((M, K), generator=gen, dtype=torch.float32).to(torch.bfloat16).to(device)


def default_input_scale(x: torch.Tensor) -> float:
    """Per-tensor activation scale of the W4A4 path: amax(x)/(6*448)."""
    a = float(x.float().abs().max())
    return a / (6.0 * 448.0) if a > 0 else 1.0


def mel_filterbank(sr: int = 16000, n_fft: int = 400, n_mels: int = 128, device="cuda") -> torch.Tensor:
    """A Slaney-style mel filterbank (linear below 1 kHz, logarithmic above, area-normalised triangles) in the form the
    log-mel front end takes it: float32 [n_fft / 2 + 1, n_mels], i.e. transposed.  Stands in for the filter file the
    engine loads at start-up (Infer-engine/src/main.c:271-309), which is not part of the reference tree."""
    import numpy as np

    def hz_to_mel(f):
        f = np.asarray(f, np.float64)
        return np.where(f >= 1000.0, 15.0 + np.log(np.maximum(f, 1e-12) / 1000.0) / (np.log(6.4) / 27.0), f / (200.0 / 3.0))

    def mel_to_hz(m):
        m = np.asarray(m, np.float64)
        return np.where(m >= 15.0, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3.0))

    freqs = np.linspace(0.0, sr / 2.0, n_fft // 2 + 1)
    pts = mel_to_hz(np.linspace(hz_to_mel(0.0), hz_to_mel(sr / 2.0), n_mels + 2))
    ramps = pts[:, None] - freqs[None, :]
    w = np.maximum(0.0, np.minimum(-ramps[:-2] / np.diff(pts)[:-1, None], ramps[2:] / np.diff(pts)[1:, None]))
    w *= (2.0 / (pts[2:n_mels + 2] - pts[:n_mels]))[:, None]
    return torch.from_numpy(np.ascontiguousarray(w.T.astype(np.float32))).to(device)
