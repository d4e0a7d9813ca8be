"""Host-side mirror of the reference's weight store and of the ``linear_proj`` dispatcher.

reference: ``Tensor`` / ``WeightStore`` / dtype tags in Infer-engine/include/types.h:8-35,
88-95,145-168; ``linear_proj`` and ``linear_proj_pair_same_input`` in
Infer-engine/cuda/decoder.cu:861-978; ``prefer_nvfp4_cutlass`` at :142-151.

Differences that are deliberate: name lookups go through a dict instead of a linear string
scan, and scalar tensors (``weight_scale_2``, ``input_scale``) are read from the device once
and cached by name (the reference caches them by device pointer, decoder.cu:165-194).
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from . import ops

DTYPE_FP32 = 0
DTYPE_BF16 = 1
DTYPE_FP16 = 2
DTYPE_UINT8 = 3   # packed FP4 (2 values per byte)
DTYPE_FP8 = 4     # E4M3 block scales

_TORCH_TO_TAG = {torch.float32: DTYPE_FP32, torch.bfloat16: DTYPE_BF16, torch.float16: DTYPE_FP16,
                 torch.uint8: DTYPE_UINT8, torch.float8_e4m3fn: DTYPE_FP8}

#: safetensors dtype string -> tag (Infer-engine/src/safetensors.c:48-55)
SAFETENSORS_DTYPES = {"F32": DTYPE_FP32, "BF16": DTYPE_BF16, "F16": DTYPE_FP16, "U8": DTYPE_UINT8,
                      "F8_E4M3": DTYPE_FP8}


@dataclass
class Tensor:
    data: torch.Tensor
    dtype: int

    @property
    def shape(self):
        return tuple(self.data.shape)


@dataclass
class WeightStore:
    tensors: Dict[str, Tensor] = field(default_factory=dict)
    _scalars: Dict[str, float] = field(default_factory=dict)

    def add(self, name: str, data: torch.Tensor, dtype: Optional[int] = None):
        if dtype is None:
            dtype = _TORCH_TO_TAG[data.dtype]
        self.tensors[name] = Tensor(data, dtype)
        self._scalars.pop(name, None)

    def get(self, name: str) -> Optional[Tensor]:
        """``ws_get``: None when absent."""
        return self.tensors.get(name)

    def require(self, name: str) -> Tensor:
        """``wget`` (decoder.cu:849-854): a missing weight is fatal."""
        t = self.tensors.get(name)
        if t is None:
            raise KeyError(f"Weight not found: {name}")
        return t

    def scalar(self, name: str, fallback: float) -> float:
        """``decoder_scalar_read_cached``: one device read per scalar, then cached."""
        if name in self._scalars:
            return self._scalars[name]
        t = self.tensors.get(name)
        if t is None:
            return fallback
        v = float(t.data.reshape(-1)[0].float().item())
        self._scalars[name] = v
        return v


def prefer_nvfp4_cutlass() -> bool:
    """``GLMASR_USE_CUTLASS_NVFP4`` set and not "0" selects the W4A4 path (decoder.cu:142-151).
    Read on every call here so tests can flip it; the reference caches the first read."""
    env = os.environ.get("GLMASR_USE_CUTLASS_NVFP4", "")
    return bool(env) and env != "0"


_warned = False


def _warn_fallback():
    global _warned
    if not _warned:
        print("GLMASR_USE_CUTLASS_NVFP4 requested but native path is not ready, falling back to bf16 dequant path",
              file=sys.stderr)
        _warned = True


def proj_names(prefix: str):
    """The five tensor names of one projection (decoder.cu:1069-1073)."""
    return (f"{prefix}.weight", f"{prefix}.weight_scale", f"{prefix}.weight_scale_2", f"{prefix}.input_scale",
            f"{prefix}.pre_quant_scale")


def linear_proj(ws: WeightStore, x: torch.Tensor, w_name: str, ws_name: str, ws2_name: str, in_name: str,
                pre_name: str, M: int, N: int, K: int, use_native_nvfp4: bool = True,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """reference: linear_proj, Infer-engine/cuda/decoder.cu:861-921.  bf16 weight -> bf16_linear;
    packed FP4 weight -> nvfp4_linear when requested by the environment (falling back with one
    warning if it returns -1), else fp4_linear."""
    tw = ws.require(w_name)
    tws = ws.get(ws_name)
    tpre = ws.get(pre_name)
    input_scale = ws.scalar(in_name, 1.0)
    global_scale = ws.scalar(ws2_name, 1.0)
    x = x[:M]
    if tw.dtype == DTYPE_BF16:
        return ops.bf16_linear(x, tw.data)
    if tw.dtype != DTYPE_UINT8:
        raise TypeError(f"Unsupported decoder weight dtype {tw.dtype} for {w_name}")
    scales = tws.data.view(torch.uint8) if tws is not None else None
    pre = tpre.data if tpre is not None else None
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if use_native_nvfp4 and prefer_nvfp4_cutlass():
        status = ops.nvfp4_linear(out, x, tw.data, scales, input_scale, global_scale, pre, None, M, N, K)
        if status == 0:
            return out
        _warn_fallback()
    return ops.fp4_linear(x, tw.data, scales, global_scale, pre, None, out=out)


def linear_proj_pair_same_input(ws: WeightStore, x: torch.Tensor, prefix0: str, prefix1: str, M: int, N: int,
                                K: int, epilogue: int = ops.EPI_STORE) -> Optional[torch.Tensor]:
    """reference: linear_proj_pair_same_input, Infer-engine/cuda/decoder.cu:923-978: two
    same-input projections as one GEMM writing [M, 2N].  Returns None ("0" in the reference)
    when the pair cannot be fused there: mixed dtypes, or either has a pre_quant_scale.
    The reference never takes the W4A4 path here; this one does when the environment asks
    for it and both members share their input_scale."""
    w0, s0, g0, i0, p0 = proj_names(prefix0)
    w1, s1, g1, i1, p1 = proj_names(prefix1)
    tw0, tw1 = ws.require(w0), ws.require(w1)
    if tw0.dtype == DTYPE_BF16 and tw1.dtype == DTYPE_BF16:
        return ops.bf16_linear(x[:M], torch.cat([tw0.data, tw1.data], dim=0))
    if tw0.dtype != DTYPE_UINT8 or tw1.dtype != DTYPE_UINT8:
        return None
    if ws.get(p0) is not None or ws.get(p1) is not None:
        return None
    a = ops.Fp4Tensor(tw0.data, ws.require(s0).data.view(torch.uint8), ws.scalar(g0, 1.0), ws.scalar(i0, 1.0))
    b = ops.Fp4Tensor(tw1.data, ws.require(s1).data.view(torch.uint8), ws.scalar(g1, 1.0), ws.scalar(i1, 1.0))
    mode = ops.MODE_W4A16
    if prefer_nvfp4_cutlass() and a.input_scale == b.input_scale:
        mode = ops.MODE_W4A4
    return ops.fp4_linear_fused(mode, x[:M], [a, b], epilogue=epilogue, input_scale=a.input_scale)


def linear_proj_triple_same_input_bf16(ws: WeightStore, x: torch.Tensor, w0_name: str, w1_name: str, w2_name: str,
                                       M: int, N0: int, N1: int, K: int) -> Optional[torch.Tensor]:
    """reference: linear_proj_triple_same_input_bf16, Infer-engine/cuda/decoder.cu:980-1013: the bf16-only
    q|k|v fusion, one GEMM writing [M, N0 + 2 N1] from the three weights laid end to end.  Returns None
    ("0" in the reference) unless all three weights are bf16 -- FP4 weights are fused by
    ops.fp4_linear_fused instead."""
    tws = [ws.require(n) for n in (w0_name, w1_name, w2_name)]
    if any(t.dtype != DTYPE_BF16 for t in tws):
        return None
    w = torch.cat([tws[0].data[:N0, :K], tws[1].data[:N1, :K], tws[2].data[:N1, :K]], dim=0).contiguous()
    return ops.bf16_linear(x[:M], w)


_compare_done = False


def should_compare_nvfp4_once() -> bool:
    """reference: should_compare_nvfp4_once, Infer-engine/cuda/decoder.cu:196-204 (GLMASR_NVFP4_COMPARE_ONCE=1)."""
    return os.environ.get("GLMASR_NVFP4_COMPARE_ONCE", "")[:1] == "1"


def compare_nvfp4_once(x: torch.Tensor, w_packed: torch.Tensor, w_scales: torch.Tensor, input_scale: float,
                       global_scale: float, pre_quant_scale: Optional[torch.Tensor], M: int, N: int, K: int,
                       tag: str, out: Optional[torch.Tensor] = None, force: bool = False):
    """reference: compare_nvfp4_once, Infer-engine/cuda/decoder.cu:206-275 -- the engine's only in-tree numerical
    check: run one projection through nvfp4_linear (native) and fp4_linear (fallback), report the largest and
    the mean absolute difference on stderr in the reference's format, and leave the native result in ``out``.
    Runs once per process and only when GLMASR_NVFP4_COMPARE_ONCE=1 (``force`` skips both conditions).
    Returns the statistics as a dict, or None when it did not run or the native path refused the shape."""
    global _compare_done
    if not force and (_compare_done or not should_compare_nvfp4_once()):
        return None
    _compare_done = True
    native = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if ops.nvfp4_linear(native, x[:M], w_packed, w_scales, input_scale, global_scale, pre_quant_scale, None, M, N, K) != 0:
        sys.stderr.write(f"NVFP4_COMPARE {tag} native_status=fail\n")
        return None
    fallback = ops.fp4_linear(x[:M], w_packed, w_scales, global_scale, pre_quant_scale, None)
    a, b = native.float().flatten(), fallback.float().flatten()
    d = (a - b).abs()
    idx = int(torch.argmax(d).item())
    stats = {"max_abs": float(d[idx].item()), "mean_abs": float(d.double().mean().item()), "idx": idx,
             "native": float(a[idx].item()), "fallback": float(b[idx].item())}
    sys.stderr.write("NVFP4_COMPARE %s M=%d N=%d K=%d max_abs=%.6f mean_abs=%.6f idx=%d native=%.6f fallback=%.6f\n"
                     % (tag, M, N, K, stats["max_abs"], stats["mean_abs"], idx, stats["native"], stats["fallback"]))
    if out is not None:
        out[:M, :N].copy_(native)
    return stats
