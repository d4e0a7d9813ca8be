"""Helpers shared by the GPU tests: numpy bf16-bit arrays <-> torch CUDA tensors, tolerances."""
import numpy as np
import torch


def to_dev_bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def to_dev_u8(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint8)).cuda()


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def ulp_diff(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in bf16 ulps between two finite bf16 arrays (sign-magnitude aware)."""
    def key(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)
    return np.abs(key(a_bits) - key(b_bits))


# Tolerances of the parity bars (bf16 outputs, fp32 accumulation in an unspecified order):
REL_TOL_VS_ORACLE = 1e-2      # stated bar: bf16-out relative error <= 1e-2
REL_TOL_TIGHT = 4e-3          # what the same arithmetic with a different summation order gives


def bf16_unit_excess(got_bits: np.ndarray, want_bits: np.ndarray, floor: float = 2.0 ** -6):
    """How far two finite bf16 arrays are apart, in units of one bf16 step AT THE VALUE'S MAGNITUDE (the step of
    `floor` for values closer to zero than that: where a result comes out of a cancellation -- 1 + tanh, a*c - b*s,
    v + 4 -- a unit in the last place of the tiny result says nothing).  Returns (largest distance in such units,
    fraction of elements whose bits differ)."""
    def f32(b):
        return (b.astype(np.uint32) << 16).view(np.float32)
    got, want = f32(np.ascontiguousarray(got_bits)), f32(np.ascontiguousarray(want_bits))
    mag = np.maximum(np.maximum(np.abs(want), np.abs(got)), floor)
    unit = 2.0 ** (np.floor(np.log2(mag)) - 7)
    return float((np.abs(got - want) / unit).max()), float((got_bits != want_bits).mean())
