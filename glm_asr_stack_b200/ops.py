"""Host-side mirror of the Infer-engine operator interface for the FP4 linear path.

Same names, argument meaning and error behaviour as the reference's C entry points
(Infer-engine/include/cuda_kernels.h), taking torch CUDA tensors instead of raw pointers.
torch is used only for device memory; every computation happens inside libglmasr_fp4.so.
"""
from __future__ import annotations

import ctypes
import weakref
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import Fp4Weight, LayerWeights

MODE_W4A4 = 0
MODE_W4A16 = 1
EPI_STORE = 0
EPI_SILU_GATE = 1
EPI_RESIDUAL = 2


_tracked = {}


def _forget(ptr: int):
    _tracked.pop(ptr, None)
    try:
        _lib.load().glmasr_fp4_forget(ctypes.c_void_p(ptr))
    except Exception:
        pass


def _track_scales(w_scales: Optional[torch.Tensor]):
    """The library caches the re-tiled copy of a weight's scales by device pointer.  torch may
    hand the same address to a different tensor later, so drop the cache entry when the tensor
    that owned the address goes away (the C host calls glmasr_fp4_forget from safetensors_free)."""
    if w_scales is None:
        return
    ptr = w_scales.data_ptr()
    fin = _tracked.get(ptr)
    if fin is not None and fin.alive:
        return
    _tracked[ptr] = weakref.finalize(w_scales, _forget, ptr)


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("expected a CUDA tensor")
    return ctypes.c_void_p(t.data_ptr())


def _check(t: torch.Tensor, dtype, name: str):
    if t.dtype != dtype:
        raise TypeError(f"{name}: expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: must be contiguous")


@dataclass
class Fp4Tensor:
    """One FP4 weight as the safetensors loader leaves it on the device
    (Infer-engine/src/safetensors.c:48-55): ``weight`` U8 [N, K/2], ``weight_scale`` F8_E4M3
    bytes [N, K/16], scalar ``weight_scale_2``; optional ``input_scale`` / ``pre_quant_scale``."""

    w_packed: torch.Tensor
    w_scales: torch.Tensor
    w_global_scale: float
    input_scale: float = 1.0
    pre_quant_scale: Optional[torch.Tensor] = None

    @property
    def N(self) -> int:
        return self.w_packed.shape[0]

    @property
    def K(self) -> int:
        return self.w_packed.shape[1] * 2

    def c_struct(self) -> Fp4Weight:
        return Fp4Weight(self.w_packed.data_ptr(), self.w_scales.data_ptr(), float(self.w_global_scale), self.N)


def fp4_dequant_to_bf16(packed_w: torch.Tensor, block_scales: Optional[torch.Tensor], global_scale: float,
                        rows: Optional[int] = None, cols: Optional[int] = None) -> torch.Tensor:
    """reference: fp4_dequant_to_bf16, Infer-engine/cuda/kernels.cu:234-246."""
    lib = _lib.load()
    _check(packed_w, torch.uint8, "packed_w")
    rows = packed_w.shape[0] if rows is None else rows
    cols = packed_w.shape[1] * 2 if cols is None else cols
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device=packed_w.device)
    lib.fp4_dequant_to_bf16(_ptr(out), _ptr(packed_w), _ptr(block_scales), float(global_scale), rows, cols)
    return out


def fp4_linear(x: torch.Tensor, w_packed: torch.Tensor, w_scales: Optional[torch.Tensor], w_global_scale: float,
               pre_quant_scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """reference: fp4_linear (W4A16), Infer-engine/cuda/kernels.cu:1297-1318."""
    lib = _lib.load()
    _check(x, torch.bfloat16, "x")
    _check(w_packed, torch.uint8, "w_packed")
    M, K = x.shape
    N = w_packed.shape[0]
    if w_packed.shape[1] * 2 != K:
        raise ValueError("w_packed must be [N, K/2]")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    scratch = torch.empty((M, K), dtype=torch.bfloat16, device=x.device) if pre_quant_scale is not None else None
    lib.fp4_linear(None, _ptr(out), None, _ptr(scratch), _ptr(x), _ptr(w_packed), _ptr(w_scales),
                   float(w_global_scale), _ptr(pre_quant_scale), _ptr(bias), M, N, K)
    return out


def nvfp4_cutlass_available() -> int:
    return _lib.load().nvfp4_cutlass_available()


def nvfp4_linear(out: torch.Tensor, x: torch.Tensor, w_packed: torch.Tensor, w_scales: Optional[torch.Tensor],
                 input_scale: float, w_global_scale: float, pre_quant_scale: Optional[torch.Tensor] = None,
                 bias: Optional[torch.Tensor] = None, M: Optional[int] = None, N: Optional[int] = None,
                 K: Optional[int] = None) -> int:
    """reference: nvfp4_linear (W4A4), Infer-engine/cuda/nvfp4_cutlass.cu:118-270.
    Returns 0 on success, -1 when the reference would (bad sizes, missing scales, K % 16,
    input_scale <= 0); ``out`` is untouched in that case."""
    lib = _lib.load()
    _track_scales(w_scales)
    M = x.shape[0] if M is None else M
    K = x.shape[1] if K is None else K
    N = w_packed.shape[0] if N is None else N
    return lib.nvfp4_linear(None, _ptr(out), None, _ptr(x), _ptr(w_packed), _ptr(w_scales), float(input_scale),
                            float(w_global_scale), _ptr(pre_quant_scale), _ptr(bias), M, N, K)


def nvfp4_linear_noalloc(out: torch.Tensor, x: torch.Tensor, w_packed: torch.Tensor, w_scales: torch.Tensor,
                         input_scale: float, w_global_scale: float) -> int:
    """glmasr_nvfp4_linear_noalloc: the W4A4 linear for callers that must not allocate device
    memory (for instance a decode loop running after the engine has handed all free memory to the
    KV pool).  Temporaries live in a fixed array inside the library; returns -1 for sizes beyond it
    (M > 512, K > 8192, ceil128(N)*K > 32 Mi) or unsupported alignment.  Calls must not overlap
    on the GPU: they share that array."""
    lib = _lib.load()
    M, K = x.shape
    N = w_packed.shape[0]
    return lib.glmasr_nvfp4_linear_noalloc(_ptr(out), _ptr(x), _ptr(w_packed), _ptr(w_scales), float(input_scale),
                                           float(w_global_scale), M, N, K)


def bf16_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """reference: bf16_linear, Infer-engine/cuda/kernels.cu:1147-1193."""
    lib = _lib.load()
    _check(x, torch.bfloat16, "x")
    _check(w, torch.bfloat16, "w")
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    lib.bf16_linear(None, _ptr(out), _ptr(x), _ptr(w), _ptr(bias), M, N, K)
    return out


def silu_mul_split_packed(packed_gate_up: torch.Tensor) -> torch.Tensor:
    """reference: silu_mul_split_packed, Infer-engine/cuda/kernels.cu:1252-1273."""
    lib = _lib.load()
    _check(packed_gate_up, torch.bfloat16, "packed_gate_up")
    M, N2 = packed_gate_up.shape
    out = torch.empty((M, N2 // 2), dtype=torch.bfloat16, device=packed_gate_up.device)
    lib.silu_mul_split_packed(_ptr(out), _ptr(packed_gate_up), M, N2 // 2)
    return out


def silu_elementwise_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """reference: silu_elementwise_mul (in place on gate), Infer-engine/cuda/kernels.cu:405-421."""
    lib = _lib.load()
    _check(gate, torch.bfloat16, "gate")
    _check(up, torch.bfloat16, "up")
    lib.silu_elementwise_mul(_ptr(gate), _ptr(up), gate.numel())
    return gate


def residual_add(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """reference: residual_add, Infer-engine/cuda/kernels.cu:741-761."""
    lib = _lib.load()
    _check(a, torch.bfloat16, "a")
    _check(b, torch.bfloat16, "b")
    out = torch.empty_like(a) if out is None else out
    lib.residual_add(_ptr(out), _ptr(a), _ptr(b), a.numel())
    return out


def lm_head_argmax_batched(hidden: torch.Tensor, lm_weight: torch.Tensor) -> torch.Tensor:
    """reference: lm_head_argmax_batched, Infer-engine/cuda/kernels.cu:1443-1459.  Returns the
    token ids as a HOST int32 tensor (the reference copies them to the host synchronously)."""
    lib = _lib.load()
    _check(hidden, torch.bfloat16, "hidden")
    _check(lm_weight, torch.bfloat16, "lm_weight")
    rows, dim = hidden.shape
    vocab = lm_weight.shape[0]
    tokens = torch.empty(rows, dtype=torch.int32)
    lib.lm_head_argmax_batched(None, _ptr(hidden), _ptr(lm_weight), rows, dim, vocab,
                               ctypes.c_void_p(tokens.data_ptr()))
    return tokens


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, out: Optional[torch.Tensor] = None):
    """reference: rmsnorm, Infer-engine/cuda/kernels.cu:252-295."""
    lib = _lib.load()
    _check(x, torch.bfloat16, "x")
    out = torch.empty_like(x) if out is None else out
    lib.rmsnorm(_ptr(out), _ptr(x), _ptr(weight), float(eps), x.shape[0], x.shape[1])
    return out


def embedding_lookup(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """reference: embedding_lookup, Infer-engine/cuda/kernels.cu:712-736 (ids int32 on the device)."""
    lib = _lib.load()
    out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.bfloat16, device=table.device)
    lib.embedding_lookup(_ptr(out), _ptr(table), _ptr(ids), ids.numel(), table.shape[1])
    return out


def rope_single_token(t: torch.Tensor, positions: torch.Tensor, n_heads: int, head_dim: int) -> torch.Tensor:
    """In place; reference: rope_batched_single_token_kernel, Infer-engine/cuda/decoder.cu:605-632."""
    _lib.load().glmasr_rope_single_token(_ptr(t), _ptr(positions), t.shape[0], n_heads, head_dim)
    return t


def rope_qk_cache(qkv: torch.Tensor, k_col: int, v_col: int, positions: torch.Tensor, slot_mapping: torch.Tensor,
                  k_cache: torch.Tensor, v_cache: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int) -> torch.Tensor:
    """RoPE on q and k of the new-token rows (in place) + K / V rows into the paged cache, one launch
    (Infer-engine/cuda/decoder.cu:605-632 twice and cuda/paged_kv.cu:70-97)."""
    rc = _lib.load().glmasr_rope_qk_cache(_ptr(qkv), qkv.stride(0), k_col, v_col, _ptr(positions), _ptr(slot_mapping),
                                          _ptr(k_cache), _ptr(v_cache), qkv.shape[0], q_heads, kv_heads, head_dim)
    if rc != 0:
        raise ValueError("glmasr_rope_qk_cache rejected the layout")
    return qkv


def rmsnorm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float, input_scale: float):
    """rmsnorm + activation quantiser in one launch.  Returns (packed [rows, dim/2] u8, tiled scales u8)."""
    rows, dim = x.shape
    packed = torch.empty((rows, dim // 2), dtype=torch.uint8, device=x.device)
    tiled = torch.zeros(((rows + 127) // 128) * (dim // 64) * 512, dtype=torch.uint8, device=x.device)
    rc = _lib.load().glmasr_rmsnorm_quant(_ptr(packed), _ptr(tiled), _ptr(x), _ptr(weight), float(eps),
                                          float(input_scale), rows, dim)
    if rc != 0:
        raise ValueError("glmasr_rmsnorm_quant rejected the arguments")
    return packed, tiled


def reshape_and_cache(k_cache, v_cache, key, value, slot_mapping, num_kv_heads, head_dim, block_size):
    """reference: reshape_and_cache, Infer-engine/cuda/paged_kv.cu:70-97, 424-438."""
    _lib.load().reshape_and_cache(_ptr(k_cache), _ptr(v_cache), _ptr(key), _ptr(value), _ptr(slot_mapping),
                                  key.shape[0], num_kv_heads, head_dim, block_size)


def paged_decode_attention(query, k_cache, v_cache, block_tables, seq_lens, num_q_heads, num_kv_heads, head_dim,
                           block_size) -> torch.Tensor:
    """reference: paged_decode_attention, Infer-engine/cuda/paged_kv.cu:440-519."""
    out = torch.empty_like(query)
    _lib.load().paged_decode_attention(_ptr(out), _ptr(query), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                                       _ptr(seq_lens), query.shape[0], num_q_heads, num_kv_heads, head_dim,
                                       block_size, block_tables.shape[1])
    return out


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    lib = _lib.load()
    _check(logits, torch.bfloat16, "logits")
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    rc = lib.glmasr_argmax_rows(_ptr(logits), _ptr(out), rows, vocab)
    if rc != 0:
        raise RuntimeError("glmasr_argmax_rows failed")
    return out


def quantize_bf16_to_fp4(x: torch.Tensor, input_scale: float, pre_quant_scale: Optional[torch.Tensor] = None):
    """reference: quantize_bf16_to_fp4_kernel, Infer-engine/cuda/nvfp4_cutlass.cu:35-87.
    Returns (packed [M, K/2] u8, scales [M, K/16] u8)."""
    lib = _lib.load()
    _check(x, torch.bfloat16, "x")
    M, K = x.shape
    packed = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((M, K // 16), dtype=torch.uint8, device=x.device)
    rc = lib.glmasr_quantize_bf16_to_fp4(_ptr(packed), _ptr(scales), _ptr(x), _ptr(pre_quant_scale),
                                         float(input_scale), M, K)
    if rc != 0:
        raise ValueError("glmasr_quantize_bf16_to_fp4 rejected the arguments")
    return packed, scales


def swizzle_rowwise_scales(scales: torch.Tensor) -> torch.Tensor:
    """reference: swizzle_rowwise_scales_kernel, Infer-engine/cuda/nvfp4_cutlass.cu:89-111."""
    lib = _lib.load()
    _check(scales, torch.uint8, "scales")
    rows, cols = scales.shape
    n = ((rows + 127) // 128 * 128) * ((cols + 3) // 4 * 4)
    dst = torch.empty(n, dtype=torch.uint8, device=scales.device)
    rc = lib.glmasr_swizzle_rowwise_scales(_ptr(dst), _ptr(scales), rows, cols)
    if rc != 0:
        raise ValueError("glmasr_swizzle_rowwise_scales rejected the arguments")
    return dst


def fp4_linear_fused(mode: int, x: torch.Tensor, weights: Sequence[Fp4Tensor], epilogue: int = EPI_STORE,
                     residual: Optional[torch.Tensor] = None, input_scale: float = 1.0,
                     pre_quant_scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                     ldx: Optional[int] = None, M: Optional[int] = None) -> torch.Tensor:
    """Up to three same-input FP4 projections in one GEMM with a fused epilogue
    (glmasr_fp4_linear_fused; replaces linear_proj_pair_same_input + silu_mul_split_packed /
    residual_add, Infer-engine/cuda/decoder.cu:923-978)."""
    lib = _lib.load()
    if x.dtype != torch.bfloat16:
        raise TypeError("x must be bf16")
    K = weights[0].K
    M = x.shape[0] if M is None else M
    ldx = x.stride(0) if ldx is None else ldx
    n_out = weights[0].N if epilogue == EPI_SILU_GATE else sum(w.N for w in weights)
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    for w in weights:
        _track_scales(w.w_scales)
    arr = (Fp4Weight * len(weights))(*[w.c_struct() for w in weights])
    scratch = torch.empty((M, K), dtype=torch.bfloat16, device=x.device) if (
        pre_quant_scale is not None and mode == MODE_W4A16) else None
    rc = lib.glmasr_fp4_linear_fused(mode, _ptr(out), out.stride(0), _ptr(x), ldx, arr, len(weights),
                                     float(input_scale), _ptr(pre_quant_scale), _ptr(scratch), epilogue,
                                     _ptr(residual), M, K)
    if rc != 0:
        raise ValueError("glmasr_fp4_linear_fused rejected the arguments")
    return out


def fp4_linear_quantized(xq: torch.Tensor, xq_sf: torch.Tensor, weights: Sequence[Fp4Tensor], input_scale: float,
                         epilogue: int = EPI_STORE, out: Optional[torch.Tensor] = None, resident: bool = False,
                         q_out_input_scale: float = 0.0, M: Optional[int] = None):
    """W4A4 linear on an activation that is already quantised (glmasr_fp4_linear_quantized): xq e2m1 bytes
    [M, K/2] and its 128x4-tiled scales as rmsnorm_quant returns them.  EPI_RESIDUAL adds into `out` in place.
    EPI_SILU_GATE with q_out_input_scale > 0 returns (packed [M, N/2] u8, tiled scales u8) for a following W4A4
    GEMM instead of a bf16 tensor.  resident=True runs it as one phase of the co-resident layer-tail kernel."""
    lib = _lib.load()
    K = weights[0].K
    M = xq.shape[0] if M is None else M
    for w in weights:
        _track_scales(w.w_scales)
    arr = (Fp4Weight * len(weights))(*[w.c_struct() for w in weights])
    n_out = weights[0].N if epilogue == EPI_SILU_GATE else sum(w.N for w in weights)
    q_out = q_sf = None
    if epilogue == EPI_SILU_GATE and q_out_input_scale > 0.0:
        q_out = torch.empty((M, n_out // 2), dtype=torch.uint8, device=xq.device)
        q_sf = torch.zeros(((M + 127) // 128) * (n_out // 64) * 512, dtype=torch.uint8, device=xq.device)
    if out is None and not (q_out is not None and resident):
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=xq.device)
    rc = lib.glmasr_fp4_linear_quantized(1 if resident else 0, _ptr(out), out.stride(0) if out is not None else n_out,
                                         _ptr(xq), _ptr(xq_sf), arr, len(weights), float(input_scale), epilogue,
                                         _ptr(out) if epilogue == EPI_RESIDUAL else None, M, K, _ptr(q_out), _ptr(q_sf),
                                         float(q_out_input_scale))
    if rc != 0:
        raise ValueError("glmasr_fp4_linear_quantized rejected the arguments")
    return (q_out, q_sf) if q_out is not None else out


def decode_layer_tail(hidden: torch.Tensor, attn_q: torch.Tensor, attn_sf: torch.Tensor, lw: "LayerWeights",
                      post_attention_norm: torch.Tensor, next_lw: Optional["LayerWeights"] = None,
                      next_input_norm: Optional[torch.Tensor] = None, max_phases: int = 0):
    """o + residual | norm + quantiser | gate|up + SiLU-gate + quantiser | down + residual [| norm + quantiser |
    q|k|v of the next layer] as one co-resident launch (glmasr_decode_layer_tail), in place on `hidden`.
    Returns (next_qkv or None, norm_q, norm_sf, act_q, act_sf)."""
    M, H = hidden.shape
    F = lw.ffn
    dev = hidden.device
    norm_q = torch.zeros((M, H // 2), dtype=torch.uint8, device=dev)
    norm_sf = torch.zeros(((M + 127) // 128) * (H // 64) * 512, dtype=torch.uint8, device=dev)
    act_q = torch.zeros((M, F // 2), dtype=torch.uint8, device=dev)
    act_sf = torch.zeros(((M + 127) // 128) * (F // 64) * 512, dtype=torch.uint8, device=dev)
    qkv = None
    if next_lw is not None:
        qkv = torch.zeros((M, next_lw.q.N + next_lw.k.N + next_lw.v.N), dtype=torch.bfloat16, device=dev)
    rc = _lib.load().glmasr_decode_layer_tail(_ptr(hidden), M, _ptr(attn_q), _ptr(attn_sf), ctypes.byref(lw),
                                              _ptr(post_attention_norm), ctypes.byref(next_lw) if next_lw is not None else None,
                                              _ptr(next_input_norm), _ptr(qkv), _ptr(norm_q), _ptr(norm_sf), _ptr(act_q),
                                              _ptr(act_sf), int(max_phases))
    if rc != 0:
        raise ValueError("glmasr_decode_layer_tail rejected the arguments")
    return qkv, norm_q, norm_sf, act_q, act_sf


def make_layer_weights(q, k, v, o, gate, up, down, hidden: int, ffn: int) -> LayerWeights:
    for w in (q, k, v, o, gate, up, down):
        _track_scales(w.w_scales)
    return LayerWeights(q.c_struct(), k.c_struct(), v.c_struct(), o.c_struct(), gate.c_struct(), up.c_struct(),
                        down.c_struct(), float(q.input_scale), float(o.input_scale), float(gate.input_scale),
                        float(down.input_scale), hidden, ffn)


def layer_proj(mode: int, hidden_in: torch.Tensor, lw: LayerWeights, out: Optional[torch.Tensor] = None):
    """The four fused FP4 projections of one decoder layer on device tensors (glmasr_fp4_layer_proj)."""
    lib = _lib.load()
    out = torch.empty_like(hidden_in) if out is None else out
    rc = lib.glmasr_fp4_layer_proj(mode, _ptr(out), _ptr(hidden_in), ctypes.byref(lw), hidden_in.shape[0])
    if rc != 0:
        raise RuntimeError("glmasr_fp4_layer_proj failed")
    return out


def layer_proj_host(mode: int, hidden_in_host: torch.Tensor, hidden_out_host: torch.Tensor, lw: LayerWeights):
    """Same through HOST (pinned) buffers: copy in, run, copy out, synchronise."""
    lib = _lib.load()
    rc = lib.glmasr_fp4_layer_proj_host(mode, ctypes.c_void_p(hidden_out_host.data_ptr()),
                                        ctypes.c_void_p(hidden_in_host.data_ptr()), ctypes.byref(lw),
                                        hidden_in_host.shape[0])
    if rc != 0:
        raise RuntimeError("glmasr_fp4_layer_proj_host failed")
    return hidden_out_host


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, eps: float = 1e-5,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """reference: layernorm, Infer-engine/cuda/kernels.cu:299-356."""
    lib = _lib.load()
    _check(x, torch.bfloat16, "x")
    rows, dim = x.shape
    if out is None:
        out = torch.empty_like(x)
    lib.layernorm(_ptr(out), _ptr(x), _ptr(weight), _ptr(bias), float(eps), rows, dim)
    return out


def gelu_inplace(x: torch.Tensor) -> torch.Tensor:
    """reference: gelu_inplace, Infer-engine/cuda/kernels.cu:364-381."""
    _check(x, torch.bfloat16, "x")
    _lib.load().gelu_inplace(_ptr(x), x.numel())
    return x


def rope_encoder(q: torch.Tensor, k: torch.Tensor, num_heads: int, head_dim: int, partial_factor: float = 0.5):
    """reference: rope_encoder, Infer-engine/cuda/kernels.cu:427-484; q, k [seq_len, num_heads * head_dim] in place."""
    _lib.load().rope_encoder(_ptr(q), _ptr(k), q.shape[0], num_heads, head_dim, float(partial_factor))
    return q, k


def residual_add_bias(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """reference: residual_add_bias, Infer-engine/cuda/kernels.cu:763-795."""
    out = torch.empty_like(a)
    _lib.load().residual_add_bias(_ptr(out), _ptr(a), _ptr(b), _ptr(bias), a.shape[0], a.shape[1])
    return out


def conv1d_forward(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], stride: int, padding: int) -> torch.Tensor:
    """reference: conv1d_forward, Infer-engine/cuda/kernels.cu:1561-1629; x [in_ch, len], weight [out_ch, in_ch, k]."""
    in_ch, ln = x.shape
    out_ch, _, ks = weight.shape
    out_len = (ln + 2 * padding - ks) // stride + 1
    out = torch.empty((out_ch, out_len), dtype=torch.bfloat16, device=x.device)
    _lib.load().conv1d_forward(_ptr(out), _ptr(x), _ptr(weight), _ptr(bias), in_ch, out_ch, ln, ks, stride, padding)
    return out


def transpose_2d(x: torch.Tensor) -> torch.Tensor:
    out = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=x.device)
    _lib.load().transpose_2d(_ptr(out), _ptr(x), x.shape[0], x.shape[1])
    return out


def bf16_linear_gelu(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """reference: bf16_linear_gelu, Infer-engine/cuda/kernels.cu:1211-1250."""
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _lib.load().bf16_linear_gelu(None, _ptr(out), _ptr(x), _ptr(w), _ptr(bias), M, N, K)
    return out


def encoder_forward_packed(ws, cfg, hidden: torch.Tensor, seq_lens: Sequence[int], seq_offsets: Sequence[int]) -> torch.Tensor:
    """reference: encoder_forward_packed, Infer-engine/cuda/encoder.cu:2441-2462; in place on hidden [rows, enc_hidden].
    ws: an object whose ``.c`` is the C WeightStore, cfg: the C ModelConfig."""
    n = len(seq_lens)
    lens = (ctypes.c_int * n)(*[int(v) for v in seq_lens])
    offs = (ctypes.c_int * n)(*[int(v) for v in seq_offsets])
    _lib.load().encoder_forward_packed(None, ctypes.byref(ws.c), _ptr(hidden), hidden.shape[0], n, lens, offs, ctypes.byref(cfg))
    return hidden


def audio_encode_batched(ws, cfg, mel_time_major: torch.Tensor, n_frames: Sequence[int], out: Optional[torch.Tensor] = None):
    """glmasr_audio_encode_batched: mel_time_major bf16 [windows, stride] (window i holds [n_i, num_mel_bins]) ->
    (bf16 [windows, max_tokens, dec_hidden], tokens per window)."""
    w = mel_time_major.shape[0]
    max_tokens = max(((int(n) + 1) // 2) // 4 for n in n_frames)
    if out is None:
        out = torch.zeros((w, max_tokens, cfg.dec_hidden), dtype=torch.bfloat16, device=mel_time_major.device)
    nf = (ctypes.c_int * w)(*[int(v) for v in n_frames])
    tok = (ctypes.c_int * w)()
    rc = _lib.load().glmasr_audio_encode_batched(ctypes.byref(ws.c), ctypes.byref(cfg), _ptr(mel_time_major),
                                                 mel_time_major.stride(0), nf, w, _ptr(out), out.stride(0), tok)
    if rc != 0:
        raise ValueError("glmasr_audio_encode_batched rejected the arguments")
    return out, list(tok)


def mel_spectrogram(pcm: torch.Tensor, mel_filters_t: torch.Tensor) -> torch.Tensor:
    """reference: mel_spectrogram, Infer-engine/cuda/mel.cu:253-294.  pcm float32 [num_samples] and the
    transposed filterbank float32 [201, 128] on the device -> bf16 [128, n_frames]."""
    lib = _lib.load()
    _check(pcm, torch.float32, "pcm")
    _check(mel_filters_t, torch.float32, "mel_filters_t")
    ns = pcm.numel()
    n = min(max((ns + 159) // 160, 1), 3000)
    out = torch.empty((128, n), dtype=torch.bfloat16, device=pcm.device)
    frames = ctypes.c_int(0)
    lib.mel_spectrogram(_ptr(pcm), ns, _ptr(mel_filters_t), _ptr(out), ctypes.byref(frames))
    assert frames.value == n
    return out


def mel_spectrogram_batched(pcm: torch.Tensor, num_samples: Sequence[int], mel_filters_t: torch.Tensor,
                            time_major: bool = False, out: Optional[torch.Tensor] = None):
    """glmasr_mel_spectrogram_batched: pcm float32 [windows, stride]; returns (bf16 [windows, 128 * 3000] buffer whose
    window i holds [128, n_i] or [n_i, 128] at its start, list of n_i)."""
    lib = _lib.load()
    _check(pcm, torch.float32, "pcm")
    w = pcm.shape[0]
    if out is None:
        out = torch.zeros((w, 128 * 3000), dtype=torch.bfloat16, device=pcm.device)
    ns = (ctypes.c_int * w)(*[int(v) for v in num_samples])
    frames = (ctypes.c_int * w)()
    rc = lib.glmasr_mel_spectrogram_batched(_ptr(pcm), pcm.stride(0), ns, w, _ptr(mel_filters_t), _ptr(out), out.stride(0),
                                            1 if time_major else 0, frames)
    if rc != 0:
        raise ValueError("glmasr_mel_spectrogram_batched rejected the arguments")
    return out, list(frames)


def status() -> int:
    """Synchronise; return and clear the first device-side status code (0 = ok)."""
    return _lib.load().glmasr_fp4_status()


def launch_count() -> int:
    return int(_lib.load().glmasr_launch_count())


def profile_enable(on: bool):
    _lib.load().glmasr_profile_enable(1 if on else 0)


def profile_read(max_entries: int = 4096):
    """[(ms, flops, bytes)] of the GEMM launches recorded since the last read."""
    arr = (ctypes.c_double * max_entries)
    ms, fl, by = arr(), arr(), arr()
    n = _lib.load().glmasr_profile_read(max_entries, ms, fl, by)
    if n < 0:
        raise RuntimeError("glmasr_profile_read failed")
    return [(ms[i], fl[i], by[i]) for i in range(n)]


def set_stream(stream: Optional[torch.cuda.Stream]):
    _lib.load().glmasr_set_stream(ctypes.c_void_p(stream.cuda_stream) if stream is not None else None)


def prepack(w: Fp4Tensor) -> int:
    _track_scales(w.w_scales)
    return _lib.load().glmasr_fp4_prepack(_ptr(w.w_scales), w.N, w.K)


def cleanup():
    _lib.load().glmasr_fp4_cleanup()
