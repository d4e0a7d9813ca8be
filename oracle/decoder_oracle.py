"""CPU oracle for the decode step's glue and for the whole batched decode step (numpy).

TEST INFRASTRUCTURE ONLY (see fp4_oracle.py).  Restates, with reference file:line citations:
RMSNorm, rotate-half RoPE for one new token, the paged-KV write, paged GQA decode attention and
the layer sequence of decoder_decode_step_batched.  Pinned on a GPU against the reference's own
kernels (oracle/_ref) by tests/test_gpu_decoder.py.
"""
from __future__ import annotations

import numpy as np

import fp4_oracle as o

F32 = np.float32


def rmsnorm(x_bits: np.ndarray, w_bits: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:252-295 in the reference's own summation order: lane l of
    a warp adds x[l]^2, x[l+32]^2, ... sequentially in fp32, then a shfl_down tree (16,8,4,2,1);
    rms = sqrtf(sum/dim + eps); out = bf16((x / rms) * w)."""
    x = o.bf16_bits_to_f32(x_bits)
    w = o.bf16_bits_to_f32(w_bits)
    rows, dim = x.shape
    assert dim % 32 == 0
    sq = (x * x).astype(F32).reshape(rows, dim // 32, 32)
    lane = np.zeros((rows, 32), F32)
    for j in range(dim // 32):                      # sequential per lane, fp32
        lane = (lane + sq[:, j, :]).astype(F32)
    off = 16
    while off > 0:                                  # lane i += lane i+off (only lane 0 matters)
        lane[:, :off] = (lane[:, :off] + lane[:, off:2 * off]).astype(F32)
        off //= 2
    rms = np.sqrt((lane[:, 0] / F32(dim) + F32(eps)).astype(F32)).astype(F32)
    return o.f32_to_bf16_bits(((x / rms[:, None]).astype(F32) * w[None, :]).astype(F32))


def rope_single_token(t_bits: np.ndarray, positions: np.ndarray, n_heads: int, head_dim: int) -> np.ndarray:
    """Infer-engine/cuda/decoder.cu:605-632 (rotate-half, theta 10000, position per sequence).
    cos/sin/pow come from numpy's float32 routines, which can differ from CUDA's by an ulp, so
    comparisons with the GPU use a one-bf16-ulp tolerance."""
    t = o.bf16_bits_to_f32(t_bits).reshape(-1, n_heads, head_dim).copy()
    half = head_dim // 2
    d = np.arange(half, dtype=F32)
    inv_freq = (F32(1.0) / np.power(F32(10000.0), (F32(2.0) * d) / F32(head_dim)).astype(F32)).astype(F32)
    theta = (positions.astype(F32)[:, None] * inv_freq[None, :]).astype(F32)
    c, s = np.cos(theta).astype(F32)[:, None, :], np.sin(theta).astype(F32)[:, None, :]
    v0, v1 = t[:, :, :half].copy(), t[:, :, half:].copy()
    t[:, :, :half] = (v0 * c - v1 * s).astype(F32)
    t[:, :, half:] = (v0 * s + v1 * c).astype(F32)
    return o.f32_to_bf16_bits(t.reshape(t_bits.shape))


def reshape_and_cache(k_cache, v_cache, key_bits, value_bits, slot_mapping):
    """Infer-engine/cuda/paged_kv.cu:70-97; caches are [num_slots, kv_heads*head_dim] views."""
    k_cache[slot_mapping] = key_bits
    v_cache[slot_mapping] = value_bits


def paged_decode_attention(q_bits, k_cache, v_cache, block_tables, seq_lens, n_q_heads, n_kv_heads, head_dim,
                           block_size) -> np.ndarray:
    """Infer-engine/cuda/paged_kv.cu:321-422 / 440-519 in float64 (the reference's fp32 online
    softmax differs by rounding only): softmax(q.K/sqrt(d)) V over seq_lens tokens, negative
    block ids masked, out = acc / (sum + 1e-9), zeros for seq_len <= 0.
    k_cache / v_cache: bf16 bits [num_slots, kv_heads*head_dim]."""
    n = q_bits.shape[0]
    q = o.bf16_bits_to_f32(q_bits).astype(np.float64).reshape(n, n_q_heads, head_dim)
    out = np.zeros((n, n_q_heads, head_dim), np.float64)
    group = n_q_heads // n_kv_heads
    scale = 1.0 / np.sqrt(float(head_dim))
    for s in range(n):
        L = int(seq_lens[s])
        if L <= 0:
            continue
        t = np.arange(L)
        blk = block_tables[s, t // block_size]
        ok = blk >= 0
        slots = blk[ok].astype(np.int64) * block_size + (t[ok] % block_size)
        if slots.size == 0:
            continue
        K = o.bf16_bits_to_f32(k_cache[slots]).astype(np.float64).reshape(-1, n_kv_heads, head_dim)
        V = o.bf16_bits_to_f32(v_cache[slots]).astype(np.float64).reshape(-1, n_kv_heads, head_dim)
        for h in range(n_q_heads):
            kv = h // group
            sc = (K[:, kv, :] @ q[s, h]) * scale
            p = np.exp(sc - sc.max())
            out[s, h] = (p @ V[:, kv, :]) / (p.sum() + 1e-9)
    return o.f32_to_bf16_bits(out.reshape(n, n_q_heads * head_dim).astype(F32))


PROJECTIONS = ("q", "k", "v", "o", "gate", "up", "down")


def projection_mix(w4a16, w4a4, mode):
    """The arithmetic of each of the seven projections as a dict name -> linear(x_bits, w).

    ``mode``: "w4a16"     every projection through fp4_linear (the reference without GLMASR_USE_CUTLASS_NVFP4);
              "reference" the reference WITH the switch: q, o, down through nvfp4_linear (linear_proj,
                          Infer-engine/cuda/decoder.cu:861-921, called with use_native_nvfp4 = true), k|v and
                          gate|up through the fused pair, which always dequantises and runs a bf16 GEMM
                          (linear_proj_pair_same_input, decoder.cu:923-978; call sites :2017, :2107);
              "all_w4a4"  every projection through nvfp4_linear (what the reference does for pairs that carry a
                          pre_quant_scale, and what this library does for all pairs with GLMASR_NVFP4_PAIRS=1)."""
    if mode == "w4a16":
        return {n: w4a16 for n in PROJECTIONS}
    if mode == "all_w4a4":
        return {n: w4a4 for n in PROJECTIONS}
    assert mode == "reference", mode
    return {n: (w4a4 if n in ("q", "o", "down") else w4a16) for n in PROJECTIONS}


def _per_projection(linear):
    return linear if isinstance(linear, dict) else {n: linear for n in PROJECTIONS}


def decode_step(hidden_bits, layers, final_norm_bits, k_caches, v_caches, block_tables, cached_lens, slot_mapping,
                n_q_heads, n_kv_heads, head_dim, block_size, linear):
    """Infer-engine/cuda/decoder.cu:1972-2139: the layer sequence of one batched decode step.
    `layers[l]` holds norm1, norm2 (bf16 bits) and q,k,v,o,gate,up,down weights; `linear(x_bits, w)`
    is the projection oracle to use (fp4_oracle.linear_o1 or nvfp4_linear bound to its scales), or a dict
    with one such function per projection name (see projection_mix).
    Caches are updated in place.  Returns the final-normed hidden state (bf16 bits)."""
    lin = _per_projection(linear)
    h = hidden_bits.copy()
    H = h.shape[1]
    kvw = n_kv_heads * head_dim
    total = (cached_lens + 1).astype(np.int32)
    for l, Lw in enumerate(layers):
        x = rmsnorm(h, Lw["norm1"])
        q = rope_single_token(lin["q"](x, Lw["q"]), cached_lens, n_q_heads, head_dim)
        k = rope_single_token(lin["k"](x, Lw["k"]), cached_lens, n_kv_heads, head_dim)
        v = lin["v"](x, Lw["v"])
        reshape_and_cache(k_caches[l], v_caches[l], k, v, slot_mapping)
        a = paged_decode_attention(q, k_caches[l], v_caches[l], block_tables, total, n_q_heads, n_kv_heads, head_dim,
                                   block_size)
        h = o.residual_add(lin["o"](a, Lw["o"]), h)
        x = rmsnorm(h, Lw["norm2"])
        act = o.silu_mul_split_packed(np.concatenate([lin["gate"](x, Lw["gate"]), lin["up"](x, Lw["up"])], axis=1))
        h = o.residual_add(lin["down"](act, Lw["down"]), h)
        assert h.shape[1] == H and k.shape[1] == kvw
    return rmsnorm(h, final_norm_bits)


def prefill_attention(q_bits, k_bits, v_bits, seq_offsets, seq_lens, n_q_heads, n_kv_heads, head_dim, causal=True):
    """Per-sequence softmax(Q K^T / sqrt(d) [+ causal mask]) V with q head h reading kv head h // group, float64
    (the attention step of Infer-engine/cuda/decoder.cu:1401-1441; gqa_attention's arithmetic)."""
    q = o.bf16_bits_to_f32(q_bits).astype(np.float64)
    k = o.bf16_bits_to_f32(k_bits).astype(np.float64)
    v = o.bf16_bits_to_f32(v_bits).astype(np.float64)
    T = q.shape[0]
    out = np.zeros((T, n_q_heads * head_dim), np.float64)
    group = n_q_heads // n_kv_heads
    scale = 1.0 / np.sqrt(float(head_dim))
    for off, ln in zip(seq_offsets, seq_lens):
        if ln <= 0:
            continue
        rows = slice(off, off + ln)
        for h in range(n_q_heads):
            kv = h // group
            Q = q[rows, h * head_dim:(h + 1) * head_dim]
            K = k[rows, kv * head_dim:(kv + 1) * head_dim]
            V = v[rows, kv * head_dim:(kv + 1) * head_dim]
            s = (Q @ K.T) * scale
            if causal:
                s = np.where(np.tril(np.ones((ln, ln), bool)), s, -np.inf)
            p = np.exp(s - s.max(axis=1, keepdims=True))
            out[rows, h * head_dim:(h + 1) * head_dim] = (p @ V) / p.sum(axis=1, keepdims=True)
    return o.f32_to_bf16_bits(out.astype(F32))


def prefill(hidden_bits, layers, final_norm_bits, k_caches, v_caches, seq_offsets, seq_lens, slot_mapping,
            n_q_heads, n_kv_heads, head_dim, linear):
    """Infer-engine/cuda/decoder.cu:1219-1557: the layer sequence of a batched variable-length prefill.
    Positions start at 0 in every sequence; caches are updated in place (slot_mapping per token row).
    Returns the final-normed hidden states (bf16 bits)."""
    lin = _per_projection(linear)
    h = hidden_bits.copy()
    pos = np.zeros(h.shape[0], np.int32)
    for off, ln in zip(seq_offsets, seq_lens):
        pos[off:off + ln] = np.arange(ln)
    for l, Lw in enumerate(layers):
        x = rmsnorm(h, Lw["norm1"])
        q = rope_single_token(lin["q"](x, Lw["q"]), pos, n_q_heads, head_dim)
        k = rope_single_token(lin["k"](x, Lw["k"]), pos, n_kv_heads, head_dim)
        v = lin["v"](x, Lw["v"])
        reshape_and_cache(k_caches[l], v_caches[l], k, v, slot_mapping)
        a = prefill_attention(q, k, v, seq_offsets, seq_lens, n_q_heads, n_kv_heads, head_dim)
        h = o.residual_add(lin["o"](a, Lw["o"]), h)
        x = rmsnorm(h, Lw["norm2"])
        act = o.silu_mul_split_packed(np.concatenate([lin["gate"](x, Lw["gate"]), lin["up"](x, Lw["up"])], axis=1))
        h = o.residual_add(lin["down"](act, Lw["down"]), h)
    return rmsnorm(h, final_norm_bits)
