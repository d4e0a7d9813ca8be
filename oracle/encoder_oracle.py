"""CPU restatement of the audio encoder, its convolution front end and the projector (numpy).
TEST INFRASTRUCTURE ONLY.  Every function cites the reference code it follows; GEMMs accumulate in float64
(cuBLAS promises fp32 accumulation in an unspecified order), everything else is float32 in the reference's
order of operations with its bf16 roundings.  Pinned on a GPU against the reference's own kernels
(oracle/_ref: layernorm, gelu_inplace, conv1d_forward, encoder_forward_packed) by tests/test_gpu_encoder.py.
"""
from __future__ import annotations

import numpy as np

import fp4_oracle as o

F32 = np.float32


def _mm(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    return (x.astype(np.float64) @ w.astype(np.float64).T).astype(F32)


def layernorm(x_bits, w_bits, b_bits=None, eps=1e-5) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:299-345: one warp per row; lane l adds x[l], x[l+32], ... sequentially in fp32,
    shuffle-down tree (16, 8, 4, 2, 1), lane 0's total; mean = sum / dim; the same for (x - mean)^2; inv_std =
    1 / sqrtf(var + eps); out = bf16((x - mean) * inv_std * w + b) with the last multiply-add fused (nvcc's default
    contraction), which a float64 multiply-add rounded once to float32 reproduces."""
    x = o.bf16_bits_to_f32(x_bits)
    rows, dim = x.shape

    def warp_sum(v):                                   # v: [rows, dim] float32
        pad = (-dim) % 32
        vp = np.pad(v, ((0, 0), (0, pad))).reshape(rows, -1, 32)
        lane = np.zeros((rows, 32), F32)
        for j in range(vp.shape[1]):                   # sequential per lane (padding adds exact zeros)
            lane = (lane + vp[:, j, :]).astype(F32)
        off = 16
        while off > 0:
            lane[:, :off] = (lane[:, :off] + lane[:, off:2 * off]).astype(F32)
            off //= 2
        return lane[:, 0]

    mean = (warp_sum(x) / F32(dim)).astype(F32)
    d = (x - mean[:, None]).astype(F32)
    var = (warp_sum((d * d).astype(F32)) / F32(dim)).astype(F32)
    inv_std = (F32(1.0) / np.sqrt((var + F32(eps)).astype(F32)).astype(F32)).astype(F32)
    val = (d * inv_std[:, None]).astype(F32)
    w = o.bf16_bits_to_f32(w_bits)
    b = o.bf16_bits_to_f32(b_bits) if b_bits is not None else np.zeros(dim, F32)
    out = (val.astype(np.float64) * w[None, :].astype(np.float64) + b[None, :].astype(np.float64)).astype(F32)
    return o.f32_to_bf16_bits(out)


def gelu_f32(v: np.ndarray) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:364-372: 0.5 v (1 + tanh(0.79788456 (v + 0.044715 v^3))) in float32."""
    v = v.astype(F32)
    arg = (F32(0.79788456) * (v + (F32(0.044715) * v * v * v).astype(F32)).astype(F32)).astype(F32)
    return (F32(0.5) * v * (F32(1.0) + np.tanh(arg).astype(F32))).astype(F32)


def gelu_inplace(x_bits) -> np.ndarray:
    return o.f32_to_bf16_bits(gelu_f32(o.bf16_bits_to_f32(x_bits)))


def bf16_linear(x_bits, w_bits, bias_bits=None) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:1147-1193 with its default cuBLASLt bias epilogue: bf16(acc + bias)."""
    acc = _mm(o.bf16_bits_to_f32(x_bits), o.bf16_bits_to_f32(w_bits))
    if bias_bits is not None:
        acc = (acc + o.bf16_bits_to_f32(bias_bits)[None, :]).astype(F32)
    return o.f32_to_bf16_bits(acc)


def bf16_linear_gelu(x_bits, w_bits, bias_bits=None) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:1211-1250 with the fused epilogue: bf16(gelu(acc + bias))."""
    acc = _mm(o.bf16_bits_to_f32(x_bits), o.bf16_bits_to_f32(w_bits))
    if bias_bits is not None:
        acc = (acc + o.bf16_bits_to_f32(bias_bits)[None, :]).astype(F32)
    return o.f32_to_bf16_bits(gelu_f32(acc))


def residual_add_bias(a_bits, b_bits, bias_bits=None) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:763-782: bf16(bf16(a + bias[col]) + b)."""
    av = o.bf16_bits_to_f32(a_bits)
    if bias_bits is not None:
        av = (av + o.bf16_bits_to_f32(bias_bits)[None, :]).astype(F32)
    av = o.round_bf16(av)
    return o.f32_to_bf16_bits((av + o.bf16_bits_to_f32(b_bits)).astype(F32))


def rope_tables(max_pos: int):
    """Infer-engine/cuda/encoder.cu:1572-1597: cos / sin of pos * powf(10000, -(2 d) / 32), d < 16, all in float32
    on the host.  numpy's float32 powf / cosf / sinf may differ from the C library's in the last place."""
    d = np.arange(16, dtype=F32)
    inv_freq = np.power(F32(10000.0), (-(F32(2.0) * d) / F32(32.0)).astype(F32)).astype(F32)
    theta = (np.arange(max_pos, dtype=F32)[:, None] * inv_freq[None, :]).astype(F32)
    return np.cos(theta).astype(F32), np.sin(theta).astype(F32)


def rope(t_bits, positions, num_heads, head_dim) -> np.ndarray:
    """Infer-engine/cuda/encoder.cu:1604-1642: dims (d, d + 16), d < 16, of every head rotated by the table's angle;
    dims 32 .. head_dim - 1 unchanged.  t_bits: [rows, num_heads * head_dim]."""
    cos_t, sin_t = rope_tables(int(positions.max()) + 1)
    t = o.bf16_bits_to_f32(t_bits).reshape(-1, num_heads, head_dim).copy()
    c, s = cos_t[positions][:, None, :], sin_t[positions][:, None, :]
    a, b = t[:, :, :16].copy(), t[:, :, 16:32].copy()
    t[:, :, :16] = (a * c - b * s).astype(F32)
    t[:, :, 16:32] = (b * c + a * s).astype(F32)
    return o.f32_to_bf16_bits(t.reshape(t_bits.shape))


def attention(q_bits, k_bits, v_bits, seq_offsets, seq_lens, num_heads, head_dim) -> np.ndarray:
    """Non-causal softmax(Q K^T / sqrt(d)) V per sequence and head (Infer-engine/cuda/encoder.cu:1870-1970), float64."""
    q = o.bf16_bits_to_f32(q_bits).astype(np.float64)
    k = o.bf16_bits_to_f32(k_bits).astype(np.float64)
    v = o.bf16_bits_to_f32(v_bits).astype(np.float64)
    out = np.zeros_like(q)
    scale = 1.0 / np.sqrt(float(head_dim))
    for off, ln in zip(seq_offsets, seq_lens):
        if ln <= 0:
            continue
        r = slice(off, off + ln)
        for h in range(num_heads):
            c = slice(h * head_dim, (h + 1) * head_dim)
            s = (q[r, c] @ k[r, c].T) * scale
            p = np.exp(s - s.max(axis=1, keepdims=True))
            out[r, c] = (p @ v[r, c]) / p.sum(axis=1, keepdims=True)
    return o.f32_to_bf16_bits(out.astype(F32))


def encoder_forward_packed(hidden_bits, layers, norm_w, norm_b, seq_offsets, seq_lens, num_heads, head_dim) -> np.ndarray:
    """Infer-engine/cuda/encoder.cu:1974-2188.  layers[l]: dict of bf16 bit arrays ln1_w/b, q_w/b, k_w, v_w/b, o_w/b,
    ln2_w/b, fc1_w/b, fc2_w/b.  Rows outside every sequence are carried along like the reference does (they go
    through the row-wise operations and see no attention)."""
    h = hidden_bits.copy()
    pos = np.zeros(h.shape[0], np.int64)
    for off, ln in zip(seq_offsets, seq_lens):
        pos[off:off + ln] = np.arange(ln)
    for L in layers:
        x = layernorm(h, L["ln1_w"], L.get("ln1_b"))
        q = rope(bf16_linear(x, L["q_w"], L.get("q_b")), pos, num_heads, head_dim)
        k = rope(bf16_linear(x, L["k_w"]), pos, num_heads, head_dim)
        v = bf16_linear(x, L["v_w"], L.get("v_b"))
        a = attention(q, k, v, seq_offsets, seq_lens, num_heads, head_dim)
        h = residual_add_bias(bf16_linear(a, L["o_w"]), h, L.get("o_b"))
        x = layernorm(h, L["ln2_w"], L.get("ln2_b"))
        f = bf16_linear_gelu(x, L["fc1_w"], L.get("fc1_b"))
        h = residual_add_bias(bf16_linear(f, L["fc2_w"]), h, L.get("fc2_b"))
    return layernorm(h, norm_w, norm_b)


def conv1d_forward(in_bits, w_bits, bias_bits, stride, padding) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:1561-1629: input [in_ch, len], weight [out_ch, in_ch, k], out [out_ch, out_len].  One
    GEMM per tap accumulating into the bf16 output (the partial sums are rounded to bf16 after every tap), then the
    bias added to the bf16 result and rounded again."""
    x = o.bf16_bits_to_f32(in_bits)
    w = o.bf16_bits_to_f32(w_bits)
    in_ch, ln = x.shape
    out_ch, _, ks = w.shape
    out_len = (ln + 2 * padding - ks) // stride + 1
    out = np.zeros((out_ch, out_len), F32)
    t = np.arange(out_len) * stride - padding
    for k in range(ks):
        src = t + k
        ok = (src >= 0) & (src < ln)
        shifted = np.where(ok[None, :], x[:, np.clip(src, 0, ln - 1)], F32(0))          # [in_ch, out_len]
        part = (w[:, :, k].astype(np.float64) @ shifted.astype(np.float64)).astype(F32)
        out = o.round_bf16((part + out).astype(F32)) if k else o.round_bf16(part)
    if bias_bits is not None:
        out = o.round_bf16((out + o.bf16_bits_to_f32(bias_bits)[:, None]).astype(F32))
    return o.f32_to_bf16_bits(out)


def audio_encode(mel_bits, conv1, conv2, layers, norm_w, norm_b, proj1, proj2, num_heads, head_dim) -> np.ndarray:
    """Infer-engine/src/engine.c:1111-1160 for one window: mel [mels, frames] -> conv1 -> GELU -> conv2 -> GELU ->
    transpose -> encoder -> groups of four frames -> linear + GELU -> linear.  conv*/proj*: (weight bits, bias bits).
    Returns [frames' / 4, dec_hidden] bf16 bits."""
    c1 = gelu_inplace(conv1d_forward(mel_bits, conv1[0], conv1[1], 1, 1))
    c2 = gelu_inplace(conv1d_forward(c1, conv2[0], conv2[1], 2, 1))
    h = np.ascontiguousarray(c2.T)                                   # [enc_seq_len, hidden]
    n = h.shape[0]
    h = encoder_forward_packed(h, layers, norm_w, norm_b, [0], [n], num_heads, head_dim)
    g = n // 4
    cat = h[:g * 4].reshape(g, -1)
    return bf16_linear(bf16_linear_gelu(cat, proj1[0], proj1[1]), proj2[0], proj2[1])
