"""CPU oracle for the GLM-ASR Infer-engine FP4-weight linear path (numpy).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module:
it is the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

Parity status: the reference ships no tests, golden vectors or CPU code for
this path, so this restatement is pinned in two other ways:
  * the rounding primitives (e2m1 / e4m3 encode) are checked bit-for-bit
    against NVIDIA's host-callable ``__nv_fp4_e2m1`` / ``__nv_fp8_e4m3``
    constructors (the ones the reference's quantiser calls) and against
    ``ml_dtypes``;
  * the whole-function outputs are checked against fixtures under
    ``tests/golden/`` that were produced by running the reference's own
    ``fp4_linear`` / ``nvfp4_linear`` / ``fp4_dequant_to_bf16`` objects
    (compiled unmodified from the reference sources) on a B200.

Every function cites the reference file:line (paths inside the reference
project) whose arithmetic it restates.  All float math is done in float32 in
the same operation order as the reference kernels so that element-wise
functions are bit-exact; only GEMM accumulation order is unspecified (cuBLAS).
"""
from __future__ import annotations

import numpy as np

F32 = np.float32

# --------------------------------------------------------------------------
# bf16 helpers (numpy has no bfloat16; carry bf16 as uint16 bit patterns)
# --------------------------------------------------------------------------


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit pattern (``__float2bfloat16``)."""
    x = np.ascontiguousarray(x, dtype=F32)
    u = x.view(np.uint32)
    nan = np.isnan(x)
    rounded = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
    rounded = np.where(nan, np.uint16(0x7FFF), rounded)
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << np.uint32(16)).view(F32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bf16, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# --------------------------------------------------------------------------
# a1: number formats
# --------------------------------------------------------------------------

#: Infer-engine/cuda/kernels.cu:96-99 -- nibble -> value
E2M1_LUT = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
     -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=F32)


def e4m3_decode_ref(b: np.ndarray) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:103-120 (``fp8_to_float_e4m3``).

    The reference treats every bit pattern as a number: 0x7F / 0xFF decode to
    +-480 instead of NaN.
    """
    b = np.asarray(b, dtype=np.uint8)
    sign = (b >> 7) & 1
    exp = ((b >> 3) & 0x0F).astype(np.int32)
    mant = (b & 0x07).astype(F32)
    den = (mant / F32(8.0)) * F32(0.015625)
    nor = ((F32(8.0) + mant) / F32(8.0)) * np.exp2((exp - 7).astype(F32)).astype(F32)
    v = np.where(exp == 0, den, nor).astype(F32)
    return np.where(sign == 1, -v, v).astype(F32)


#: all 256 decodes, handy as a table
E4M3_TABLE = e4m3_decode_ref(np.arange(256, dtype=np.uint8))


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3 byte, RNE, saturate-to-finite (+-448), NaN -> 0x7F.

    Restates ``__nv_fp8_e4m3(float)`` (= ``__nv_cvt_float_to_fp8(x,
    __NV_SATFINITE, __NV_E4M3)``), which Infer-engine/cuda/nvfp4_cutlass.cu:68
    uses for the activation block scale.
    """
    x = np.asarray(x, dtype=F32)
    sign = np.signbit(x).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    out = np.zeros(x.shape, dtype=np.uint8)
    # candidates: all finite non-negative e4m3 values (0x00..0x7E), monotone
    vals = E4M3_TABLE[:0x7F].astype(np.float64)
    idx = np.searchsorted(vals, a, side="left")          # first vals[idx] >= a
    idx = np.clip(idx, 1, 0x7E)
    lo = vals[idx - 1]
    hi = vals[idx]
    dlo = a - lo
    dhi = hi - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((idx % 2) == 0))   # tie -> even code
    code = np.where(pick_hi, idx, idx - 1)
    code = np.where(a >= 448.0, 0x7E, code)
    code = np.where(a == 0.0, 0, code)
    out = code.astype(np.uint8) | sign
    out = np.where(np.isnan(x), np.uint8(0x7F), out)
    return out.astype(np.uint8)


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> e2m1 nibble, RNE, saturate-to-finite (+-6).

    Restates ``__nv_fp4_e2m1(float)`` (``__nv_cvt_float_to_fp4(x, __NV_E2M1,
    cudaRoundNearest)``), used by Infer-engine/cuda/nvfp4_cutlass.cu:79-80.
    NaN maps to the positive maximum 0x7, as the NVIDIA conversion does.
    """
    x = np.asarray(x, dtype=F32)
    sign = np.signbit(x).astype(np.uint8) << 3
    a = np.abs(x).astype(np.float64)
    vals = E2M1_LUT[:8].astype(np.float64)
    idx = np.clip(np.searchsorted(vals, a, side="left"), 1, 7)
    lo = vals[idx - 1]
    hi = vals[idx]
    dlo = a - lo
    dhi = hi - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((idx % 2) == 0))
    code = np.where(pick_hi, idx, idx - 1)
    code = np.where(a >= 6.0, 7, code)
    code = np.where(a == 0.0, 0, code)
    out = code.astype(np.uint8) | sign
    out = np.where(np.isnan(x), np.uint8(0x7), out)
    return out.astype(np.uint8)


def pack_nibbles(q: np.ndarray) -> np.ndarray:
    """[..., K] nibbles -> [..., K/2] bytes: even k in bits 0-3, odd k in bits
    4-7 (Infer-engine/cuda/kernels.cu:205-219, nvfp4_cutlass.cu:81)."""
    q = np.asarray(q, dtype=np.uint8)
    assert q.shape[-1] % 2 == 0
    return ((q[..., 0::2] & 0x0F) | ((q[..., 1::2] & 0x0F) << 4)).astype(np.uint8)


def unpack_nibbles(p: np.ndarray) -> np.ndarray:
    p = np.asarray(p, dtype=np.uint8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = p & 0x0F
    out[..., 1::2] = (p >> 4) & 0x0F
    return out


# --------------------------------------------------------------------------
# a2: fp4_dequant_to_bf16
# --------------------------------------------------------------------------


def dequant_f32(packed_w: np.ndarray, block_scales: np.ndarray | None,
                global_scale: float) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:188-232 without the final bf16 rounding:
    ``(lut[nibble] * e4m3(scale[r, c/16])) * global`` in float32."""
    q = unpack_nibbles(packed_w)
    w = E2M1_LUT[q]
    if block_scales is not None:
        s = E4M3_TABLE[np.asarray(block_scales, dtype=np.uint8)]
        w = (w * np.repeat(s, 16, axis=-1)[..., : w.shape[-1]]).astype(F32)
    return (w * F32(global_scale)).astype(F32)


def fp4_dequant_to_bf16(packed_w, block_scales, global_scale) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:188-246; returns bf16 bit patterns [rows, cols]."""
    return f32_to_bf16_bits(dequant_f32(packed_w, block_scales, global_scale))


# --------------------------------------------------------------------------
# a3/a4: fp4_linear (W4A16 fallback) and the fp32 oracle O1
# --------------------------------------------------------------------------


def apply_prequant(x_bits: np.ndarray, pre_bits: np.ndarray) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:1280-1295: bf16(x[m,k] * pre[k])."""
    return f32_to_bf16_bits(bf16_bits_to_f32(x_bits) * bf16_bits_to_f32(pre_bits)[None, :])


def _matmul_f32(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """x[M,K] @ w[N,K]^T with float64 accumulation, returned float32.

    cuBLAS only promises fp32 accumulation in an unspecified order
    (Infer-engine/cuda/kernels.cu:1165-1177); float64 is the order-free
    stand-in the tolerance tests compare against.
    """
    return (x.astype(np.float64) @ w.astype(np.float64).T).astype(F32)


def linear_o1(x_bits, packed_w, block_scales, global_scale, pre_bits=None) -> np.ndarray:
    """O1: float32 dequantise-then-matmul of the stored FP4 format; weights are
    NOT rounded to bf16.  Returns bf16 bits [M, N]."""
    x = bf16_bits_to_f32(x_bits)
    if pre_bits is not None:
        x = (x * bf16_bits_to_f32(pre_bits)[None, :]).astype(F32)
    w = dequant_f32(packed_w, block_scales, global_scale)
    return f32_to_bf16_bits(_matmul_f32(x, w))


def fp4_linear(x_bits, packed_w, block_scales, global_scale, pre_bits=None,
               bias_bits=None) -> np.ndarray:
    """O1': Infer-engine/cuda/kernels.cu:1297-1318 -- optional a3, then a2 (weights
    rounded to bf16), then ``bf16_linear`` (kernels.cu:1147-1193: fp32 accumulate,
    bf16 out; a non-NULL bias is added by the GEMM epilogue / add_bias kernel)."""
    if pre_bits is not None:
        x_bits = apply_prequant(x_bits, pre_bits)
    w = bf16_bits_to_f32(fp4_dequant_to_bf16(packed_w, block_scales, global_scale))
    acc = _matmul_f32(bf16_bits_to_f32(x_bits), w)
    if bias_bits is not None:
        acc = (acc + bf16_bits_to_f32(bias_bits)[None, :]).astype(F32)
    return f32_to_bf16_bits(acc)


# --------------------------------------------------------------------------
# a5: activation quantiser, a6: scale swizzle, a7: nvfp4_linear (W4A4), O2
# --------------------------------------------------------------------------


def quantize_bf16_to_fp4(x_bits: np.ndarray, input_scale: float,
                         pre_bits: np.ndarray | None = None):
    """Infer-engine/cuda/nvfp4_cutlass.cu:35-87.

    Returns (packed [M, K/2] u8, scales [M, K/16] u8) for the M real rows (the
    reference also zero-fills scale rows M..ceil16(M)).
    """
    inv_in = F32(1.0) / F32(input_scale)                       # nvfp4_cutlass.cu:172
    x = bf16_bits_to_f32(x_bits)
    if pre_bits is not None:
        x = (x * bf16_bits_to_f32(pre_bits)[None, :]).astype(F32)
    M, K = x.shape
    assert K % 16 == 0
    xb = x.reshape(M, K // 16, 16)
    amax = np.abs(xb).max(axis=-1).astype(F32)
    with np.errstate(divide="ignore", invalid="ignore"):
        scale = np.where(amax > 0, ((inv_in * amax).astype(F32) / F32(6.0)).astype(F32), F32(0)).astype(F32)
        s_byte = e4m3_encode(scale)
        # (float)s_fp8 is NVIDIA's decode; identical to the table for finite codes
        scale_rounded = np.where(scale > 0, E4M3_TABLE[s_byte], F32(0)).astype(F32)
        out_scale = np.where(scale_rounded > 0, (inv_in / scale_rounded).astype(F32), F32(0)).astype(F32)
    q = e2m1_encode((xb * out_scale[..., None]).astype(F32)).reshape(M, K)
    return pack_nibbles(q), s_byte.astype(np.uint8)


def swizzled_scale_index(r, c, col_tiles):
    """Infer-engine/cuda/nvfp4_cutlass.cu:101-109."""
    r = np.asarray(r, dtype=np.int64)
    c = np.asarray(c, dtype=np.int64)
    return ((((r // 128) * col_tiles + c // 4) * 32 + (r % 128) % 32) * 4 + (r % 128) // 32) * 4 + c % 4


def swizzle_rowwise_scales(scales: np.ndarray) -> np.ndarray:
    """Infer-engine/cuda/nvfp4_cutlass.cu:89-111 into a zero-filled buffer of
    ceil128(rows) * ceil4(cols) bytes (the memsets at :167-170)."""
    rows, cols = scales.shape
    rows_p = (rows + 127) // 128 * 128
    cols_p = (cols + 3) // 4 * 4
    out = np.zeros(rows_p * cols_p, dtype=np.uint8)
    rr, cc = np.meshgrid(np.arange(rows), np.arange(cols), indexing="ij")
    out[swizzled_scale_index(rr, cc, cols_p // 4)] = scales
    return out


def nvfp4_linear(x_bits, packed_w, block_scales, input_scale, global_scale,
                 pre_bits=None) -> np.ndarray:
    """O2: Infer-engine/cuda/nvfp4_cutlass.cu:118-270 -- quantise activations (a5),
    block-scaled FP4 x FP4 product with fp32 accumulation, alpha =
    input_scale * w_global_scale, bf16 out.  ``bias`` is ignored by the
    reference (:163).  Returns bf16 bits [M, N]."""
    xq, xs = quantize_bf16_to_fp4(x_bits, input_scale, pre_bits)
    xa = dequant_f32(xq, xs, 1.0)
    wa = dequant_f32(packed_w, block_scales, 1.0)
    alpha = F32(input_scale) * F32(global_scale)
    acc = _matmul_f32(xa, wa)
    return f32_to_bf16_bits((acc * alpha).astype(F32))


def nvfp4_linear_args_ok(M, N, K, w_scales_present, input_scale) -> bool:
    """Guards at Infer-engine/cuda/nvfp4_cutlass.cu:128-131 (return -1 when False)."""
    return M > 0 and N > 0 and K > 0 and w_scales_present and K % 16 == 0 and input_scale > 0.0


# --------------------------------------------------------------------------
# a12/a13/a14: fused-away elementwise ops
# --------------------------------------------------------------------------


def silu_mul_split_packed(packed_gate_up_bits: np.ndarray) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:1252-1264: [M, 2N] -> bf16((g*sigmoid(g))*u)."""
    M, N2 = packed_gate_up_bits.shape
    N = N2 // 2
    g = bf16_bits_to_f32(packed_gate_up_bits[:, :N])
    u = bf16_bits_to_f32(packed_gate_up_bits[:, N:])
    sig = (F32(1.0) / (F32(1.0) + np.exp(-g).astype(F32))).astype(F32)
    return f32_to_bf16_bits(((g * sig).astype(F32) * u).astype(F32))


def silu_elementwise_mul(gate_bits, up_bits):
    """Infer-engine/cuda/kernels.cu:405-413: bf16(g*sigmoid(g)*u), left to right."""
    g = bf16_bits_to_f32(gate_bits)
    u = bf16_bits_to_f32(up_bits)
    sig = (F32(1.0) / (F32(1.0) + np.exp(-g).astype(F32))).astype(F32)
    return f32_to_bf16_bits(((g * sig).astype(F32) * u).astype(F32))


def residual_add(a_bits, b_bits):
    """Infer-engine/cuda/kernels.cu:741-752: bf16(float(a)+float(b))."""
    return f32_to_bf16_bits((bf16_bits_to_f32(a_bits) + bf16_bits_to_f32(b_bits)).astype(F32))


def argmax_rows_ref(logits_bits: np.ndarray, threads: int = 256) -> np.ndarray:
    """Infer-engine/cuda/kernels.cu:1387-1426 including its tie-break, simulated literally:
    each of the 256 threads keeps the lowest index of its strided maximum, then a
    strict-``>`` tree reduce merges slot t+off into slot t (the lower slot keeps ties), which
    orders tied threads by their bit-reversed id."""
    rows, vocab = logits_bits.shape
    vals = bf16_bits_to_f32(logits_bits)
    out = np.zeros(rows, dtype=np.int32)
    for r in range(rows):
        best_val = np.full(threads, F32(-1e20), dtype=F32)
        best_idx = np.zeros(threads, dtype=np.int64)
        for t in range(threads):
            v = vals[r, t::threads]
            if v.size:
                j = int(np.argmax(v))            # first occurrence of the max
                if v[j] > best_val[t]:
                    best_val[t] = v[j]
                    best_idx[t] = t + j * threads
        off = threads // 2
        while off > 0:
            take = best_val[off:2 * off] > best_val[:off]
            best_val[:off] = np.where(take, best_val[off:2 * off], best_val[:off])
            best_idx[:off] = np.where(take, best_idx[off:2 * off], best_idx[:off])
            off //= 2
        out[r] = best_idx[0]
    return out


# --------------------------------------------------------------------------
# Synthetic weight quantiser (builder-defined: the reference only ever loads
# pre-quantised checkpoints).  Same rounding rules as the activation quantiser.
# --------------------------------------------------------------------------


def quantize_weight(w: np.ndarray):
    """fp32 [N, K] -> (packed [N, K/2], scales [N, K/16], global fp32).

    g = amax(W)/(6*448); per 16-K block s = e4m3(amax_blk/(6*g));
    q = e2m1(w/(float(s)*g)); low nibble = even k.
    """
    w = np.asarray(w, dtype=F32)
    N, K = w.shape
    assert K % 16 == 0
    g = F32(np.abs(w).max()) / F32(6.0 * 448.0)
    if g == 0:
        g = F32(1.0)
    wb = w.reshape(N, K // 16, 16)
    amax = np.abs(wb).max(axis=-1).astype(F32)
    s_byte = e4m3_encode((amax / (F32(6.0) * g)).astype(F32))
    s = E4M3_TABLE[s_byte]
    with np.errstate(divide="ignore", invalid="ignore"):
        denom = (s * g).astype(F32)
        y = np.where(denom[..., None] > 0, (wb / denom[..., None]).astype(F32), F32(0)).astype(F32)
    q = e2m1_encode(y).reshape(N, K)
    return pack_nibbles(q), s_byte.astype(np.uint8), float(g)


# --------------------------------------------------------------------------
# Seeded inputs of the benchmark configurations (shapes only; synthetic data)
# --------------------------------------------------------------------------


def seeded_weight(N: int, K: int, seed: int):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K), dtype=F32) * F32(0.02)).astype(F32)
    return quantize_weight(w)


def seeded_activation(M: int, K: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return f32_to_bf16_bits(rng.standard_normal((M, K), dtype=F32))


def default_input_scale(x_bits: np.ndarray) -> float:
    """input_scale = amax(x)/(6*448) (per-tensor activation scale of the W4A4 path)."""
    a = float(np.abs(bf16_bits_to_f32(x_bits)).max())
    return float(F32(a) / F32(6.0 * 448.0)) if a > 0 else 1.0


def rel_err(a_bits, b_bits) -> float:
    a = bf16_bits_to_f32(a_bits).astype(np.float64)
    b = bf16_bits_to_f32(b_bits).astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def cosine(a_bits, b_bits) -> float:
    a = bf16_bits_to_f32(a_bits).astype(np.float64).ravel()
    b = bf16_bits_to_f32(b_bits).astype(np.float64).ravel()
    return float(a @ b / max(np.linalg.norm(a) * np.linalg.norm(b), 1e-30))
