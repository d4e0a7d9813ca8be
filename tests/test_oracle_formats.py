"""CPU tests of the oracle itself: number formats, rounding, index math, tie-breaks.

The reference has no tests or golden vectors for this path; these known-answer tests pin the
oracle's primitives against (a) the constants written in the reference source, (b) NVIDIA's
host-callable converters that the reference's quantiser calls, (c) an independent plain-C
restatement, (d) ml_dtypes.
"""
import ctypes

import numpy as np
import pytest

import fp4_oracle as o


def test_e2m1_lut_matches_reference_table():
    # Infer-engine/cuda/kernels.cu:96-99
    want = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    assert o.E2M1_LUT.tolist() == want
    assert np.signbit(o.E2M1_LUT[8])


def test_e4m3_decode_all_256_codes():
    # Infer-engine/cuda/kernels.cu:103-120: closed form, no NaN pattern
    for b in range(256):
        s, e, m = b >> 7, (b >> 3) & 15, b & 7
        v = (m / 8.0) * 2.0 ** -6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7)
        v = -v if s else v
        assert o.E4M3_TABLE[b] == np.float32(v), b
    assert o.E4M3_TABLE[0x7F] == 480.0 and o.E4M3_TABLE[0xFF] == -480.0
    assert o.E4M3_TABLE[0x7E] == 448.0 and o.E4M3_TABLE[0x01] == 2.0 ** -9


def test_e4m3_decode_matches_ml_dtypes_except_nan_codes():
    import ml_dtypes
    b = np.arange(256, dtype=np.uint8)
    ml = b.view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    ok = ~np.isnan(ml)
    assert np.array_equal(ml[ok], o.E4M3_TABLE[ok])
    assert set(np.nonzero(~ok)[0]) == {0x7F, 0xFF}


def _sweep():
    rng = np.random.default_rng(0)
    xs = [rng.standard_normal(50000).astype(np.float32) * s for s in (1e-3, 1e-2, 0.1, 1, 10, 100, 1000)]
    tab = o.E4M3_TABLE[:0x7F].astype(np.float64)
    mids = ((tab[1:] + tab[:-1]) / 2).astype(np.float32)
    e2 = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0], dtype=np.float32)
    pts = np.concatenate([mids, tab.astype(np.float32), e2,
                          np.array([0, 448, 449, 463.9, 464, 465, 480, 1e9, np.inf, 2.0 ** -10, 2.0 ** -11],
                                   dtype=np.float32)])
    pts = np.concatenate([pts, np.nextafter(pts, np.float32(0)), np.nextafter(pts, np.float32(np.inf))])
    return np.concatenate(xs + [pts, -pts])


def test_encoders_match_nvidia_host_converters(oracle_libs):
    nv = ctypes.CDLL(oracle_libs["nv"])
    xs = _sweep()
    out = np.zeros(xs.size, np.uint8)
    nv.nv_e4m3_encode(xs.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), xs.size)
    assert np.array_equal(o.e4m3_encode(xs), out)
    nv.nv_e2m1_encode(xs.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), xs.size)
    assert np.array_equal(o.e2m1_encode(xs) & 0xF, out & 0xF)
    nan = np.array([np.nan], np.float32)
    assert o.e4m3_encode(nan)[0] == 0x7F and o.e2m1_encode(nan)[0] == 0x7


def test_e2m1_known_answers():
    # values checked when the blueprint was written: 0.75 -> 1.0, 2.5 -> 2.0 (ties to even), 500 -> 448 for e4m3
    assert o.E2M1_LUT[o.e2m1_encode(np.float32([0.75]))][0] == 1.0
    assert o.E2M1_LUT[o.e2m1_encode(np.float32([2.5]))][0] == 2.0
    assert o.E2M1_LUT[o.e2m1_encode(np.float32([-100.0]))][0] == -6.0
    assert o.E4M3_TABLE[o.e4m3_encode(np.float32([500.0]))][0] == 448.0


def test_c_oracle_agrees_with_numpy(oracle_libs):
    c = ctypes.CDLL(oracle_libs["c"])
    c.oracle_e4m3_encode.restype = ctypes.c_uint8
    c.oracle_e4m3_encode.argtypes = [ctypes.c_float]
    c.oracle_e2m1_encode.restype = ctypes.c_uint8
    c.oracle_e2m1_encode.argtypes = [ctypes.c_float]
    c.oracle_e4m3_decode.restype = ctypes.c_float
    c.oracle_e4m3_decode.argtypes = [ctypes.c_uint8]
    xs = _sweep()[::13]
    assert np.array_equal(np.array([c.oracle_e4m3_encode(float(v)) for v in xs], np.uint8), o.e4m3_encode(xs))
    assert np.array_equal(np.array([c.oracle_e2m1_encode(float(v)) for v in xs], np.uint8) & 0xF,
                          o.e2m1_encode(xs) & 0xF)
    assert [c.oracle_e4m3_decode(b) for b in range(256)] == o.E4M3_TABLE.tolist()

    # whole functions on a small seeded case
    M, N, K = 9, 24, 64
    P = ctypes.c_void_p
    pw, sw, g = o.seeded_weight(N, K, 3)
    x = o.seeded_activation(M, K, 4)
    pre = o.f32_to_bf16_bits(np.random.default_rng(5).uniform(0.5, 2, K).astype(np.float32))
    deq = np.zeros((N, K), np.uint16)
    c.oracle_fp4_dequant_to_bf16(deq.ctypes.data_as(P), pw.ctypes.data_as(P), sw.ctypes.data_as(P),
                                 ctypes.c_float(g), N, K)
    assert np.array_equal(deq, o.fp4_dequant_to_bf16(pw, sw, g))
    qp = np.zeros((M, K // 2), np.uint8)
    qs = np.zeros((M, K // 16), np.uint8)
    isc = o.default_input_scale(x)
    c.oracle_quantize_bf16_to_fp4(qp.ctypes.data_as(P), qs.ctypes.data_as(P), x.ctypes.data_as(P),
                                  pre.ctypes.data_as(P), ctypes.c_float(isc), M, K)
    p2, s2 = o.quantize_bf16_to_fp4(x, isc, pre)
    assert np.array_equal(qp, p2) and np.array_equal(qs, s2)
    out = np.zeros((M, N), np.uint16)
    scratch = np.zeros((N, K), np.uint16)
    c.oracle_fp4_linear(out.ctypes.data_as(P), scratch.ctypes.data_as(P), x.ctypes.data_as(P), pw.ctypes.data_as(P),
                        sw.ctypes.data_as(P), ctypes.c_float(g), pre.ctypes.data_as(P), M, N, K)
    ref = o.fp4_linear(x, pw, sw, g, pre)
    # fp32 sequential accumulation vs float64: at most one bf16 ulp apart
    assert o.rel_err(out, ref) < 3e-3
    c.oracle_swizzled_scale_index.restype = ctypes.c_size_t
    for r, cc, t in [(0, 0, 1), (5, 3, 2), (37, 6, 2), (127, 7, 2), (128, 0, 2), (300, 130, 33)]:
        assert c.oracle_swizzled_scale_index(r, cc, t) == int(o.swizzled_scale_index(r, cc, t))


def test_nibble_order_and_dequant_known_answer():
    # byte 0x21 -> k even = nibble 1 (0.5), k odd = nibble 2 (1.0); scale 0x38 = 1.0; global 2
    packed = np.array([[0x21, 0xF7]], np.uint8)
    scales = np.array([[0x38]], np.uint8)
    d = o.bf16_bits_to_f32(o.fp4_dequant_to_bf16(packed, scales, 2.0))
    assert d.tolist() == [[1.0, 2.0, 12.0, -12.0]]
    assert o.unpack_nibbles(o.pack_nibbles(np.arange(16, dtype=np.uint8)[None])).tolist() == [list(range(16))]


def test_swizzle_index_hand_picked():
    # Infer-engine/cuda/nvfp4_cutlass.cu:101-109, worked by hand
    assert int(o.swizzled_scale_index(0, 0, 1)) == 0
    assert int(o.swizzled_scale_index(1, 0, 1)) == 16
    assert int(o.swizzled_scale_index(32, 0, 1)) == 4
    assert int(o.swizzled_scale_index(33, 2, 1)) == 16 + 4 + 2
    assert int(o.swizzled_scale_index(0, 4, 2)) == 512
    assert int(o.swizzled_scale_index(128, 0, 2)) == 1024
    s = np.arange(130 * 6, dtype=np.uint32).astype(np.uint8).reshape(130, 6)
    t = o.swizzle_rowwise_scales(s)
    assert t.size == 256 * 8
    assert t[int(o.swizzled_scale_index(129, 5, 2))] == s[129, 5]
    # it is a permutation of the real entries, zero elsewhere
    assert np.array_equal(np.sort(t[t != 0]), np.sort(s[s != 0].ravel()))


def test_quantizer_edge_cases():
    K = 32
    x = np.zeros((3, K), np.float32)
    x[1, :16] = 3.0                       # constant block
    x[2, 0] = 1e-30                       # scale underflows to e4m3 zero -> everything quantises to 0
    xb = o.f32_to_bf16_bits(x)
    p, s = o.quantize_bf16_to_fp4(xb, 1.0)
    assert not p[0].any() and not s[0].any()
    # amax 3, input_scale 1: scale = 0.5 exactly -> q = 3/0.5 = 6 -> code 7 everywhere in the block
    assert s[1, 0] == o.e4m3_encode(np.float32([0.5]))[0] and (p[1, :8] == 0x77).all() and not p[1, 8:].any()
    assert not p[2].any() and s[2, 0] == 0
    assert o.nvfp4_linear_args_ok(1, 1, 16, True, 1.0)
    assert not o.nvfp4_linear_args_ok(1, 1, 24, True, 1.0)
    assert not o.nvfp4_linear_args_ok(0, 1, 16, True, 1.0)
    assert not o.nvfp4_linear_args_ok(1, 1, 16, False, 1.0)
    assert not o.nvfp4_linear_args_ok(1, 1, 16, True, 0.0)


def test_argmax_tie_break_matches_reference_order():
    v = np.full((3, 600), -1.0, np.float32)
    # Traced by hand through the reference's tree (kernels.cu:1414-1420): slot t absorbs slot
    # t+off on strict >, so tied threads are ordered by their bit-reversed id.
    v[0, [300, 5]] = 2.0        # threads 44 (0b00101100) and 5 (0b00000101): bit 0 differs, 44 wins -> 300
    v[1, [261, 300]] = 2.0      # threads 5 and 44 again ...
    v[1, 4 + 256] = 2.0         # ... and thread 4: bitrev(4)=32 < bitrev(44)=52 < bitrev(5)=160 -> 260
    v[2, :] = -3e38             # nothing beats the -1e20 floor -> 0
    got = o.argmax_rows_ref(o.f32_to_bf16_bits(v))
    assert got.tolist() == [300, 260, 0]
    # same thread, two maxima: the first (lowest index) is kept
    w = np.full((1, 1000), -1.0, np.float32)
    w[0, [7 + 512, 7 + 256]] = 5.0
    assert o.argmax_rows_ref(o.f32_to_bf16_bits(w)).tolist() == [263]


def test_o1_o1prime_o2_relationships_small():
    M, N, K = 32, 48, 256
    pw, sw, g = o.seeded_weight(N, K, 0)
    x = o.seeded_activation(M, K, 1)
    o1 = o.linear_o1(x, pw, sw, g)
    o1p = o.fp4_linear(x, pw, sw, g)
    o2 = o.nvfp4_linear(x, pw, sw, o.default_input_scale(x), g)
    assert o.rel_err(o1p, o1) < 5e-3            # bf16 rounding of weights and outputs only
    assert 2e-2 < o.rel_err(o2, o1) < 2e-1      # activation quantisation error is large and expected
    assert o.cosine(o2, o1) > 0.98


def test_silu_residual_match_plain_formulas():
    rng = np.random.default_rng(0)
    gu = o.f32_to_bf16_bits(rng.standard_normal((4, 16)).astype(np.float32) * 3)
    out = o.bf16_bits_to_f32(o.silu_mul_split_packed(gu))
    g = o.bf16_bits_to_f32(gu[:, :8]).astype(np.float64)
    u = o.bf16_bits_to_f32(gu[:, 8:]).astype(np.float64)
    assert np.allclose(out, g / (1 + np.exp(-g)) * u, rtol=1e-2, atol=1e-3)
    a = o.f32_to_bf16_bits(rng.standard_normal(64).astype(np.float32))
    b = o.f32_to_bf16_bits(rng.standard_normal(64).astype(np.float32))
    assert np.array_equal(o.residual_add(a, b),
                          o.f32_to_bf16_bits(o.bf16_bits_to_f32(a) + o.bf16_bits_to_f32(b)))
