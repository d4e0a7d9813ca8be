"""GPU parity, element-wise kernels: bit-exact against the oracle (integer/byte work and fp32
element-wise math in the reference's operation order)."""
import numpy as np
import pytest
import torch

import fp4_oracle as o
from gpu_util import bits_of, to_dev_bf16, to_dev_u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from glm_asr_stack_b200 import ops as _ops
    assert torch.cuda.is_available()
    return _ops


@pytest.mark.parametrize("rows,cols", [(1, 16), (7, 64), (128, 2048), (513, 272)])
def test_dequant_bit_exact(ops, rows, cols):
    pw, sw, g = o.seeded_weight(rows, cols, 11)
    sw[0, 0] = 0x7F                                   # the reference decodes 0x7F as 480, not NaN
    sw[-1, -1] = 0x01                                 # smallest subnormal scale
    out = ops.fp4_dequant_to_bf16(to_dev_u8(pw), to_dev_u8(sw), g)
    assert np.array_equal(bits_of(out), o.fp4_dequant_to_bf16(pw, sw, g))
    out = ops.fp4_dequant_to_bf16(to_dev_u8(pw), None, 0.5)      # NULL scales -> 1
    assert np.array_equal(bits_of(out), o.fp4_dequant_to_bf16(pw, None, 0.5))


def test_dequant_odd_column_count(ops):
    # packed pitch (cols+1)/2, scale pitch (cols+15)/16 (Infer-engine/cuda/kernels.cu:213,224)
    rows, cols = 5, 37
    rng = np.random.default_rng(0)
    pw = rng.integers(0, 256, (rows, (cols + 1) // 2), dtype=np.uint8)
    sw = rng.integers(0x20, 0x50, (rows, (cols + 15) // 16), dtype=np.uint8)
    out = ops.fp4_dequant_to_bf16(to_dev_u8(pw), to_dev_u8(sw), 0.125, rows, cols)
    q = o.unpack_nibbles(pw)[:, :cols]
    want = (o.E2M1_LUT[q] * np.repeat(o.E4M3_TABLE[sw], 16, axis=1)[:, :cols]).astype(np.float32) * np.float32(0.125)
    assert np.array_equal(bits_of(out), o.f32_to_bf16_bits(want))


@pytest.mark.parametrize("M,K,with_pre", [(1, 16, False), (17, 64, True), (129, 2048, False), (300, 512, True),
                                          (1100, 2048, False), (1030, 4096, False), (1025, 2048, True)])
def test_activation_quantiser_bit_exact(ops, M, K, with_pre):
    x = o.seeded_activation(M, K, 5)
    xf = o.bf16_bits_to_f32(x)
    xf[0, :16] = 0.0                                   # all-zero block
    if M > 1:
        xf[1, :16] = 1e-30                             # scale rounds to zero
        xf[-1, -16:] = 1e4                             # saturating values
    x = o.f32_to_bf16_bits(xf)
    pre = o.f32_to_bf16_bits(np.random.default_rng(1).uniform(0.5, 2.0, K).astype(np.float32)) if with_pre else None
    isc = 0.37 * o.default_input_scale(x)
    p, s = ops.quantize_bf16_to_fp4(to_dev_bf16(x), isc, to_dev_bf16(pre) if with_pre else None)
    wp, wsc = o.quantize_bf16_to_fp4(x, isc, pre)
    assert np.array_equal(s.cpu().numpy(), wsc)
    assert np.array_equal(p.cpu().numpy(), wp)


@pytest.mark.parametrize("rows,cols", [(1, 1), (130, 6), (256, 128), (10000, 128)])
def test_scale_swizzle_bit_exact(ops, rows, cols):
    s = np.random.default_rng(2).integers(0, 256, (rows, cols), dtype=np.uint8)
    got = ops.swizzle_rowwise_scales(to_dev_u8(s)).cpu().numpy()
    assert np.array_equal(got, o.swizzle_rowwise_scales(s))


def test_silu_and_residual_bit_exact(ops):
    rng = np.random.default_rng(3)
    gu = o.f32_to_bf16_bits(rng.standard_normal((33, 2 * 96)).astype(np.float32) * 4)
    assert np.array_equal(bits_of(ops.silu_mul_split_packed(to_dev_bf16(gu))), o.silu_mul_split_packed(gu))
    g = o.f32_to_bf16_bits(rng.standard_normal(1000).astype(np.float32) * 4)
    u = o.f32_to_bf16_bits(rng.standard_normal(1000).astype(np.float32))
    assert np.array_equal(bits_of(ops.silu_elementwise_mul(to_dev_bf16(g), to_dev_bf16(u))),
                          o.silu_elementwise_mul(g, u))
    assert np.array_equal(bits_of(ops.residual_add(to_dev_bf16(g), to_dev_bf16(u))), o.residual_add(g, u))


def test_argmax_with_ties_matches_reference_order(ops):
    rng = np.random.default_rng(4)
    vocab = 59264
    v = rng.standard_normal((6, vocab)).astype(np.float32)
    v[1, [300, 5, 40000]] = 9.0                 # ties across threads
    v[2, [7 + 512, 7 + 256]] = 9.0              # ties inside one thread's slice
    v[3, :] = -3e38                             # below the -1e20 floor -> 0
    v[4, vocab - 1] = 50.0                      # last element
    bits = o.f32_to_bf16_bits(v)
    got = ops.argmax_rows(to_dev_bf16(bits)).cpu().numpy()
    assert got.tolist() == o.argmax_rows_ref(bits).tolist()
    # the wide-row kernel cuts a row into column ranges and merges them by a per-row counter that must be back at
    # zero after every launch, also when the row count (and with it the scratch layout) changes between launches
    for rows in (256, 5, 300, 5):
        w = rng.standard_normal((rows, vocab)).astype(np.float32)
        w[rows // 2, [11, 20000, 45000, vocab - 3]] = 7.5
        wb = o.f32_to_bf16_bits(w)
        for _ in range(2):
            assert ops.argmax_rows(to_dev_bf16(wb)).cpu().numpy().tolist() == o.argmax_rows_ref(wb).tolist()
    # unaligned row pitch (vocab not a multiple of 8)
    b2 = o.f32_to_bf16_bits(rng.standard_normal((3, 1001)).astype(np.float32))
    assert ops.argmax_rows(to_dev_bf16(b2)).cpu().numpy().tolist() == o.argmax_rows_ref(b2).tolist()
