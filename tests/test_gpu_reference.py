"""GPU: the reference's own kernels (oracle/_ref, compiled unmodified from the reference
sources) run beside the oracle and beside this library on the same inputs.  This is what pins
the oracle: element-wise functions must agree bit for bit, the GEMMs within bf16 rounding."""
import numpy as np
import pytest
import torch

import fp4_oracle as o
import ref_lib
from gpu_util import REL_TOL_TIGHT, bits_of, to_dev_bf16, to_dev_u8

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_lib.available(), reason="oracle/_ref not built")]


@pytest.fixture(scope="module")
def ref():
    return ref_lib.RefLib()


@pytest.fixture(scope="module")
def ops():
    from glm_asr_stack_b200 import ops as _ops
    return _ops


def test_reference_dequant_equals_oracle_and_library(ref, ops):
    pw, sw, g = o.seeded_weight(300, 512, 1)
    sw[0, 0] = 0x7F
    sw[1, 1] = 0x03
    want = o.fp4_dequant_to_bf16(pw, sw, g)
    assert np.array_equal(bits_of(ref.fp4_dequant_to_bf16(to_dev_u8(pw), to_dev_u8(sw), g)), want)
    assert np.array_equal(bits_of(ops.fp4_dequant_to_bf16(to_dev_u8(pw), to_dev_u8(sw), g)), want)


@pytest.mark.parametrize("M,N,K,pre", [(16, 128, 256, False), (130, 384, 512, True), (256, 6144, 2048, False)])
def test_reference_fp4_linear_vs_oracle_and_library(ref, ops, M, N, K, pre):
    pw, sw, g = o.seeded_weight(N, K, 0)
    x = o.seeded_activation(M, K, 1)
    pb = o.f32_to_bf16_bits(np.random.default_rng(2).uniform(0.5, 2, K).astype(np.float32)) if pre else None
    r = bits_of(ref.fp4_linear(to_dev_bf16(x), to_dev_u8(pw), to_dev_u8(sw), g, to_dev_bf16(pb) if pre else None))
    assert o.rel_err(r, o.fp4_linear(x, pw, sw, g, pb)) <= REL_TOL_TIGHT          # oracle O1' == reference
    mine = bits_of(ops.fp4_linear(to_dev_bf16(x), to_dev_u8(pw), to_dev_u8(sw), g, to_dev_bf16(pb) if pre else None))
    assert o.rel_err(mine, r) <= REL_TOL_TIGHT


@pytest.mark.parametrize("M,N,K,pre", [(16, 128, 256, False), (130, 384, 512, True), (256, 6144, 2048, False)])
def test_reference_nvfp4_linear_vs_oracle_and_library(ref, ops, M, N, K, pre):
    pw, sw, g = o.seeded_weight(N, K, 0)
    x = o.seeded_activation(M, K, 1)
    isc = o.default_input_scale(x)
    pb = o.f32_to_bf16_bits(np.random.default_rng(2).uniform(0.5, 2, K).astype(np.float32)) if pre else None
    rc, r = ref.nvfp4_linear(to_dev_bf16(x), to_dev_u8(pw), to_dev_u8(sw), isc, g, to_dev_bf16(pb) if pre else None)
    assert rc == 0, "the reference's cuBLASLt FP4 path did not run on this GPU"
    r = bits_of(r)
    assert o.rel_err(r, o.nvfp4_linear(x, pw, sw, isc, g, pb)) <= REL_TOL_TIGHT    # oracle O2 == reference
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    assert ops.nvfp4_linear(out, to_dev_bf16(x), to_dev_u8(pw), to_dev_u8(sw), isc, g,
                            to_dev_bf16(pb) if pre else None) == 0
    assert o.rel_err(bits_of(out), r) <= REL_TOL_TIGHT


def test_reference_elementwise_equal_oracle(ref):
    rng = np.random.default_rng(3)
    gu = o.f32_to_bf16_bits(rng.standard_normal((20, 128)).astype(np.float32) * 4)
    assert np.array_equal(bits_of(ref.silu_mul_split_packed(to_dev_bf16(gu))), o.silu_mul_split_packed(gu))
    a = o.f32_to_bf16_bits(rng.standard_normal(999).astype(np.float32))
    b = o.f32_to_bf16_bits(rng.standard_normal(999).astype(np.float32))
    assert np.array_equal(bits_of(ref.residual_add(to_dev_bf16(a), to_dev_bf16(b))), o.residual_add(a, b))


def test_reference_argmax_tie_break_equals_oracle(ref, ops):
    rows, dim, vocab = 4, 64, 2048
    h = np.zeros((rows, dim), np.float32)
    w = np.zeros((vocab, dim), np.float32)
    h[:, 0] = 1.0
    w[[300, 5, 1500], 0] = 3.0          # three tied maxima in every row
    w[7, 0] = 2.0
    hb, wb = o.f32_to_bf16_bits(h), o.f32_to_bf16_bits(w)
    logits = o.f32_to_bf16_bits(o.bf16_bits_to_f32(hb) @ o.bf16_bits_to_f32(wb).T)
    want = o.argmax_rows_ref(logits).tolist()
    assert ref.lm_head_argmax_batched(to_dev_bf16(hb), to_dev_bf16(wb)).tolist() == want
    assert ops.lm_head_argmax_batched(to_dev_bf16(hb), to_dev_bf16(wb)).tolist() == want
