"""CPU: the oracle against golden vectors recorded from the reference's own kernels
(tests/golden/*.npz, produced on a B200 by tests/golden/make_golden_ref.py)."""
import glob
import os

import numpy as np
import pytest

import fp4_oracle as o

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    path = os.path.join(GOLD, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} not recorded yet")
    return np.load(path)


def test_fixture_set_is_present():
    names = {os.path.basename(p) for p in glob.glob(os.path.join(GOLD, "*.npz"))}
    assert {"ref_dequant.npz", "ref_fp4_linear_a.npz", "ref_fp4_linear_b.npz", "ref_elementwise.npz"} <= names


def test_dequant_bit_exact():
    z = load("ref_dequant.npz")
    assert np.array_equal(o.fp4_dequant_to_bf16(z["packed"], z["scales"], float(z["g"])), z["out"])


@pytest.mark.parametrize("tag", ["a", "b"])
def test_fp4_linear_within_rounding(tag):
    z = load(f"ref_fp4_linear_{tag}.npz")
    pre = z["pre"] if z["pre"].size else None
    mine = o.fp4_linear(z["x"], z["packed"], z["scales"], float(z["g"]), pre)
    assert o.rel_err(mine, z["out"]) <= 4e-3      # fp32 accumulation order + one bf16 rounding


@pytest.mark.parametrize("tag", ["a", "b"])
def test_nvfp4_linear_within_rounding(tag):
    z = load(f"ref_nvfp4_linear_{tag}.npz")
    pre = z["pre"] if z["pre"].size else None
    mine = o.nvfp4_linear(z["x"], z["packed"], z["scales"], float(z["input_scale"]), float(z["g"]), pre)
    assert o.rel_err(mine, z["out"]) <= 4e-3


def test_elementwise_bit_exact_and_argmax():
    z = load("ref_elementwise.npz")
    assert np.array_equal(o.silu_mul_split_packed(z["gate_up"]), z["silu"])
    assert np.array_equal(o.residual_add(z["a"], z["b"]), z["residual"])
    assert o.argmax_rows_ref(z["logits"]).tolist() == z["tokens"].tolist()
