"""Host-side logic that needs no GPU: weight store, dispatcher rules, synthetic quantiser."""
import numpy as np
import pytest
import torch

import fp4_oracle as o
from glm_asr_stack_b200 import ops, synth, weights


def test_synth_quantiser_is_bit_identical_to_the_oracle_quantiser():
    rng = np.random.default_rng(0)
    w = rng.standard_normal((48, 512), dtype=np.float32) * 0.02
    w[0, :16] = 0.0
    w[1, 3] = w.max() * 3
    p, s, g = o.quantize_weight(w)
    pt, st, gt = synth.quantize_weight(torch.from_numpy(w))
    assert np.array_equal(pt.numpy(), p) and np.array_equal(st.numpy(), s) and g == gt


def test_synth_e2m1_ties_to_even():
    y = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.75, 0.0])
    assert synth.e2m1_encode(y).tolist() == o.e2m1_encode(y.numpy()).tolist()


def test_weight_store_lookup_and_scalar_cache():
    ws = weights.WeightStore()
    ws.add("a.weight_scale_2", torch.tensor([0.25]))
    assert ws.get("missing") is None
    with pytest.raises(KeyError, match="Weight not found"):
        ws.require("missing")
    assert ws.scalar("a.weight_scale_2", 1.0) == 0.25
    assert ws.scalar("absent", 7.0) == 7.0
    ws.tensors["a.weight_scale_2"].data[0] = 9.0          # cached, like the reference's pointer cache
    assert ws.scalar("a.weight_scale_2", 1.0) == 0.25
    assert weights.SAFETENSORS_DTYPES["U8"] == weights.DTYPE_UINT8
    assert weights.SAFETENSORS_DTYPES["F8_E4M3"] == weights.DTYPE_FP8


def test_proj_names_follow_the_checkpoint_layout():
    n = weights.proj_names("language_model.model.layers.3.mlp.down_proj")
    assert n[0].endswith("down_proj.weight") and n[1].endswith(".weight_scale")
    assert n[2].endswith(".weight_scale_2") and n[3].endswith(".input_scale") and n[4].endswith(".pre_quant_scale")


def _fake_store(pre=False, bf16=False):
    ws = weights.WeightStore()
    for i, name in enumerate(("gate", "up")):
        if bf16:
            ws.add(f"{name}.weight", torch.zeros((4, 32), dtype=torch.bfloat16))
        else:
            ws.add(f"{name}.weight", torch.zeros((4, 16), dtype=torch.uint8))
            ws.add(f"{name}.weight_scale", torch.zeros((4, 2), dtype=torch.uint8), weights.DTYPE_FP8)
        ws.add(f"{name}.weight_scale_2", torch.tensor([0.5 + i]))
        ws.add(f"{name}.input_scale", torch.tensor([2.0]))
    if pre:
        ws.add("up.pre_quant_scale", torch.ones(32, dtype=torch.bfloat16))
    return ws


def test_dispatcher_rules(monkeypatch):
    calls = []
    monkeypatch.setattr(ops, "nvfp4_linear", lambda out, *a, **k: calls.append("nvfp4") or (-1 if a[3] <= 0 else 0))
    monkeypatch.setattr(ops, "fp4_linear", lambda *a, **k: calls.append("fp4") or k.get("out"))
    monkeypatch.setattr(ops, "bf16_linear", lambda *a, **k: calls.append("bf16"))
    monkeypatch.setattr(ops, "fp4_linear_fused", lambda mode, *a, **k: calls.append(("fused", mode)))
    x = torch.zeros((2, 32), dtype=torch.bfloat16)
    ws = _fake_store()
    names = weights.proj_names("gate")

    monkeypatch.delenv("GLMASR_USE_CUTLASS_NVFP4", raising=False)
    weights.linear_proj(ws, x, *names, 2, 4, 32, out=x)
    assert calls == ["fp4"]                                    # default: W4A16 fallback

    calls.clear()
    monkeypatch.setenv("GLMASR_USE_CUTLASS_NVFP4", "1")
    weights.linear_proj(ws, x, *names, 2, 4, 32, out=x)
    assert calls == ["nvfp4"]                                  # opt-in: W4A4

    calls.clear()
    weights.linear_proj(ws, x, *names, 2, 4, 32, use_native_nvfp4=False, out=x)
    assert calls == ["fp4"]

    calls.clear()
    monkeypatch.setenv("GLMASR_USE_CUTLASS_NVFP4", "0")
    weights.linear_proj(ws, x, *names, 2, 4, 32, out=x)
    assert calls == ["fp4"]                                    # "0" means off

    calls.clear()
    monkeypatch.setenv("GLMASR_USE_CUTLASS_NVFP4", "1")
    ws.add("gate.input_scale", torch.tensor([0.0]))            # nvfp4_linear returns -1 -> warn + fall back
    weights.linear_proj(ws, x, *names, 2, 4, 32, out=x)
    assert calls == ["nvfp4", "fp4"]

    calls.clear()
    weights.linear_proj(_fake_store(bf16=True), x, *names, 2, 4, 32)
    assert calls == ["bf16"]


def test_pair_fusion_rules(monkeypatch):
    calls = []
    monkeypatch.setattr(ops, "fp4_linear_fused", lambda mode, *a, **k: calls.append(mode) or "fused")
    x = torch.zeros((2, 32), dtype=torch.bfloat16)
    monkeypatch.delenv("GLMASR_USE_CUTLASS_NVFP4", raising=False)
    assert weights.linear_proj_pair_same_input(_fake_store(), x, "gate", "up", 2, 4, 32) == "fused"
    assert calls == [ops.MODE_W4A16]
    # the reference refuses to fuse when either member has a pre_quant_scale (decoder.cu:961-963)
    assert weights.linear_proj_pair_same_input(_fake_store(pre=True), x, "gate", "up", 2, 4, 32) is None
    monkeypatch.setenv("GLMASR_USE_CUTLASS_NVFP4", "1")
    calls.clear()
    weights.linear_proj_pair_same_input(_fake_store(), x, "gate", "up", 2, 4, 32)
    assert calls == [ops.MODE_W4A4]


def test_triple_bf16_fusion_rules(monkeypatch):
    """reference decoder.cu:980-1013: only three bf16 weights fuse; the weights are laid end to end."""
    seen = {}
    monkeypatch.setattr(ops, "bf16_linear", lambda x, w, *a, **k: seen.setdefault("w", w) is None or "fused")
    x = torch.zeros((2, 32), dtype=torch.bfloat16)
    st = weights.WeightStore()
    for i, (n, rows) in enumerate((("q", 8), ("k", 4), ("v", 4))):
        st.add(f"{n}.weight", torch.full((rows, 32), float(i), dtype=torch.bfloat16))
    assert weights.linear_proj_triple_same_input_bf16(st, x, "q.weight", "k.weight", "v.weight", 2, 8, 4, 32) == "fused"
    assert seen["w"].shape == (16, 32) and seen["w"][8, 0] == 1 and seen["w"][12, 0] == 2
    # any FP4 member: no fusion here (the FP4 fusion is fp4_linear_fused)
    mixed = weights.WeightStore()
    mixed.add("q.weight", torch.zeros((8, 16), dtype=torch.uint8))
    mixed.add("k.weight", torch.zeros((4, 32), dtype=torch.bfloat16))
    mixed.add("v.weight", torch.zeros((4, 32), dtype=torch.bfloat16))
    assert weights.linear_proj_triple_same_input_bf16(mixed, x, "q.weight", "k.weight", "v.weight", 2, 8, 4, 32) is None


def test_compare_nvfp4_once_runs_once_and_reports(monkeypatch, capsys):
    """reference decoder.cu:196-275: gated by GLMASR_NVFP4_COMPARE_ONCE=1, once per process, reference's line format."""
    native = torch.tensor([[1.0, 2.0], [3.0, 4.5]], dtype=torch.bfloat16)
    fallback = torch.tensor([[1.0, 2.0], [3.0, 4.0]], dtype=torch.bfloat16)
    monkeypatch.setattr(ops, "nvfp4_linear", lambda out, *a, **k: out.copy_(native) is None or 0)
    monkeypatch.setattr(ops, "fp4_linear", lambda *a, **k: fallback)
    monkeypatch.setattr(weights, "_compare_done", False)
    x = torch.zeros((2, 16), dtype=torch.bfloat16)
    args = (x, None, None, 1.0, 1.0, None, 2, 2, 16, "layer0.q")
    monkeypatch.delenv("GLMASR_NVFP4_COMPARE_ONCE", raising=False)
    assert weights.compare_nvfp4_once(*args) is None                      # not asked for
    monkeypatch.setenv("GLMASR_NVFP4_COMPARE_ONCE", "1")
    out = torch.zeros((2, 2), dtype=torch.bfloat16)
    st = weights.compare_nvfp4_once(*args, out=out)
    assert st["max_abs"] == 0.5 and st["idx"] == 3 and st["native"] == 4.5 and st["fallback"] == 4.0
    assert abs(st["mean_abs"] - 0.125) < 1e-9 and torch.equal(out, native)
    assert "NVFP4_COMPARE layer0.q M=2 N=2 K=16 max_abs=0.500000 mean_abs=0.125000 idx=3" in capsys.readouterr().err
    assert weights.compare_nvfp4_once(*args) is None                      # only once per process


def test_ops_reject_cpu_tensors():
    with pytest.raises(ValueError):
        ops.fp4_dequant_to_bf16(torch.zeros((2, 8), dtype=torch.uint8), None, 1.0)
