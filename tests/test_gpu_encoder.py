"""GPU parity of the audio encoder path (LayerNorm, GELU, partial rotary embedding, convolution front end,
head_dim-64 non-causal attention, encoder_forward_packed, the batched audio path) against the CPU oracle and,
where oracle/_ref is built, against the reference's own kernels on the same inputs.

Tolerances: residual_add_bias and the transposition are bit-exact; LayerNorm, GELU and the rotary embedding are
float32 formulas whose last bit depends on the math library (numpy versus CUDA): at most one bf16 unit, nearly all
values equal; GEMM-based stages (convolutions, linear + GELU, attention, the whole encoder) are bf16 outputs of
fp32 accumulations in an unspecified order: relative error <= 1e-2 (the path's stated bar), in practice <= 4e-3.
"""
import numpy as np
import pytest
import torch

import encoder_oracle as eo
import fp4_oracle as o
import ref_lib
from gpu_util import REL_TOL_TIGHT, REL_TOL_VS_ORACLE, bf16_unit_excess, bits_of, to_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from glm_asr_stack_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def ref():
    if not ref_lib.available():
        return None
    r = ref_lib.RefLib()
    return r if r.has_encoder() else None


def rb(rng, shape, scale=1.0, mean=0.0):
    return o.f32_to_bf16_bits((rng.standard_normal(shape) * scale + mean).astype(np.float32))


def near(got, want, frac_equal=0.99):
    """Within one bf16 step at the value's magnitude, and nearly all values bit-equal."""
    excess, differ = bf16_unit_excess(got, want)
    return excess <= 1.0 and differ <= 1.0 - frac_equal


@pytest.mark.parametrize("rows,dim", [(1, 1280), (37, 1280), (300, 256), (5, 2560), (3, 96)])
def test_layernorm(ops, ref, rows, dim):
    rng = np.random.default_rng(rows + dim)
    x, w, b = rb(rng, (rows, dim), 2.0, 0.3), rb(rng, (dim,), 0.1, 1.0), rb(rng, (dim,), 0.1)
    got = bits_of(ops.layernorm(to_dev_bf16(x), to_dev_bf16(w), to_dev_bf16(b)))
    assert near(got, eo.layernorm(x, w, b))
    xd = to_dev_bf16(x)
    ops.layernorm(xd, to_dev_bf16(w), to_dev_bf16(b), out=xd)               # in place, as the final norm runs
    assert np.array_equal(bits_of(xd), got)
    if ref is not None:
        assert np.array_equal(got, bits_of(ref.layernorm(to_dev_bf16(x), to_dev_bf16(w), to_dev_bf16(b))))


def test_gelu_and_residual_add_bias(ops, ref):
    rng = np.random.default_rng(3)
    x = rb(rng, (333, 77), 2.0)
    got = bits_of(ops.gelu_inplace(to_dev_bf16(x)))
    assert near(got, eo.gelu_inplace(x))
    if ref is not None:
        assert near(got, bits_of(ref.gelu_inplace(to_dev_bf16(x))), 0.999)
    a, b, bias = rb(rng, (50, 1280)), rb(rng, (50, 1280)), rb(rng, (1280,), 0.1)
    assert np.array_equal(bits_of(ops.residual_add_bias(to_dev_bf16(a), to_dev_bf16(b), to_dev_bf16(bias))),
                          eo.residual_add_bias(a, b, bias))
    assert np.array_equal(bits_of(ops.residual_add_bias(to_dev_bf16(a), to_dev_bf16(b), None)), eo.residual_add_bias(a, b))
    t = rb(rng, (45, 70))
    assert np.array_equal(bits_of(ops.transpose_2d(to_dev_bf16(t))), t.T)


def test_rope_encoder(ops):
    rng = np.random.default_rng(4)
    n, heads, hd = 1500, 20, 64
    q, k = rb(rng, (n, heads * hd)), rb(rng, (n, heads * hd))
    qd, kd = to_dev_bf16(q), to_dev_bf16(k)
    ops.rope_encoder(qd, kd, heads, hd)
    pos = np.arange(n)
    assert near(bits_of(qd), eo.rope(q, pos, heads, hd), 0.98) and near(bits_of(kd), eo.rope(k, pos, heads, hd), 0.98)
    got = bits_of(qd).reshape(n, heads, hd)
    assert np.array_equal(got[:, :, 32:], q.reshape(n, heads, hd)[:, :, 32:])       # dims 32..63 untouched
    assert np.array_equal(got[0], q.reshape(n, heads, hd)[0])                       # position 0 is the identity


@pytest.mark.parametrize("in_ch,out_ch,ln,stride", [(128, 256, 300, 1), (256, 256, 301, 2), (128, 1280, 3000, 1)])
def test_conv1d_forward(ops, ref, in_ch, out_ch, ln, stride):
    rng = np.random.default_rng(in_ch + ln)
    x, w, b = rb(rng, (in_ch, ln)), rb(rng, (out_ch, in_ch, 3), 0.05), rb(rng, (out_ch,), 0.1)
    got = bits_of(ops.conv1d_forward(to_dev_bf16(x), to_dev_bf16(w), to_dev_bf16(b), stride, 1))
    want = eo.conv1d_forward(x, w, b, stride, 1)
    assert got.shape == want.shape
    assert o.rel_err(got, want) <= REL_TOL_VS_ORACLE
    if ref is not None:
        r = bits_of(ref.conv1d_forward(to_dev_bf16(x), to_dev_bf16(w), to_dev_bf16(b), stride, 1))
        assert o.rel_err(r, want) <= REL_TOL_TIGHT                 # pins the oracle's per-tap rounding to the reference
        assert o.rel_err(got, r) <= REL_TOL_VS_ORACLE
    assert ops.status() == 0


def test_bf16_linear_gelu(ops):
    rng = np.random.default_rng(6)
    M, N, K = 375, 4096, 5120
    x, w, b = rb(rng, (M, K)), rb(rng, (N, K), 0.02), rb(rng, (N,), 0.1)
    got = bits_of(ops.bf16_linear_gelu(to_dev_bf16(x), to_dev_bf16(w), to_dev_bf16(b)))
    assert o.rel_err(got, eo.bf16_linear_gelu(x, w, b)) <= REL_TOL_TIGHT
    assert ops.status() == 0


@pytest.mark.parametrize("lens", [[1500], [70, 1, 33, 128, 64], [130, 0, 257]])
def test_attention_head_dim_64_non_causal(ops, lens):
    from glm_asr_stack_b200 import engine
    rng = np.random.default_rng(len(lens))
    heads, hd = 20, 64
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    T, H = int(offs[-1]), heads * hd
    qkv = rb(rng, (T, 3 * H))
    buf = to_dev_bf16(qkv)
    got = bits_of(engine.prefill_attention(buf[:, :H], buf[:, H:2 * H], buf[:, 2 * H:], torch.from_numpy(offs).cuda(),
                                           max(lens), heads, heads, hd, False))
    want = eo.attention(qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:], offs[:-1], lens, heads, hd)
    for off, ln in zip(offs[:-1], lens):
        if ln:
            assert o.rel_err(got[off:off + ln], want[off:off + ln]) <= REL_TOL_TIGHT
    assert ops.status() == 0


def build_tower(rng, hidden, heads, ffn, layers, mels=128, proj_mid=512, dec_hidden=256):
    """A small random audio tower as a WeightStore plus the oracle's view of it."""
    from glm_asr_stack_b200 import engine
    ws = engine.WeightStore()
    cfg = engine.model_config(dec_hidden, 1, 2, 1, 128, 512, 1000)
    engine.encoder_config(cfg, hidden, layers, heads, 64, ffn, mels, 3000, proj_mid)
    np_w = {}

    def add(name, shape, std, mean=0.0):
        bits = rb(rng, shape, std, mean)
        np_w[name] = bits
        ws.add(name, to_dev_bf16(bits))

    add("audio_tower.conv1.weight", (hidden, mels, 3), 0.05)
    add("audio_tower.conv1.bias", (hidden,), 0.05)
    add("audio_tower.conv2.weight", (hidden, hidden, 3), 0.03)
    add("audio_tower.conv2.bias", (hidden,), 0.05)
    lyr = []
    for l in range(layers):
        p = f"audio_tower.layers.{l}."
        L = {}
        for key, nm, shape, std, mean in [
                ("ln1_w", "input_layernorm.weight", (hidden,), 0.1, 1.0), ("ln1_b", "input_layernorm.bias", (hidden,), 0.05, 0.0),
                ("q_w", "self_attn.q_proj.weight", (hidden, hidden), 0.04, 0.0), ("q_b", "self_attn.q_proj.bias", (hidden,), 0.05, 0.0),
                ("k_w", "self_attn.k_proj.weight", (hidden, hidden), 0.04, 0.0),
                ("v_w", "self_attn.v_proj.weight", (hidden, hidden), 0.04, 0.0), ("v_b", "self_attn.v_proj.bias", (hidden,), 0.05, 0.0),
                ("o_w", "self_attn.o_proj.weight", (hidden, hidden), 0.04, 0.0), ("o_b", "self_attn.o_proj.bias", (hidden,), 0.05, 0.0),
                ("ln2_w", "post_attention_layernorm.weight", (hidden,), 0.1, 1.0),
                ("ln2_b", "post_attention_layernorm.bias", (hidden,), 0.05, 0.0),
                ("fc1_w", "mlp.fc1.weight", (ffn, hidden), 0.04, 0.0), ("fc1_b", "mlp.fc1.bias", (ffn,), 0.05, 0.0),
                ("fc2_w", "mlp.fc2.weight", (hidden, ffn), 0.04, 0.0), ("fc2_b", "mlp.fc2.bias", (hidden,), 0.05, 0.0)]:
            add(p + nm, shape, std, mean)
            L[key] = np_w[p + nm]
        lyr.append(L)
    add("audio_tower.norm.weight", (hidden,), 0.1, 1.0)
    add("audio_tower.norm.bias", (hidden,), 0.05)
    add("multi_modal_projector.linear_1.weight", (proj_mid, 4 * hidden), 0.03)
    add("multi_modal_projector.linear_1.bias", (proj_mid,), 0.05)
    add("multi_modal_projector.linear_2.weight", (dec_hidden, proj_mid), 0.03)
    add("multi_modal_projector.linear_2.bias", (dec_hidden,), 0.05)
    return ws, cfg, lyr, np_w


def test_encoder_forward_packed_small_model(ops, ref):
    """Three sequences with a gap of foreign rows between them: rows of no sequence go through the row-wise
    operations but neither give nor receive attention."""
    rng = np.random.default_rng(40)
    hidden, heads, ffn, layers = 256, 4, 512, 2
    ws, cfg, lyr, np_w = build_tower(rng, hidden, heads, ffn, layers)
    lens, offs = [70, 33, 128], [0, 75, 110]
    rows = 240
    h0 = rb(rng, (rows, hidden))
    got = bits_of(ops.encoder_forward_packed(ws, cfg, to_dev_bf16(h0), lens, offs))
    assert ops.status() == 0
    want = eo.encoder_forward_packed(h0, lyr, np_w["audio_tower.norm.weight"], np_w["audio_tower.norm.bias"], offs, lens, heads, 64)
    inside = np.zeros(rows, bool)
    for off, ln in zip(offs, lens):
        inside[off:off + ln] = True
    err = o.rel_err(got[inside], want[inside])
    assert err <= REL_TOL_VS_ORACLE and o.cosine(got[inside], want[inside]) >= 0.999, err
    if ref is not None:
        r = bits_of(ref.encoder_forward_packed(ws, cfg, to_dev_bf16(h0), lens, offs))
        assert o.rel_err(r[inside], want[inside]) <= REL_TOL_VS_ORACLE        # pins the oracle's layer sequence to the reference
        assert o.rel_err(got[inside], r[inside]) <= REL_TOL_VS_ORACLE


def test_encoder_real_width_two_layers(ops, ref):
    """d = 1280, 20 heads x 64, FFN 5120, one window of 1500 frames and a short one: two layers under the oracle."""
    rng = np.random.default_rng(41)
    hidden, heads, ffn, layers = 1280, 20, 5120, 2
    ws, cfg, lyr, np_w = build_tower(rng, hidden, heads, ffn, layers)
    lens, offs = [1500, 333], [0, 1500]
    h0 = rb(rng, (1833, hidden))
    got = bits_of(ops.encoder_forward_packed(ws, cfg, to_dev_bf16(h0), lens, offs))
    assert ops.status() == 0
    want = eo.encoder_forward_packed(h0, lyr, np_w["audio_tower.norm.weight"], np_w["audio_tower.norm.bias"], offs, lens, heads, 64)
    err = o.rel_err(got, want)
    assert err <= REL_TOL_VS_ORACLE and o.cosine(got, want) >= 0.999, err
    if ref is not None:
        r = bits_of(ref.encoder_forward_packed(ws, cfg, to_dev_bf16(h0), lens, offs))
        assert o.rel_err(got, r) <= REL_TOL_VS_ORACLE and o.rel_err(r, want) <= REL_TOL_VS_ORACLE


def test_audio_encode_batched_small_model(ops):
    """Log-mel features (time-major) -> convolutions -> encoder -> projector for a ragged batch, window by window
    against the oracle's single-window chain."""
    rng = np.random.default_rng(42)
    hidden, heads, ffn, layers = 256, 4, 512, 2
    ws, cfg, lyr, np_w = build_tower(rng, hidden, heads, ffn, layers)
    frames = [400, 37, 3000, 1001]
    W = len(frames)
    mel = np.zeros((W, 3000, 128), np.uint16)
    for i, n in enumerate(frames):
        mel[i, :n] = o.f32_to_bf16_bits(rng.uniform(-1.5, 1.5, (n, 128)).astype(np.float32))
    out, tokens = ops.audio_encode_batched(ws, cfg, to_dev_bf16(mel.reshape(W, -1)), frames)
    assert ops.status() == 0
    assert tokens == [((n + 1) // 2) // 4 for n in frames]
    for i, n in enumerate(frames):
        want = eo.audio_encode(np.ascontiguousarray(mel[i, :n].T), (np_w["audio_tower.conv1.weight"], np_w["audio_tower.conv1.bias"]),
                               (np_w["audio_tower.conv2.weight"], np_w["audio_tower.conv2.bias"]), lyr,
                               np_w["audio_tower.norm.weight"], np_w["audio_tower.norm.bias"],
                               (np_w["multi_modal_projector.linear_1.weight"], np_w["multi_modal_projector.linear_1.bias"]),
                               (np_w["multi_modal_projector.linear_2.weight"], np_w["multi_modal_projector.linear_2.bias"]), heads, 64)
        got = bits_of(out[i, :tokens[i]])
        assert got.shape == want.shape
        err = o.rel_err(got, want)
        assert err <= REL_TOL_VS_ORACLE and o.cosine(got, want) >= 0.999, (i, err)
