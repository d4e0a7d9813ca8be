"""The co-resident layer-tail kernel of the decode step (csrc/decode_tail.cu) against the library's regular GEMM
kernels on the same quantised activation: every GEMM phase kind (plain store over three weight tensors, in-place
residual, SiLU-gate with the quantising epilogue) must give the same BYTES, at the toy and at the real decoder
shapes, for one and for two row tiles.  The whole step with and without the kernel is compared in
test_decode_step_same_bytes_with_and_without_the_layer_tail.
"""
import os
import pickle
import subprocess
import sys

import numpy as np
import pytest

import fp4_oracle as o

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _weight(N, K, seed):
    import torch

    from glm_asr_stack_b200 import ops
    pw, sw, g = o.seeded_weight(N, K, seed)
    return ops.Fp4Tensor(torch.from_numpy(pw).cuda(), torch.from_numpy(sw).cuda(), g)


def _quantised_rows(M, K, seed, input_scale):
    import torch

    from glm_asr_stack_b200 import ops
    from gpu_util import to_dev_bf16
    x = to_dev_bf16(o.seeded_activation(M, K, seed))
    w = torch.ones(K, dtype=torch.bfloat16, device="cuda")
    return ops.rmsnorm_quant(x, w, 1e-5, input_scale)


@pytest.mark.parametrize("M", [5, 128, 200, 256])
@pytest.mark.parametrize("shape", ["toy", "real"])
def test_resident_gemm_phases_equal_the_regular_kernels(M, shape):
    import torch

    from glm_asr_stack_b200 import ops
    from gpu_util import bits_of, to_dev_bf16
    H, F, KV = (256, 512, 128) if shape == "toy" else (2048, 6144, 512)
    isc = 0.004
    xq, xsf = _quantised_rows(M, H, 3, isc)
    # q | k | v: three weight tensors, plain store
    qkv = [_weight(H, H, 10), _weight(KV, H, 11), _weight(KV, H, 12)]
    a = ops.fp4_linear_quantized(xq, xsf, qkv, isc)
    b = ops.fp4_linear_quantized(xq, xsf, qkv, isc, resident=True)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert np.array_equal(bits_of(a), bits_of(b)), "q|k|v"
    # o-sized projection with the residual added in place
    wo = [_weight(H, H, 13)]
    res = o.seeded_activation(M, H, 5)
    a, b = to_dev_bf16(res), to_dev_bf16(res)
    ops.fp4_linear_quantized(xq, xsf, wo, isc, epilogue=ops.EPI_RESIDUAL, out=a)
    ops.fp4_linear_quantized(xq, xsf, wo, isc, epilogue=ops.EPI_RESIDUAL, out=b, resident=True)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(a), bits_of(b)), "o + residual"
    # gate | up with SiLU-gate, quantised for the down projection, then down (K = F) with the residual
    gu = [_weight(F, H, 14), _weight(F, H, 15)]
    isc_down = 0.002
    qa, sa = ops.fp4_linear_quantized(xq, xsf, gu, isc, epilogue=ops.EPI_SILU_GATE, q_out_input_scale=isc_down)
    qb, sb = ops.fp4_linear_quantized(xq, xsf, gu, isc, epilogue=ops.EPI_SILU_GATE, q_out_input_scale=isc_down, resident=True)
    torch.cuda.synchronize()
    assert torch.equal(qa[:M], qb[:M]), "SiLU-gate codes"
    # scales of the rows that exist (the tiled layout holds 128-row tiles; rows past M are never written)
    sa_t = sa.view(-1, F // 64, 32, 4, 4).cpu().numpy()
    sb_t = sb.view(-1, F // 64, 32, 4, 4).cpu().numpy()
    for r in range(M):
        assert np.array_equal(sa_t[r >> 7, :, r & 31, (r & 127) >> 5], sb_t[r >> 7, :, r & 31, (r & 127) >> 5]), ("SiLU-gate scales", r)
    wd = [_weight(H, F, 16)]
    a, b = to_dev_bf16(res), to_dev_bf16(res)
    ops.fp4_linear_quantized(qa, sa, wd, isc_down, epilogue=ops.EPI_RESIDUAL, out=a, M=M)
    ops.fp4_linear_quantized(qa, sa, wd, isc_down, epilogue=ops.EPI_RESIDUAL, out=b, resident=True, M=M)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert np.array_equal(bits_of(a), bits_of(b)), "down + residual"


def _sf_rows(sf, K, M):
    """The scale bytes of rows < M out of a 128x4-tiled scale buffer: [M, K/64, 4]."""
    t = sf.view(-1, K // 64, 32, 4, 4).cpu().numpy()
    return np.stack([t[r >> 7, :, r & 31, (r & 127) >> 5] for r in range(M)])


@pytest.mark.parametrize("M", [5, 256])
@pytest.mark.parametrize("shape", ["toy", "real"])
def test_layer_tail_phase_by_phase(M, shape):
    """glmasr_decode_layer_tail stopped after 1..6 phases against the same operations run one launch at a time
    (regular GEMM kernels, glmasr_rmsnorm_quant): every hand-over buffer and the hidden state equal byte for byte."""
    import torch

    from glm_asr_stack_b200 import ops
    from gpu_util import bits_of, to_dev_bf16
    H, F, KV = (256, 512, 128) if shape == "toy" else (2048, 6144, 512)
    in_o, in_gu, in_down, in_qkv = 0.004, 0.003, 0.002, 0.0035
    w = {n: _weight(N, K, 20 + i) for i, (n, N, K) in enumerate(
        [("q", H, H), ("k", KV, H), ("v", KV, H), ("o", H, H), ("gate", F, H), ("up", F, H), ("down", H, F)])}
    lw = ops.make_layer_weights(w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"], H, F)
    lw.in_qkv, lw.in_o, lw.in_gate_up, lw.in_down = in_qkv, in_o, in_gu, in_down
    rng = np.random.default_rng(3)
    norm2 = to_dev_bf16(o.f32_to_bf16_bits((1.0 + 0.2 * rng.standard_normal(H)).astype(np.float32)))
    norm1 = to_dev_bf16(o.f32_to_bf16_bits((1.0 + 0.2 * rng.standard_normal(H)).astype(np.float32)))
    attn_q, attn_sf = _quantised_rows(M, H, 7, in_o)
    hid0 = o.seeded_activation(M, H, 9)
    # one launch per operation
    hid = to_dev_bf16(hid0)
    ops.fp4_linear_quantized(attn_q, attn_sf, [w["o"]], in_o, epilogue=ops.EPI_RESIDUAL, out=hid)
    want_hid1 = bits_of(hid).copy()
    nq, nsf = ops.rmsnorm_quant(hid, norm2, 1e-5, in_gu)
    gq, gsf = ops.fp4_linear_quantized(nq, nsf, [w["gate"], w["up"]], in_gu, epilogue=ops.EPI_SILU_GATE, q_out_input_scale=in_down)
    ops.fp4_linear_quantized(gq, gsf, [w["down"]], in_down, epilogue=ops.EPI_RESIDUAL, out=hid, M=M)
    want_hid2 = bits_of(hid).copy()
    nq2, nsf2 = ops.rmsnorm_quant(hid, norm1, 1e-5, in_qkv)
    want_qkv = bits_of(ops.fp4_linear_quantized(nq2, nsf2, [w["q"], w["k"], w["v"]], in_qkv))
    torch.cuda.synchronize()
    for phases in (1, 2, 3, 4, 5, 6):
        h = to_dev_bf16(hid0)
        qkv, tq, tsf, aq, asf = ops.decode_layer_tail(h, attn_q, attn_sf, lw, norm2, lw, norm1, max_phases=phases)
        torch.cuda.synchronize()
        assert ops.status() == 0
        assert np.array_equal(bits_of(h), want_hid1 if phases < 4 else want_hid2), ("hidden", phases)
        if phases in (2, 3, 4):
            assert torch.equal(tq, nq) and np.array_equal(_sf_rows(tsf, H, M), _sf_rows(nsf, H, M)), ("norm", phases)
        if phases >= 3:
            assert torch.equal(aq, gq) and np.array_equal(_sf_rows(asf, F, M), _sf_rows(gsf, F, M)), ("SiLU-gate", phases)
        if phases >= 5:
            assert torch.equal(tq, nq2) and np.array_equal(_sf_rows(tsf, H, M), _sf_rows(nsf2, H, M)), ("next norm", phases)
        if phases == 6:
            assert np.array_equal(bits_of(qkv), want_qkv), "next q|k|v"
    # the last layer's form: no following layer
    h = to_dev_bf16(hid0)
    ops.decode_layer_tail(h, attn_q, attn_sf, lw, norm2)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(h), want_hid2)


def test_resident_gemm_rejects_what_it_does_not_cover():
    import torch

    from glm_asr_stack_b200 import ops
    xq, xsf = _quantised_rows(300, 256, 3, 0.004)
    with pytest.raises(ValueError):                       # more than two row tiles
        ops.fp4_linear_quantized(xq, xsf, [_weight(256, 256, 1)], 0.004, resident=True)
    xq, xsf = _quantised_rows(8, 256, 3, 0.004)
    with pytest.raises(ValueError):                       # N not a multiple of 32
        ops.fp4_linear_quantized(xq, xsf, [_weight(144, 256, 1)], 0.004, resident=True)
    torch.cuda.synchronize()
    assert ops.status() == 0


def _decode_step_child(out_path, nseq):
    import ctypes

    import torch

    import test_gpu_decoder as t
    from glm_asr_stack_b200 import engine, ops
    from gpu_util import bits_of, to_dev_bf16
    rng = np.random.default_rng(11)
    ws, cfg, layers, fn, (H, F, QH, KVH, HD, L) = t.build_toy_model(rng, 0, "plain")
    bs, n = 16, nseq
    cached = np.array(([0, 15, 16, 37, 200] * 60)[:n], np.int32)
    num_blocks, max_blocks = 64 * 64, 16
    pool = engine.KVPool(num_blocks, bs, L, KVH, HD, max_seqs=n + 3, max_blocks_per_seq=max_blocks)
    perm = rng.permutation(num_blocks).tolist()
    tables = [[perm.pop() for _ in range((int(c) + 2 + bs - 1) // bs)] for c in cached]     # room for two new tokens
    bts = engine.BlockTables(pool, tables)
    pool.k.copy_(to_dev_bf16(t.rnd_bits(rng, tuple(pool.k.shape))))
    pool.v.copy_(to_dev_bf16(t.rnd_bits(rng, tuple(pool.v.shape))))
    hd = to_dev_bf16(t.rnd_bits(rng, (n, H)))
    d_lens = torch.from_numpy(cached.copy()).cuda()
    h_lens = (ctypes.c_int * n)(*cached.tolist())
    for _ in range(2):                                    # two steps: the second runs on the first one's cache
        engine.decode_step(ws, cfg, pool, bts, hd, d_lens, h_lens)
    torch.cuda.synchronize()
    assert ops.status() == 0
    with open(out_path, "wb") as f:
        pickle.dump({"hid": bits_of(hd), "k": bits_of(pool.k), "v": bits_of(pool.v), "launches": ops.launch_count()}, f)


@pytest.mark.parametrize("nseq", [5, 200])
def test_decode_step_same_bytes_with_and_without_the_layer_tail(tmp_path, nseq):
    """Two decode steps of the toy decoder with every projection in W4A4, once with one launch per operation
    (GLMASR_DECODE_TAIL=0) and once with the layer tail as one co-resident launch: hidden state and KV cache equal."""
    res = {}
    for tail in ("0", "1"):
        env = dict(os.environ, GLMASR_USE_CUTLASS_NVFP4="1", GLMASR_NVFP4_PAIRS="1", GLMASR_DECODE_TAIL=tail)
        out = str(tmp_path / f"tail_{tail}.pkl")
        code = ("import sys; sys.path[:0]=[%r,%r,%r]; import test_gpu_decode_tail as t; t._decode_step_child(%r, %d)"
                % (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests"), out, nseq))
        r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
        with open(out, "rb") as f:
            res[tail] = pickle.load(f)
    for key in ("hid", "k", "v"):
        assert np.array_equal(res["0"][key], res["1"][key]), key
    assert res["1"]["launches"] < res["0"]["launches"]
