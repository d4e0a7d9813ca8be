"""Log-mel front end (mel_spectrogram, Infer-engine/cuda/mel.cu:111-294).

CPU: properties of the oracle itself (frame count rule, the window maximum the reference computes versus the
one it means).  GPU: this library against the oracle (window maximum over the whole window) and, where the
reference's own kernel is built (oracle/_ref), the oracle's literal mode against that kernel -- which pins the
oracle's DFT / filterbank / log / clamp restatement to the reference -- on seeded pink noise with random
amplitude envelopes (the stand-in for the benchmark's audio), silence, a very short clip and a ragged batch.
Tolerance: the output is a bf16 of (log10(power) + 4) / 4 computed in fp32 by a different DFT factorisation, so
values agree to one bf16 unit of their magnitude (of 2^-6 for values closer to zero than that, where a unit in
the last place says nothing); at most a few per cent of them may differ at all.  Measured on a B200: 0.007 % of
the values differ, the reference's own cuFFT-based kernel against the same oracle 0.003 %.
"""
import numpy as np
import pytest

import fp4_oracle as o
import mel_oracle as mo


def pink_noise(seed, n=480000):
    """Pink noise with a random amplitude envelope, float32 in about [-1, 1]."""
    rng = np.random.default_rng(seed)
    spec = np.fft.rfft(rng.standard_normal(n))
    f = np.arange(spec.size, dtype=np.float64)
    f[0] = 1.0
    x = np.fft.irfft(spec / np.sqrt(f), n)
    x /= np.abs(x).max()
    knots = rng.uniform(0.05, 1.0, 16)
    env = np.interp(np.linspace(0, 15, n), np.arange(16), knots)
    return (x * env).astype(np.float32)


def test_oracle_frame_count_and_filterbank():
    assert [mo.num_frames(n) for n in (0, 1, 160, 161, 479999, 480000, 10 ** 7)] == [1, 1, 1, 2, 3000, 3000, 3000]
    f = mo.slaney_mel_filterbank()
    assert f.shape == (201, 128) and f.dtype == np.float32 and (f >= 0).all()
    assert ((f > 0).sum(0) >= 1).all()                      # every mel bin sees at least one DFT bin
    centres = (f * np.arange(201)[:, None]).sum(0) / f.sum(0)
    assert (np.diff(centres) >= 0).all() and centres[-1] > 190     # triangles march up the spectrum (the lowest are
                                                                  # narrower than a DFT bin and share one)


def test_oracle_reference_maximum_sees_one_eighth_of_the_window():
    """final_max_kernel (mel.cu:195-206) lets warp 0's share through: block maxima i with i % 256 < 32."""
    v = np.full((128, 3000), -3.0)
    v[5, 100] = 2.0            # flat index 15100 -> block 58, 58 % 256 >= 32: the reference never sees it
    assert mo.window_max(v, "intended") == 2.0
    assert mo.window_max(v, "reference") == -3.0
    v[0, 10] = 1.0             # block 0 is seen
    assert mo.window_max(v, "reference") == 1.0
    small = np.arange(200.0).reshape(2, 100)                # a single block: both agree
    assert mo.window_max(small, "reference") == mo.window_max(small, "intended") == 199.0


def _check(got_bits, want_f32, what):
    from gpu_util import bf16_unit_excess
    excess, differ = bf16_unit_excess(got_bits, o.f32_to_bf16_bits(want_f32))
    assert excess <= 1.0, (what, excess)
    assert differ <= 0.05, (what, differ)


@pytest.mark.gpu
@pytest.mark.parametrize("seed,n", [(0, 480000), (1, 479999), (2, 160 * 777 + 3), (3, 400), (4, 7)])
def test_mel_vs_oracle_and_reference_kernel(seed, n):
    import torch

    import ref_lib
    from glm_asr_stack_b200 import ops
    from gpu_util import bits_of
    filt = mo.slaney_mel_filterbank()
    pcm = pink_noise(seed)[:n] if n > 400 else pink_noise(seed, 4096)[:n]
    fd, pd = torch.from_numpy(filt).cuda(), torch.from_numpy(pcm).cuda()
    got = bits_of(ops.mel_spectrogram(pd, fd))
    assert got.shape == (128, mo.num_frames(n))
    _check(got, mo.log_mel(pcm, filt, "intended"), "library vs oracle")
    assert ops.status() == 0
    if ref_lib.available():
        ref = ref_lib.RefLib()
        if hasattr(ref.lib, "mel_spectrogram"):
            _check(bits_of(ref.mel_spectrogram(pd, fd)), mo.log_mel(pcm, filt, "reference"), "reference kernel vs literal oracle")


@pytest.mark.gpu
def test_mel_silence_and_clamp():
    import torch

    from glm_asr_stack_b200 import ops
    from gpu_util import bits_of
    filt = torch.from_numpy(mo.slaney_mel_filterbank()).cuda()
    out = ops.mel_spectrogram(torch.zeros(16000, device="cuda"), filt)
    assert out.shape == (128, 100)
    assert torch.all(out.float() == -1.5)                   # log10(1e-10) = -10 everywhere: (-10 + 4) / 4
    # one loud click: everything else sits on the floor 8 below the maximum
    pcm = np.zeros(48000, np.float32)
    pcm[24000] = 1.0
    got = o.bf16_bits_to_f32(bits_of(ops.mel_spectrogram(torch.from_numpy(pcm).cuda(), filt)))
    want = mo.log_mel(pcm, mo.slaney_mel_filterbank())
    assert np.abs(got - o.bf16_bits_to_f32(o.f32_to_bf16_bits(want))).max() <= 2.0 ** -6
    assert np.isclose(got.min(), got.max() - 2.0, atol=2.0 ** -5)          # 8 / 4


@pytest.mark.gpu
def test_mel_batched_ragged_both_layouts():
    import torch

    from glm_asr_stack_b200 import ops
    from gpu_util import bits_of
    filt_np = mo.slaney_mel_filterbank()
    filt = torch.from_numpy(filt_np).cuda()
    lens = [480000, 1, 160 * 500, 0, 333333]
    pcm = np.zeros((len(lens), 480000), np.float32)
    for i, n in enumerate(lens):
        pcm[i, :n] = pink_noise(10 + i)[:n]
    pd = torch.from_numpy(pcm).cuda()
    for time_major in (False, True):
        out, frames = ops.mel_spectrogram_batched(pd, lens, filt, time_major=time_major)
        assert frames == [mo.num_frames(n) for n in lens]
        for i, n in enumerate(lens):
            f = frames[i]
            got = bits_of(out[i, :128 * f]).reshape((f, 128) if time_major else (128, f))
            want = mo.log_mel(pcm[i, :n], filt_np)
            _check(got.T if time_major else got, want, f"window {i} time_major={time_major}")
            single = bits_of(ops.mel_spectrogram(pd[i, :n].contiguous() if n else torch.zeros(0, device="cuda"), filt))
            assert np.array_equal(got.T if time_major else got, single)
    assert ops.status() == 0
