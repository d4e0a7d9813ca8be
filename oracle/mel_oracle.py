"""CPU restatement of the reference's log-mel front end (Infer-engine/cuda/mel.cu:111-294), numpy float64.
TEST INFRASTRUCTURE ONLY.

Per window of 16 kHz PCM (mel.cu:253-294):
  n_frames = clamp(ceil(num_samples / 160), 1, 3000)                                   (:261-263)
  frame f, tap t in [0, 400): sample index f*160 + t - 200, zero outside the signal,
      times the periodic Hann window 0.5 (1 - cos(2 pi t / 400))                        (:111-126)
  400-point real DFT, bins 0..200 (cuFFT R2C)                                           (:279)
  p[m] = sum_k |X[k]|^2 filt[k, m] with the filterbank given TRANSPOSED as [201, 128]   (:132-153)
  v = log10(p + 1e-10), stored mel-major [128, n_frames]                                (:152)
  v = max(v, vmax - 8);  v = (v + 4) / 4;  bf16                                         (:217-233)

vmax is meant to be the maximum of v over the whole window.  The reference computes it in two passes, and its
second pass (final_max_kernel, :195-206, launched with 256 threads) reduces within each warp but lets thread 0
write, so only warp 0's share reaches the result: the block maxima with index i, i % 256 < 32.  With one block
maximum per 256 consecutive values of the mel-major array (block_max_kernel, :159-190) that is the maximum over
the array elements whose index j satisfies (j // 256) % 256 < 32 -- one eighth of the data.  `vmax_mode`
selects which of the two is restated: "intended" (the whole window; what this library computes) or "reference"
(the literal behaviour, used only to pin this oracle against the reference kernel).
"""
from __future__ import annotations

import numpy as np

N_FFT, HOP, N_MELS, MAX_FRAMES, N_BINS = 400, 160, 128, 3000, 201


def slaney_mel_filterbank(sr=16000, n_fft=N_FFT, n_mels=N_MELS) -> np.ndarray:
    """A Slaney-style mel filterbank (linear below 1 kHz, logarithmic above, area-normalised triangles) as the
    front end takes it: float32 [201, 128], i.e. transposed.  Stands in for the filter file the engine loads
    (Infer-engine/src/main.c:271-309), which is not part of the reference tree."""
    def hz_to_mel(f):
        f = np.asarray(f, np.float64)
        lin = f / (200.0 / 3.0)
        log = 15.0 + np.log(np.maximum(f, 1e-12) / 1000.0) / (np.log(6.4) / 27.0)
        return np.where(f >= 1000.0, log, lin)

    def mel_to_hz(m):
        m = np.asarray(m, np.float64)
        lin = m * (200.0 / 3.0)
        log = 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0))
        return np.where(m >= 15.0, log, lin)

    fft_freqs = np.linspace(0.0, sr / 2.0, n_fft // 2 + 1)
    mel_pts = mel_to_hz(np.linspace(hz_to_mel(0.0), hz_to_mel(sr / 2.0), n_mels + 2))
    fdiff = np.diff(mel_pts)
    ramps = mel_pts[:, None] - fft_freqs[None, :]
    lower = -ramps[:-2] / fdiff[:-1, None]
    upper = ramps[2:] / fdiff[1:, None]
    w = np.maximum(0.0, np.minimum(lower, upper))
    w *= (2.0 / (mel_pts[2:n_mels + 2] - mel_pts[:n_mels]))[:, None]
    return np.ascontiguousarray(w.T.astype(np.float32))          # [201, 128]


def num_frames(num_samples: int) -> int:
    return min(max((num_samples + HOP - 1) // HOP, 1), MAX_FRAMES)


def log_mel_f64(pcm: np.ndarray, filters_t: np.ndarray) -> np.ndarray:
    """log10(mel power + 1e-10) before the clamp, float64 [128, n_frames]."""
    pcm = np.asarray(pcm, np.float64)
    n = num_frames(len(pcm))
    t = np.arange(N_FFT)
    win = 0.5 * (1.0 - np.cos(2.0 * np.pi * t / N_FFT))
    idx = np.arange(n)[:, None] * HOP + t[None, :] - N_FFT // 2
    ok = (idx >= 0) & (idx < len(pcm))
    frames = np.where(ok, pcm[np.clip(idx, 0, max(len(pcm) - 1, 0))] if len(pcm) else 0.0, 0.0) * win[None, :]
    spec = np.fft.rfft(frames, axis=1)
    power = spec.real ** 2 + spec.imag ** 2                      # [n, 201]
    mel = power @ np.asarray(filters_t, np.float64)              # [n, 128]
    return np.log10(mel + 1e-10).T                                # [128, n]


def window_max(v: np.ndarray, vmax_mode: str = "intended") -> float:
    if vmax_mode == "intended":
        return float(v.max())
    assert vmax_mode == "reference"
    flat = np.ascontiguousarray(v).reshape(-1)                   # mel-major, as the kernel sees it
    n_blocks = (flat.size + 255) // 256
    if n_blocks == 1:
        return float(flat.max())
    block_max = np.array([flat[b * 256:(b + 1) * 256].max() for b in range(n_blocks)])
    seen = block_max[(np.arange(n_blocks) % 256) < 32]
    return float(seen.max())


def log_mel(pcm: np.ndarray, filters_t: np.ndarray, vmax_mode: str = "intended") -> np.ndarray:
    """float32 [128, n_frames] after the clamp and the affine map, before the bf16 rounding."""
    v = log_mel_f64(pcm, filters_t)
    v = np.maximum(v, window_max(v, vmax_mode) - 8.0)
    return ((v + 4.0) / 4.0).astype(np.float32)
