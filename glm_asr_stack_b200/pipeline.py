"""Host-side flow of one engine instance over a list of 30 s windows, through the library's C entry points:
log-mel -> convolution front end + encoder + projector -> prompt assembly -> batched prefill -> greedy decode.

Mirrors what the reference engine does per scheduler step (Infer-engine/src/engine.c:1408-1610 prefill batch with
audio encode and prompt embedding, :1734-1760 first token, :1945-1982 decode batch) with the scheduler's own limits:
at most GLMASR_MAX_SEQS sequences resident, at most GLMASR_MAX_BATCHED_TOKENS prompt tokens and max_seqs / 2
sequences per prefill step, never a prefill and a decode in the same step (Infer-engine/src/scheduler.c:236,
277-278, 330-336).  All windows decode the same number of new tokens (EOS is ignored), so the work is done in
waves: fill the resident set by prefill steps, decode it to the end, start the next wave.

PyTorch is used for device buffers, row gathers and copies only; every model computation is a call into
libglmasr_fp4.so.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import engine, ops
from .workloads import DecoderModel

# prompt of a transcription request (Infer-engine/src/engine.c:560-562, 633-649):
#   <|user|> \n <|begin_of_audio|> [audio x n] <|end_of_audio|> <|user|> \n [instruction] <|assistant|> \n
PROMPT_HEAD = (59253, 10, 59261)
PROMPT_TAIL = (59262, 59253, 10, 8705, 455, 1700, 8091, 283, 16926, 1636, 261, 8237, 7099, 63, 59254, 10)
SAMPLES_PER_WINDOW = 480000


def feature_frames(num_samples: int, max_frames: int = 3000) -> int:
    """Infer-engine/src/engine.c:576-581, 1093-1096."""
    return min(max((num_samples + 159) // 160, 1) if num_samples > 0 else 1, max_frames)


def padded_feature_frames(frames: int, max_frames: int = 3000) -> int:
    """Infer-engine/src/engine.c:594-607: pad the feature frames until the stride-2 convolution yields whole groups of 4."""
    p = min(max(frames, 1), max_frames)
    while p < max_frames and (((p + 1) // 2) % 4) != 0:
        p += 1
    return p


def audio_tokens(frames: int) -> int:
    """Infer-engine/src/engine.c:583-592."""
    return ((frames + 1) // 2 if frames > 0 else 1) // 4


@dataclass
class PipelineTimes:
    """Device time of the three phases (CUDA events), seconds."""
    audio: float = 0.0
    prefill: float = 0.0
    decode: float = 0.0
    events: list = field(default_factory=list)

    def mark(self, phase: str):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.events.append((phase, e))

    def finish(self):
        torch.cuda.synchronize()
        for (p0, e0), (_, e1) in zip(self.events[:-1], self.events[1:]):
            if p0 != "idle":
                setattr(self, p0, getattr(self, p0) + e0.elapsed_time(e1) * 1e-3)
        self.events.clear()


class AsrPipeline:
    def __init__(self, model: DecoderModel, mel_filters_t: torch.Tensor, max_seqs: int = 256, max_batched_tokens: int = 10000,
                 new_tokens: int = 256, block_size: int = 16, max_prompt_tokens: int = 19 + 375, device="cuda"):
        self.model, self.cfg, self.filters = model, model.cfg, mel_filters_t
        self.max_seqs, self.max_batched_tokens, self.new_tokens = max_seqs, max_batched_tokens, new_tokens
        self.device = device
        cfg = self.cfg
        blocks_per_seq = (max_prompt_tokens + new_tokens + block_size - 1) // block_size + 1
        self.pool = engine.KVPool(max_seqs * blocks_per_seq, block_size, cfg.dec_layers, cfg.dec_kv_heads, cfg.dec_head_dim,
                                  max_seqs, blocks_per_seq, device)
        perm = np.random.default_rng(7).permutation(max_seqs * blocks_per_seq).tolist()
        self.bts = engine.BlockTables(self.pool, [perm[s * blocks_per_seq:(s + 1) * blocks_per_seq] for s in range(max_seqs)])
        self.d_seq_lens = torch.zeros(max_seqs, dtype=torch.int32, device=device)
        self.h_seq_lens = (ctypes.c_int * max_seqs)()
        H = cfg.dec_hidden
        self.logits = torch.empty((max_seqs, cfg.vocab_size), dtype=torch.bfloat16, device=device)
        self.head = torch.tensor(PROMPT_HEAD, dtype=torch.int32, device=device)
        self.tail = torch.tensor(PROMPT_TAIL, dtype=torch.int32, device=device)
        self.prefill_group = max(1, min(max_batched_tokens // max_prompt_tokens, max_seqs // 2))
        self.pcm_dev = torch.zeros((self.prefill_group, SAMPLES_PER_WINDOW), dtype=torch.float32, device=device)
        self.mel = torch.zeros((self.prefill_group, 3000 * cfg.num_mel_bins), dtype=torch.bfloat16, device=device)
        self.hidden_dim = H

    # ---- one prefill step: windows -> first tokens ------------------------------------------------------
    def _lm_head(self, hidden: torch.Tensor) -> torch.Tensor:
        lm = self.model.lm_head
        logits = self.logits[:hidden.shape[0]]
        rc = ops.nvfp4_linear(logits, hidden, lm.w_packed, lm.w_scales, self.model.lm_head_input_scale, lm.w_global_scale)
        assert rc == 0
        return ops.argmax_rows(logits)

    def _prefill_group(self, pcm_host: torch.Tensor, num_samples: Sequence[int], slot0: int, times: PipelineTimes) -> torch.Tensor:
        g = len(num_samples)
        cfg = self.cfg
        times.mark("audio")
        frames = [padded_feature_frames(feature_frames(min(int(n), cfg.max_audio_frames * 160)), cfg.max_audio_frames) for n in num_samples]
        padded_samples = [f * 160 for f in frames]
        pcm = self.pcm_dev[:g]
        pcm.copy_(pcm_host, non_blocking=True)                    # pinned host -> device; samples past a clip's end are zeros
        _, got_frames = ops.mel_spectrogram_batched(pcm, padded_samples, self.filters, time_major=True, out=self.mel[:g])
        emb, tok = ops.audio_encode_batched(self.model.ws, cfg, self.mel[:g], got_frames)
        n_audio = [min(audio_tokens(feature_frames(int(n))), t) for n, t in zip(num_samples, tok)]
        # prompt: head ids, audio embeddings, tail ids (Infer-engine/src/engine.c:611-655, 1604-1640)
        lens = [len(PROMPT_HEAD) + a + len(PROMPT_TAIL) for a in n_audio]
        offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        total = int(offs[-1])
        hidden = torch.empty((total, self.hidden_dim), dtype=torch.bfloat16, device=self.device)
        head_rows = ops.embedding_lookup(self.model.embed, self.head)
        tail_rows = ops.embedding_lookup(self.model.embed, self.tail)
        for i, a in enumerate(n_audio):
            o0 = int(offs[i])
            hidden[o0:o0 + 3] = head_rows
            hidden[o0 + 3:o0 + 3 + a] = emb[i, :a]
            hidden[o0 + 3 + a:o0 + lens[i]] = tail_rows
        times.mark("prefill")
        engine.prefill_paged_batched(self.model.ws, cfg, self.pool, self.bts, hidden, lens, [int(v) for v in offs[:-1]], first=slot0)
        last = hidden[torch.as_tensor(offs[1:] - 1, device=self.device)]
        first_tokens = self._lm_head(last.contiguous())
        for i, ln in enumerate(lens):
            self.h_seq_lens[slot0 + i] = ln
        self.d_seq_lens[slot0:slot0 + g] = torch.tensor(lens, dtype=torch.int32, device=self.device)
        times.mark("idle")
        return first_tokens

    # ---- one wave -------------------------------------------------------------------------------------------
    def _wave(self, pcm_host: torch.Tensor, num_samples: Sequence[int], times: PipelineTimes) -> torch.Tensor:
        n = len(num_samples)
        tokens = torch.zeros((n, self.new_tokens), dtype=torch.int32, device=self.device)
        for s0 in range(0, n, self.prefill_group):
            s1 = min(n, s0 + self.prefill_group)
            tokens[s0:s1, 0] = self._prefill_group(pcm_host[s0:s1], num_samples[s0:s1], s0, times)
        times.mark("decode")
        d_lens = self.d_seq_lens[:n]
        cur = tokens[:, 0].contiguous()
        for step in range(1, self.new_tokens):
            hidden = ops.embedding_lookup(self.model.embed, cur)
            engine.decode_step(self.model.ws, self.cfg, self.pool, self.bts, hidden, d_lens, self.h_seq_lens)
            cur = self._lm_head(hidden)
            tokens[:, step] = cur
        times.mark("idle")
        return tokens

    def transcribe(self, pcm_host: torch.Tensor, num_samples: Optional[Sequence[int]] = None, times: Optional[PipelineTimes] = None):
        """pcm_host: float32 [windows, 480000] (pinned) on the host, zero-padded clips.  Returns int32 [windows, new_tokens]
        on the host (pinned) -- the greedy tokens of every window."""
        w = pcm_host.shape[0]
        if num_samples is None:
            num_samples = [SAMPLES_PER_WINDOW] * w
        times = times if times is not None else PipelineTimes()
        out = torch.empty((w, self.new_tokens), dtype=torch.int32).pin_memory()
        for w0 in range(0, w, self.max_seqs):
            w1 = min(w, w0 + self.max_seqs)
            out[w0:w1].copy_(self._wave(pcm_host[w0:w1], list(num_samples[w0:w1]), times), non_blocking=True)
        times.mark("idle")
        times.finish()
        return out


def synthetic_window(index: int, device="cuda") -> torch.Tensor:
    """One 30 s, 16 kHz window of pink noise under a random piecewise-linear amplitude envelope, seeded by the
    window's index (the stand-in for the benchmark's audio, which is not available here)."""
    n = SAMPLES_PER_WINDOW
    gen = torch.Generator(device=device).manual_seed(1000 + index)
    spec = torch.fft.rfft(torch.randn(n, generator=gen, device=device, dtype=torch.float32))
    f = torch.arange(spec.numel(), device=device, dtype=torch.float32)
    f[0] = 1.0
    x = torch.fft.irfft(spec / torch.sqrt(f), n)
    x = x / x.abs().max()
    knots = torch.rand(17, generator=gen, device=device) * 0.95 + 0.05
    pos = torch.linspace(0, 16, n, device=device)
    i0 = pos.floor().clamp(max=15).long()
    env = knots[i0] + (knots[i0 + 1] - knots[i0]) * (pos - i0)
    return (x * env).float()
