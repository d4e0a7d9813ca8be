"""ctypes access to the reference's OWN FP4 kernels, compiled unmodified from the reference
sources into oracle/_ref/libglmasr_ref.so by oracle/Makefile (test infrastructure; needs a GPU).
"""
import ctypes
import os
from ctypes import c_float, c_int, c_void_p

import torch

from conftest import ROOT

REF_SO = os.path.join(ROOT, "oracle", "_ref", "libglmasr_ref.so")
P = c_void_p


def available() -> bool:
    return os.path.exists(REF_SO)


class RefLib:
    def __init__(self):
        self.lib = ctypes.CDLL(REF_SO, mode=ctypes.RTLD_LOCAL)
        L = self.lib
        L.fp4_dequant_to_bf16.argtypes = [P, P, P, c_float, c_int, c_int]
        L.fp4_linear.argtypes = [P, P, P, P, P, P, P, c_float, P, P, c_int, c_int, c_int]
        L.nvfp4_linear.argtypes = [P, P, P, P, P, P, c_float, c_float, P, P, c_int, c_int, c_int]
        L.nvfp4_linear.restype = c_int
        L.bf16_linear.argtypes = [P, P, P, P, P, c_int, c_int, c_int]
        L.silu_mul_split_packed.argtypes = [P, P, c_int, c_int]
        L.residual_add.argtypes = [P, P, P, c_int]
        L.lm_head_argmax_batched.argtypes = [P, P, P, c_int, c_int, c_int, P]
        for f in (L.fp4_dequant_to_bf16, L.fp4_linear, L.bf16_linear, L.silu_mul_split_packed, L.residual_add,
                  L.lm_head_argmax_batched):
            f.restype = None
        L.rmsnorm.argtypes = [P, P, P, c_float, c_int, c_int]
        L.rmsnorm.restype = None
        L.reshape_and_cache.argtypes = [P, P, P, P, P, c_int, c_int, c_int, c_int]
        L.reshape_and_cache.restype = None
        L.paged_decode_attention.argtypes = [P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int]
        L.paged_decode_attention.restype = None
        if hasattr(L, "mel_spectrogram"):
            L.mel_spectrogram.argtypes = [P, c_int, P, P, P]
            L.mel_spectrogram.restype = None
        if hasattr(L, "encoder_forward_packed"):
            L.layernorm.argtypes = [P, P, P, P, c_float, c_int, c_int]
            L.layernorm.restype = None
            L.gelu_inplace.argtypes = [P, c_int]
            L.gelu_inplace.restype = None
            L.conv1d_forward.argtypes = [P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int]
            L.conv1d_forward.restype = None
            L.encoder_forward_packed.argtypes = [P, P, P, c_int, c_int, P, P, P]
            L.encoder_forward_packed.restype = None
            L.bf16_linear_gelu.argtypes = [P, P, P, P, P, c_int, c_int, c_int]
            L.bf16_linear_gelu.restype = None
        # the reference's fp4_linear / bf16_linear take a cublasHandle_t
        self.cublas = ctypes.CDLL("libcublas.so.12")
        self.handle = c_void_p()
        rc = self.cublas.cublasCreate_v2(ctypes.byref(self.handle))
        assert rc == 0, f"cublasCreate failed: {rc}"

    @staticmethod
    def _p(t):
        return None if t is None else c_void_p(t.data_ptr())

    def fp4_dequant_to_bf16(self, packed, scales, g):
        rows, cols = packed.shape[0], packed.shape[1] * 2
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device="cuda")
        self.lib.fp4_dequant_to_bf16(self._p(out), self._p(packed), self._p(scales), g, rows, cols)
        torch.cuda.synchronize()
        return out

    def fp4_linear(self, x, packed, scales, g, pre=None):
        M, K = x.shape
        N = packed.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        wscratch = torch.empty((N, K), dtype=torch.bfloat16, device="cuda")
        pscratch = torch.empty((M, K), dtype=torch.bfloat16, device="cuda")
        self.lib.fp4_linear(self.handle, self._p(out), self._p(wscratch), self._p(pscratch), self._p(x),
                            self._p(packed), self._p(scales), g, self._p(pre), None, M, N, K)
        torch.cuda.synchronize()
        return out

    def nvfp4_linear(self, x, packed, scales, input_scale, g, pre=None):
        M, K = x.shape
        N = packed.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        # the reference carves its temporaries from dequant_buf + N*K; give it ample room
        mp = (M + 127) // 128 * 128
        extra = mp * K + 4 * mp * (K // 16 + 4) + ((N + 127) // 128 * 128) * (K // 16 + 4) + 2 * mp * N + 4096
        buf = torch.empty(N * K + (extra + 1) // 2 + 1024, dtype=torch.bfloat16, device="cuda")
        rc = self.lib.nvfp4_linear(self.handle, self._p(out), self._p(buf), self._p(x), self._p(packed),
                                   self._p(scales), input_scale, g, self._p(pre), None, M, N, K)
        torch.cuda.synchronize()
        return rc, out

    def has_encoder(self):
        return hasattr(self.lib, "encoder_forward_packed")

    def layernorm(self, x, w, b, eps=1e-5):
        out = torch.empty_like(x)
        self.lib.layernorm(self._p(out), self._p(x), self._p(w), self._p(b), eps, x.shape[0], x.shape[1])
        torch.cuda.synchronize()
        return out

    def gelu_inplace(self, x):
        y = x.clone()
        self.lib.gelu_inplace(self._p(y), y.numel())
        torch.cuda.synchronize()
        return y

    def conv1d_forward(self, x, w, b, stride, padding):
        in_ch, ln = x.shape
        out_ch, _, ks = w.shape
        out_len = (ln + 2 * padding - ks) // stride + 1
        out = torch.empty((out_ch, out_len), dtype=torch.bfloat16, device="cuda")
        self.lib.conv1d_forward(self._p(out), self._p(x), self._p(w), self._p(b), in_ch, out_ch, ln, ks, stride, padding)
        torch.cuda.synchronize()
        return out

    def encoder_forward_packed(self, ws, cfg, hidden, seq_lens, seq_offsets):
        """The reference's encoder on a ctypes WeightStore / ModelConfig (same struct layouts); returns a new tensor."""
        h = hidden.clone()
        n = len(seq_lens)
        lens = (ctypes.c_int * n)(*[int(v) for v in seq_lens])
        offs = (ctypes.c_int * n)(*[int(v) for v in seq_offsets])
        self.lib.encoder_forward_packed(self.handle, ctypes.byref(ws.c), self._p(h), h.shape[0], n, lens, offs, ctypes.byref(cfg))
        torch.cuda.synchronize()
        return h

    def mel_spectrogram(self, pcm, filters_t):
        """Infer-engine/cuda/mel.cu:253-294 -> bf16 [128, n_frames]."""
        ns = pcm.numel()
        n = min(max((ns + 159) // 160, 1), 3000)
        out = torch.empty((128, n), dtype=torch.bfloat16, device="cuda")
        frames = ctypes.c_int(0)
        self.lib.mel_spectrogram(self._p(pcm), ns, self._p(filters_t), self._p(out), ctypes.byref(frames))
        torch.cuda.synchronize()
        assert frames.value == n
        return out

    def rmsnorm(self, x, w, eps=1e-5):
        out = torch.empty_like(x)
        self.lib.rmsnorm(self._p(out), self._p(x), self._p(w), eps, x.shape[0], x.shape[1])
        torch.cuda.synchronize()
        return out

    def reshape_and_cache(self, kc, vc, k, v, slots, kv_heads, head_dim, block_size):
        self.lib.reshape_and_cache(self._p(kc), self._p(vc), self._p(k), self._p(v), self._p(slots), k.shape[0],
                                   kv_heads, head_dim, block_size)
        torch.cuda.synchronize()

    def paged_decode_attention(self, q, kc, vc, bt, lens, qh, kvh, hd, bs):
        out = torch.empty_like(q)
        self.lib.paged_decode_attention(self._p(out), self._p(q), self._p(kc), self._p(vc), self._p(bt), self._p(lens),
                                        q.shape[0], qh, kvh, hd, bs, bt.shape[1])
        torch.cuda.synchronize()
        return out

    def silu_mul_split_packed(self, packed):
        M, N2 = packed.shape
        out = torch.empty((M, N2 // 2), dtype=torch.bfloat16, device="cuda")
        self.lib.silu_mul_split_packed(self._p(out), self._p(packed), M, N2 // 2)
        torch.cuda.synchronize()
        return out

    def residual_add(self, a, b):
        out = torch.empty_like(a)
        self.lib.residual_add(self._p(out), self._p(a), self._p(b), a.numel())
        torch.cuda.synchronize()
        return out

    def lm_head_argmax_batched(self, hidden, w):
        rows, dim = hidden.shape
        tokens = torch.empty(rows, dtype=torch.int32)
        self.lib.lm_head_argmax_batched(self.handle, self._p(hidden), self._p(w), rows, dim, w.shape[0],
                                        c_void_p(tokens.data_ptr()))
        return tokens
