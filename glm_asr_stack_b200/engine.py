"""ctypes mirrors of the engine structures that cross the decode entry points, and helpers that
build them from torch tensors (reference: Infer-engine/include/types.h, kv_pool.h; C layout in
include/glmasr_engine_types.h).  Used by the tests and the benchmark to call
``decoder_decode_step_batched`` exactly as the engine's ``decode_batch`` does
(Infer-engine/src/engine.c:1880-1982).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_int, c_int64, c_size_t, c_void_p
from typing import Dict, List, Optional

import torch

from . import _lib, ops
from .weights import DTYPE_BF16, DTYPE_FP32, DTYPE_FP8, DTYPE_UINT8

MAX_DIMS = 4
MAX_WEIGHTS = 2048


class CTensor(Structure):
    _fields_ = [("data", c_void_p), ("dtype", c_int), ("ndim", c_int), ("shape", c_int64 * MAX_DIMS),
                ("nbytes", c_size_t)]


class CModelConfig(Structure):
    _fields_ = [(n, c_int) for n in ("enc_hidden", "enc_layers", "enc_heads", "enc_head_dim", "enc_ffn",
                                     "num_mel_bins", "max_audio_frames", "proj_mid", "dec_hidden", "dec_layers",
                                     "dec_heads", "dec_kv_heads", "dec_head_dim", "dec_ffn", "vocab_size",
                                     "max_position_embeddings", "audio_token_id")] + \
               [("eos_ids", c_int * 4), ("pad_token_id", c_int), ("max_new_tokens", c_int)]


class CWeightStore(Structure):
    _fields_ = [("names", c_char_p * MAX_WEIGHTS), ("tensors", CTensor * MAX_WEIGHTS), ("count", c_int)]


class CKVPool(Structure):
    _fields_ = [("k_cache", c_void_p), ("v_cache", c_void_p), ("d_block_tables", c_void_p), ("max_seqs", c_int),
                ("max_blocks_per_seq", c_int), ("free_stack", POINTER(c_int)), ("free_top", c_int),
                ("num_blocks", c_int), ("block_size", c_int), ("num_layers", c_int), ("kv_heads", c_int),
                ("head_dim", c_int), ("kv_head_stride", c_int), ("block_stride", c_int), ("layer_stride", c_int),
                ("per_layer_bytes", c_size_t)]


class CBlockTable(Structure):
    _fields_ = [("d_table", c_void_p), ("max_blocks", c_int), ("num_blocks", c_int), ("h_table", POINTER(c_int)),
                ("seq_idx", c_int)]


_TAGS = {torch.float32: DTYPE_FP32, torch.bfloat16: DTYPE_BF16, torch.uint8: DTYPE_UINT8,
         torch.float8_e4m3fn: DTYPE_FP8}


class WeightStore:
    """Owns the tensors and the C ``WeightStore`` that points at them."""

    def __init__(self):
        self.c = CWeightStore()
        self.c.count = 0
        self.keep: Dict[str, torch.Tensor] = {}
        self._forget_cached_table()

    @staticmethod
    def _forget_cached_table():
        # The library keeps a per-store table of pointers and of the scalar tensors' VALUES
        # (weight_scale_2, input_scale: read once, as the reference's decoder_scalar_read_cached does).
        # A new store can reuse a freed store's address, and its tensors the old tensors' addresses, with
        # different contents, so the table is dropped whenever a store is created or changed
        # (the C host calls glmasr_decoder_forget_weights from safetensors_free).
        _lib.load().glmasr_decoder_forget_weights()

    def add(self, name: str, t: torch.Tensor, dtype: Optional[int] = None):
        self._forget_cached_table()
        i = self.c.count
        assert i < MAX_WEIGHTS
        self.keep[name] = t
        self.c.names[i] = name.encode()
        ct = self.c.tensors[i]
        ct.data = t.data_ptr()
        ct.dtype = _TAGS[t.dtype] if dtype is None else dtype
        ct.ndim = t.dim()
        for d in range(t.dim()):
            ct.shape[d] = t.shape[d]
        ct.nbytes = t.numel() * t.element_size()
        self.c.count = i + 1

    def add_fp4(self, prefix: str, w, input_scale: Optional[float] = None):
        """The five tensors of one FP4 projection under the checkpoint's names."""
        dev = w.w_packed.device
        # the library caches re-tiled scales by device pointer: drop the entry when this tensor goes away
        # (what the C host does from safetensors_free), or a later weight at the same address would inherit it
        ops._track_scales(w.w_scales)
        self.add(f"{prefix}.weight", w.w_packed)
        self.add(f"{prefix}.weight_scale", w.w_scales, DTYPE_FP8)
        self.add(f"{prefix}.weight_scale_2", torch.tensor([w.w_global_scale], dtype=torch.float32, device=dev))
        if input_scale is not None:
            self.add(f"{prefix}.input_scale", torch.tensor([input_scale], dtype=torch.float32, device=dev))


class LoadedWeightStore:
    """A C ``WeightStore`` filled by ``safetensors_load`` (Infer-engine/src/safetensors.c:57-181): the library owns
    the device memory (one allocation per file) until ``close()`` calls ``safetensors_free``."""

    def __init__(self, path: str):
        self.c = CWeightStore()
        self.c.count = 0
        rc = _lib.load().safetensors_load(os.fsencode(path), ctypes.byref(self.c))
        if rc != 0:
            raise OSError(f"safetensors_load({path!r}) failed")
        self._open = True

    def names(self) -> List[str]:
        return [self.c.names[i].decode() for i in range(self.c.count)]

    def entry(self, i: int):
        t = self.c.tensors[i]
        return {"name": self.c.names[i].decode(), "dtype": t.dtype, "shape": [int(t.shape[d]) for d in range(t.ndim)],
                "nbytes": int(t.nbytes), "data": int(t.data or 0)}

    def close(self):
        if self._open:
            _lib.load().safetensors_free(ctypes.byref(self.c))
            self._open = False

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def inspect_safetensors(path: str):
    """glmasr_safetensors_inspect: the header pass alone (no CUDA).  Returns (entries, arena_bytes); an entry's
    ``data`` is its offset inside the one device allocation a load would make."""
    lib = _lib.load()
    c = CWeightStore()
    c.count = 0
    arena = c_size_t(0)
    if lib.glmasr_safetensors_inspect(os.fsencode(path), ctypes.byref(c), ctypes.byref(arena)) != 0:
        raise OSError(f"glmasr_safetensors_inspect({path!r}) failed")
    out = []
    for i in range(c.count):
        t = c.tensors[i]
        out.append({"name": c.names[i].decode(), "dtype": t.dtype, "shape": [int(t.shape[d]) for d in range(t.ndim)],
                    "nbytes": int(t.nbytes), "data": int(t.data or 0)})
    lib.glmasr_safetensors_release_index(ctypes.byref(c))
    return out, int(arena.value)


def encoder_config(cfg: CModelConfig, hidden=1280, layers=32, heads=20, head_dim=64, ffn=5120, mels=128, max_frames=3000,
                   proj_mid=4096) -> CModelConfig:
    """Fill the audio side of a ModelConfig (Infer-engine/include/types.h:37-72; the defaults are the checkpoint's)."""
    cfg.enc_hidden, cfg.enc_layers, cfg.enc_heads, cfg.enc_head_dim, cfg.enc_ffn = hidden, layers, heads, head_dim, ffn
    cfg.num_mel_bins, cfg.max_audio_frames, cfg.proj_mid = mels, max_frames, proj_mid
    return cfg


def model_config(hidden=2048, layers=28, heads=16, kv_heads=4, head_dim=128, ffn=6144, vocab=59264) -> CModelConfig:
    c = CModelConfig()
    c.dec_hidden, c.dec_layers, c.dec_heads, c.dec_kv_heads = hidden, layers, heads, kv_heads
    c.dec_head_dim, c.dec_ffn, c.vocab_size = head_dim, ffn, vocab
    c.max_position_embeddings = 8192
    return c


class KVPool:
    """Paged KV pool with the reference's layout (Infer-engine/src/kv_pool.c:35-120): K and V each one
    allocation [layers][num_blocks][block_size][kv_heads][head_dim] bf16, device block tables
    [max_seqs, max_blocks_per_seq] int32, a host LIFO of free block ids."""

    def __init__(self, num_blocks, block_size, num_layers, kv_heads, head_dim, max_seqs, max_blocks_per_seq,
                 device="cuda"):
        row = kv_heads * head_dim
        self.k = torch.zeros((num_layers, num_blocks, block_size, row), dtype=torch.bfloat16, device=device)
        self.v = torch.zeros_like(self.k)
        self.tables = torch.full((max_seqs, max_blocks_per_seq), -1, dtype=torch.int32, device=device)
        self.free = list(range(num_blocks - 1, -1, -1))
        self._stack = (c_int * num_blocks)(*range(num_blocks))
        c = CKVPool()
        c.k_cache, c.v_cache, c.d_block_tables = self.k.data_ptr(), self.v.data_ptr(), self.tables.data_ptr()
        c.max_seqs, c.max_blocks_per_seq = max_seqs, max_blocks_per_seq
        c.free_stack = ctypes.cast(self._stack, POINTER(c_int))
        c.free_top, c.num_blocks, c.block_size, c.num_layers = num_blocks, num_blocks, block_size, num_layers
        c.kv_heads, c.head_dim, c.kv_head_stride = kv_heads, head_dim, row
        c.block_stride = block_size * row
        c.layer_stride = num_blocks * block_size * row
        c.per_layer_bytes = num_blocks * block_size * row * 2
        self.c = c
        self.block_size, self.max_blocks_per_seq = block_size, max_blocks_per_seq


class BlockTables:
    """``BlockTable[num_seqs]`` with host mirrors; row i of the pool's device table belongs to sequence i."""

    def __init__(self, pool: KVPool, tables: List[List[int]]):
        n = len(tables)
        self.arr = (CBlockTable * n)()
        self._host = []
        host = torch.full((n, pool.max_blocks_per_seq), -1, dtype=torch.int32)
        for i, blocks in enumerate(tables):
            h = (c_int * pool.max_blocks_per_seq)(*([-1] * pool.max_blocks_per_seq))
            for j, b in enumerate(blocks):
                h[j] = b
                host[i, j] = b
            self._host.append(h)
            bt = self.arr[i]
            bt.d_table = pool.tables.data_ptr() + i * pool.max_blocks_per_seq * 4
            bt.max_blocks, bt.num_blocks = pool.max_blocks_per_seq, len(blocks)
            bt.h_table = ctypes.cast(h, POINTER(c_int))
            bt.seq_idx = i
        pool.tables[:n].copy_(host.to(pool.tables.device))


def decode_step(ws: WeightStore, cfg: CModelConfig, pool: KVPool, bts: BlockTables, hidden: torch.Tensor,
                d_seq_lens: torch.Tensor, h_seq_lens):
    """Call decoder_decode_step_batched on a contiguous [num_seqs, hidden] batch (updated in place).
    h_seq_lens: ctypes int array (updated in place)."""
    lib = _lib.load()
    n = hidden.shape[0]
    ptrs = (c_void_p * n)(*[hidden.data_ptr() + i * hidden.shape[1] * 2 for i in range(n)])
    lib.decoder_decode_step_batched(None, ctypes.byref(ws.c), ptrs, ctypes.byref(pool.c), bts.arr,
                                    c_void_p(d_seq_lens.data_ptr()), h_seq_lens, n, None, None, ctypes.byref(cfg))


def prefill_paged_batched(ws: WeightStore, cfg: CModelConfig, pool: KVPool, bts: BlockTables, hidden: torch.Tensor,
                          seq_lens, seq_offsets, first: int = 0):
    """Call decoder_prefill_paged_batched on hidden [total_tokens, hidden] (updated in place).
    seq_lens / seq_offsets: host sequences of ints, one entry per sequence (rows of sequence s are
    [seq_offsets[s], seq_offsets[s] + seq_lens[s])); sequence s uses block table bts[first + s]."""
    lib = _lib.load()
    n = len(seq_lens)
    lens = (ctypes.c_int * n)(*[int(v) for v in seq_lens])
    offs = (ctypes.c_int * n)(*[int(v) for v in seq_offsets])
    tables = c_void_p(ctypes.addressof(bts.arr) + first * ctypes.sizeof(CBlockTable))
    lib.decoder_prefill_paged_batched(None, ctypes.byref(ws.c), c_void_p(hidden.data_ptr()), hidden.shape[0], n, lens, offs,
                                      ctypes.byref(pool.c), tables, None, ctypes.byref(cfg))
    return hidden


def prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                      q_heads: int, kv_heads: int, head_dim: int, causal: bool = True) -> torch.Tensor:
    """flash_fwd_vllm_gqa_launch: variable-length GQA self-attention; q / k / v may be column slices
    (row strides are passed), cu_seqlens int32 [num_seqs + 1] on the device."""
    lib = _lib.load()
    total = q.shape[0]
    out = torch.empty((total, q_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    ok = lib.flash_fwd_vllm_gqa_launch(c_void_p(q.data_ptr()), c_void_p(k.data_ptr()), c_void_p(v.data_ptr()),
                                       c_void_p(out.data_ptr()), total, int(max_seqlen), q_heads, kv_heads, head_dim,
                                       q.stride(0), k.stride(0), v.stride(0), cu_seqlens.numel() - 1,
                                       c_void_p(cu_seqlens.data_ptr()), 1 if causal else 0)
    if ok != 1:
        raise ValueError("flash_fwd_vllm_gqa_launch rejected the layout")
    return out
