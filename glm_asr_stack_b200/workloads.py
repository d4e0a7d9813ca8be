"""Synthetic instances of the benchmark configurations: a random-init FP4 decoder with the
checkpoint's tensor names, and a paged-KV decode state (benchmark configuration 2: 256 sequences, context
lengths uniform in 200-450, 16-token pages handed out from a random permutation of the pool).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List

import numpy as np
import torch

from . import engine, synth
from .ops import Fp4Tensor

PROJ = [("self_attn.q_proj", "H", "H"), ("self_attn.k_proj", "KV", "H"), ("self_attn.v_proj", "KV", "H"),
        ("self_attn.o_proj", "H", "H"), ("mlp.gate_proj", "F", "H"), ("mlp.up_proj", "F", "H"),
        ("mlp.down_proj", "H", "F")]


@dataclass
class DecoderModel:
    ws: engine.WeightStore
    cfg: engine.CModelConfig
    embed: torch.Tensor            # bf16 [vocab, hidden]
    lm_head: Fp4Tensor             # FP4 [vocab, hidden] (an extension: the reference keeps lm_head in bf16)
    lm_head_input_scale: float
    weight_bytes: int              # FP4 bytes streamed per step: packed + block scales, layers + lm_head


def build_decoder(layers=28, hidden=2048, ffn=6144, heads=16, kv_heads=4, head_dim=128, vocab=59264,
                  input_scale=0.02, device="cuda", seed0=0) -> DecoderModel:
    dims = {"H": hidden, "KV": kv_heads * head_dim, "F": ffn}
    ws = engine.WeightStore()
    nbytes = 0
    for l in range(layers):
        for i, (name, n, k) in enumerate(PROJ):
            w = synth.seeded_weight_fast(dims[n], dims[k], seed0 + 1000 * l + i, device)
            ws.add_fp4(f"language_model.model.layers.{l}.{name}", w, input_scale)
            nbytes += w.w_packed.numel() + w.w_scales.numel()
        for nm in ("input_layernorm", "post_attention_layernorm"):
            ws.add(f"language_model.model.layers.{l}.{nm}.weight",
                   torch.ones(hidden, dtype=torch.bfloat16, device=device))
    ws.add("language_model.model.norm.weight", torch.ones(hidden, dtype=torch.bfloat16, device=device))
    gen = torch.Generator(device=device).manual_seed(seed0 + 77)
    embed = (torch.randn((vocab, hidden), generator=gen, device=device) * 1.0).to(torch.bfloat16)
    lm = synth.seeded_weight_fast(vocab, hidden, seed0 + 99, device)
    nbytes += lm.w_packed.numel() + lm.w_scales.numel()
    cfg = engine.model_config(hidden, layers, heads, kv_heads, head_dim, ffn, vocab)
    return DecoderModel(ws, cfg, embed, lm, input_scale, nbytes)


@dataclass
class DecodeState:
    pool: engine.KVPool
    bts: engine.BlockTables
    cached: np.ndarray             # int32 [num_seqs]
    d_seq_lens: torch.Tensor
    h_seq_lens: ctypes.Array
    kv_read_bytes: int             # K and V bytes attention reads per step (all layers)

    def reset_lengths(self):
        self.d_seq_lens.copy_(torch.from_numpy(self.cached).to(self.d_seq_lens.device))
        for i, c in enumerate(self.cached.tolist()):
            self.h_seq_lens[i] = c


def build_decode_state(cfg, num_seqs=256, ctx_lo=200, ctx_hi=450, block_size=16, seed=2, device="cuda") -> DecodeState:
    rng = np.random.default_rng(seed)
    cached = rng.integers(ctx_lo, ctx_hi + 1, num_seqs).astype(np.int32)
    need = [(int(c) + 1 + block_size - 1) // block_size for c in cached]
    max_blocks = max(need) + 1
    num_blocks = sum(need) + 64
    pool = engine.KVPool(num_blocks, block_size, cfg.dec_layers, cfg.dec_kv_heads, cfg.dec_head_dim, num_seqs,
                         max_blocks, device)
    perm = rng.permutation(num_blocks).tolist()
    tables: List[List[int]] = []
    for nb in need:
        tables.append([perm.pop() for _ in range(nb)])
    bts = engine.BlockTables(pool, tables)
    gen = torch.Generator(device=device).manual_seed(seed)
    for t in (pool.k, pool.v):          # K, V ~ N(0, 1), layer by layer to bound the temporary
        for l in range(t.shape[0]):
            t[l].copy_(torch.randn(t[l].shape, generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16))
    d_lens = torch.from_numpy(cached.copy()).to(device)
    h_lens = (ctypes.c_int * num_seqs)(*cached.tolist())
    row_bytes = cfg.dec_kv_heads * cfg.dec_head_dim * 2
    kv_bytes = int((cached.astype(np.int64) + 1).sum()) * row_bytes * 2 * cfg.dec_layers
    return DecodeState(pool, bts, cached, d_lens, h_lens, kv_bytes)


@dataclass
class PrefillState:
    pool: engine.KVPool
    bts: engine.BlockTables
    seq_lens: List[int]
    seq_offsets: List[int]
    total_tokens: int


def build_prefill_state(cfg, num_seqs=25, seq_len=400, block_size=16, seed=4, device="cuda") -> PrefillState:
    """A prefill batch as the reference's scheduler forms it: num_seqs windows of ~seq_len tokens packed
    back to back (10000 tokens = 25 x 400 at the batch limit), each with its own blocks of a fresh pool."""
    rng = np.random.default_rng(seed)
    lens = [int(seq_len)] * num_seqs
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)[:-1].tolist()
    need = [(ln + 1 + block_size - 1) // block_size for ln in lens]
    num_blocks = sum(need) + 16
    pool = engine.KVPool(num_blocks, block_size, cfg.dec_layers, cfg.dec_kv_heads, cfg.dec_head_dim, max(num_seqs, 1),
                         max(need) + 1, device)
    perm = rng.permutation(num_blocks).tolist()
    tables = [[perm.pop() for _ in range(nb)] for nb in need]
    bts = engine.BlockTables(pool, tables)
    return PrefillState(pool, bts, lens, [int(o) for o in offs], int(sum(lens)))
