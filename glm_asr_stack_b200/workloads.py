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


def add_audio_tower(ws: engine.WeightStore, cfg, layers=32, hidden=1280, heads=20, head_dim=64, ffn=5120, mels=128,
                    proj_mid=4096, device="cuda", seed0=5000):
    """Random-init bf16 audio encoder, convolution front end and projector under the checkpoint's tensor names
    (Infer-engine/cuda/encoder.cu:1996-2186, Infer-engine/src/engine.c:1116-1153): weights ~ N(0, 0.02), LayerNorm
    weights around 1, small biases (k_proj has none).  Fills the audio fields of cfg.  Returns the bytes added."""
    engine.encoder_config(cfg, hidden, layers, heads, head_dim, ffn, mels, 3000, proj_mid)
    gen = torch.Generator(device=device).manual_seed(seed0)
    nbytes = 0

    def add(name, shape, std, mean=0.0):
        nonlocal nbytes
        t = (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std + mean).to(torch.bfloat16)
        ws.add(name, t)
        nbytes += t.numel() * 2

    add("audio_tower.conv1.weight", (hidden, mels, 3), 0.02)
    add("audio_tower.conv1.bias", (hidden,), 0.02)
    add("audio_tower.conv2.weight", (hidden, hidden, 3), 0.02)
    add("audio_tower.conv2.bias", (hidden,), 0.02)
    for l in range(layers):
        p = f"audio_tower.layers.{l}."
        for ln in ("input_layernorm", "post_attention_layernorm"):
            add(p + ln + ".weight", (hidden,), 0.1, 1.0)
            add(p + ln + ".bias", (hidden,), 0.02)
        for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
            add(p + f"self_attn.{proj}.weight", (hidden, hidden), 0.02)
            if proj != "k_proj":
                add(p + f"self_attn.{proj}.bias", (hidden,), 0.02)
        add(p + "mlp.fc1.weight", (ffn, hidden), 0.02)
        add(p + "mlp.fc1.bias", (ffn,), 0.02)
        add(p + "mlp.fc2.weight", (hidden, ffn), 0.02)
        add(p + "mlp.fc2.bias", (hidden,), 0.02)
    add("audio_tower.norm.weight", (hidden,), 0.1, 1.0)
    add("audio_tower.norm.bias", (hidden,), 0.02)
    add("multi_modal_projector.linear_1.weight", (proj_mid, 4 * hidden), 0.02)
    add("multi_modal_projector.linear_1.bias", (proj_mid,), 0.02)
    add("multi_modal_projector.linear_2.weight", (cfg.dec_hidden, proj_mid), 0.02)
    add("multi_modal_projector.linear_2.bias", (cfg.dec_hidden,), 0.02)
    return nbytes


def encoder_flops(rows_per_window: int, windows: int, hidden=1280, heads=20, head_dim=64, ffn=5120, layers=32, mels=128,
                  proj_mid=4096, dec_hidden=2048) -> float:
    """Multiply-add flops (x2) of the audio path for `windows` windows of rows_per_window encoder frames: the two
    convolutions, the layers' six GEMMs and attention (non-causal, both products), the projector."""
    t2 = rows_per_window
    t1 = 2 * t2
    conv = 2.0 * t1 * hidden * 3 * mels + 2.0 * t2 * hidden * 3 * hidden
    layer = 2.0 * t2 * (4 * hidden * hidden + 2 * hidden * ffn) + 2.0 * 2 * heads * head_dim * t2 * t2
    proj = 2.0 * (t2 // 4) * (4 * hidden * proj_mid + proj_mid * dec_hidden)
    return windows * (conv + layers * layer + proj)


def build_asr_model(dec_layers=28, enc_layers=32, device="cuda", **dec_kwargs) -> DecoderModel:
    """The FP4 decoder of build_decoder plus the bf16 audio tower and projector in the same weight store."""
    model = build_decoder(layers=dec_layers, device=device, **dec_kwargs)
    add_audio_tower(model.ws, model.cfg, layers=enc_layers, device=device)
    return model
