"""safetensors -> WeightStore (safetensors_load / safetensors_free, Infer-engine/src/safetensors.c:57-193).

CPU: the header pass (glmasr_safetensors_inspect) against the oracle's restatement of the reference parser on
files with the checkpoint's tensor kinds and on the parser's corner cases.  GPU: a load compared byte for byte
with the file, the arena's alignment, and a decode step on the loaded store equal to one on the same weights
handed over as torch tensors.
"""
import ctypes
import os

import numpy as np
import pytest

import safetensors_oracle as so

DTYPE_STR = {"u8": "U8", "fp8": "F8_E4M3", "f32": "F32", "bf16": "BF16"}


def device_bytes(ptr, nbytes):
    """nbytes of device memory at ptr, copied to the host with the CUDA runtime torch has loaded."""
    import torch  # noqa: F401  (loads libcudart)
    rt = None
    for name in ("libcudart.so.12", "libcudart.so"):
        try:
            rt = ctypes.CDLL(name)
            break
        except OSError:
            continue
    assert rt is not None, "CUDA runtime library not found"
    rt.cudaMemcpy.restype = ctypes.c_int
    rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    buf = ctypes.create_string_buffer(nbytes)
    assert rt.cudaMemcpy(buf, ctypes.c_void_p(ptr), nbytes, 2) == 0          # cudaMemcpyDeviceToHost
    return buf.raw


def corner_case_file(path, rng):
    ts = [("language_model.model.layers.0.self_attn.q_proj.weight", "U8", (8, 16), rng.integers(0, 255, 128, dtype=np.uint8).tobytes()),
          ("language_model.model.layers.0.self_attn.q_proj.weight_scale", "F8_E4M3", (8, 2), rng.integers(0, 255, 16, dtype=np.uint8).tobytes()),
          ("language_model.model.layers.0.self_attn.q_proj.weight_scale_2", "F32", (), np.float32(0.5).tobytes()),
          ("position_ids", "I64", (3,), np.arange(3, dtype=np.int64).tobytes()),                  # unknown dtype: skipped
          ("norm", "BF16", (7,), rng.integers(0, 65535, 7, dtype=np.uint16).tobytes()),          # odd byte count
          ("five_dims", "BF16", (1, 1, 2, 1, 3), rng.integers(0, 65535, 6, dtype=np.uint16).tobytes()),   # 4 dims kept
          ("empty", "F32", (0,), b""),
          ("esc\\\"aped", "F16", (2,), b"\x01\x02\x03\x04"),
          ("big", "BF16", (300, 1000), rng.integers(0, 65535, 300000, dtype=np.uint16).tobytes())]
    so.write_file(path, ts, metadata={"format": "pt", "note": "braces } ] \" inside a string"})
    return ts


def test_header_pass_matches_the_reference_parser(tmp_path, product_lib):
    from glm_asr_stack_b200 import engine
    rng = np.random.default_rng(0)
    path = str(tmp_path / "model.safetensors")
    corner_case_file(path, rng)
    want = so.load_index(path)
    got, arena = engine.inspect_safetensors(path)
    assert [g["name"] for g in got] == [w["name"] for w in want]
    assert "position_ids" not in [g["name"] for g in got]
    for g, w in zip(got, want):
        assert (g["dtype"], g["shape"], g["nbytes"]) == (w["dtype"], w["shape"], w["nbytes"]), g["name"]
    # arena layout: header order, 256-byte aligned, no overlap, everything inside the arena
    prev_end = 0
    for g in got:
        assert g["data"] % 256 == 0 and g["data"] >= prev_end
        prev_end = g["data"] + max(g["nbytes"], 4)
    assert prev_end <= arena and arena % 256 == 0


def test_header_pass_entry_limit_and_missing_file(tmp_path, product_lib):
    from glm_asr_stack_b200 import engine
    path = str(tmp_path / "many.safetensors")
    so.write_file(path, [(f"t{i}", "U8", (1,), bytes([i % 251])) for i in range(2100)])
    got, _ = engine.inspect_safetensors(path)
    assert len(got) == 2048 == len(so.load_index(path))              # MAX_WEIGHTS
    with pytest.raises(OSError):
        engine.inspect_safetensors(str(tmp_path / "absent.safetensors"))
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\xff" * 12)                                       # header length beyond the file
    with pytest.raises(OSError):
        engine.inspect_safetensors(str(bad))


@pytest.mark.gpu
def test_load_is_byte_exact_and_aligned(tmp_path):
    import torch

    from glm_asr_stack_b200 import engine
    rng = np.random.default_rng(1)
    path = str(tmp_path / "model.safetensors")
    corner_case_file(path, rng)
    # a tensor larger than one 64 MiB staging window, starting at an odd offset of the data region
    big = rng.integers(0, 255, 70 * (1 << 20) + 13, dtype=np.uint8)
    ts = [("odd", "U8", (3,), b"\x07\x08\x09"), ("huge", "U8", (big.size,), big.tobytes()),
          ("tail", "F32", (5,), rng.standard_normal(5).astype(np.float32).tobytes())]
    path2 = str(tmp_path / "large.safetensors")
    so.write_file(path2, ts)
    for p in (path, path2):
        want = so.load_index(p)
        store = engine.LoadedWeightStore(p)
        assert store.names() == [w["name"] for w in want]
        for i, w in enumerate(want):
            e = store.entry(i)
            assert (e["dtype"], e["shape"], e["nbytes"]) == (w["dtype"], w["shape"], w["nbytes"])
            assert e["data"] % 256 == 0 and e["data"] != 0
            if w["nbytes"]:
                assert device_bytes(e["data"], w["nbytes"]) == so.tensor_bytes(p, w), w["name"]
        store.close()
        assert store.c.count == 0


@pytest.mark.gpu
def test_decode_step_on_a_loaded_store_equals_the_tensor_built_one(tmp_path):
    """The toy decoder written to a safetensors file under the checkpoint's names, loaded by safetensors_load,
    against the same weights handed to the step as torch tensors: same bytes out."""
    import torch

    import test_gpu_decoder as tgd
    from glm_asr_stack_b200 import engine, ops
    from gpu_util import bits_of, to_dev_bf16
    rng = np.random.default_rng(31)
    ws, cfg, layers, fn, (H, F, QH, KVH, HD, L) = tgd.build_toy_model(rng, 700, "plain")
    tag2str = {0: "F32", 1: "BF16", 3: "U8", 4: "F8_E4M3"}
    ts = []
    for i in range(ws.c.count):
        name = ws.c.names[i].decode()
        t = ws.keep[name]
        raw = t.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes()
        scalar = name.endswith((".weight_scale_2", ".input_scale"))          # 0-dim F32 in the checkpoint
        ts.append((name, tag2str[ws.c.tensors[i].dtype], () if scalar else tuple(t.shape), raw))
    path = str(tmp_path / "model.safetensors")
    so.write_file(path, ts, metadata={"format": "pt"})
    loaded = engine.LoadedWeightStore(path)

    def run(store):
        r = np.random.default_rng(5)
        bs, n = 16, 4
        cached = np.array([3, 16, 40, 100], np.int32)
        pool = engine.KVPool(64, bs, L, KVH, HD, max_seqs=8, max_blocks_per_seq=16)
        perm = r.permutation(64).tolist()
        tables = [[perm.pop() for _ in range((int(c) + 1 + bs - 1) // bs)] for c in cached]
        bts = engine.BlockTables(pool, tables)
        pool.k.copy_(to_dev_bf16(tgd.rnd_bits(r, tuple(pool.k.shape))))
        pool.v.copy_(to_dev_bf16(tgd.rnd_bits(r, tuple(pool.v.shape))))
        hid = to_dev_bf16(tgd.rnd_bits(r, (n, H)))
        d_lens = torch.from_numpy(cached.copy()).cuda()
        h_lens = (ctypes.c_int * n)(*cached.tolist())
        engine.decode_step(store, cfg, pool, bts, hid, d_lens, h_lens)
        torch.cuda.synchronize()
        assert ops.status() == 0
        return bits_of(hid), bits_of(pool.k), bits_of(pool.v)

    a = run(ws)
    b = run(loaded)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    loaded.close()
