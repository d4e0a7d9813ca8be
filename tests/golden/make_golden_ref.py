"""Generate golden input/output vectors by RUNNING THE REFERENCE'S OWN KERNELS on a GPU.

The reference path is CUDA only (no CPU code, no tests, no fixtures), so it cannot run in a
GPU-less container.  oracle/Makefile compiles the reference sources, unmodified, into
oracle/_ref/libglmasr_ref.so; this script calls that library on seeded inputs and stores
inputs + outputs as small .npz files.  Run it on a B200 box:

    python tests/golden/make_golden_ref.py [out_dir]

The committed fixtures under tests/golden/ were produced this way; tests/test_golden_ref.py
checks the CPU oracle against them without a GPU.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")]

import fp4_oracle as o  # noqa: E402
import ref_lib  # noqa: E402
from gpu_util import bits_of, to_dev_bf16, to_dev_u8  # noqa: E402


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    ref = ref_lib.RefLib()
    rng = np.random.default_rng(2024)

    # fp4_dequant_to_bf16, including every e4m3 code as a scale
    pw = rng.integers(0, 256, (32, 64), dtype=np.uint8)
    sw = np.arange(256, dtype=np.uint8).reshape(32, 8)
    g = 0.0123
    out = bits_of(ref.fp4_dequant_to_bf16(to_dev_u8(pw), to_dev_u8(sw), g))
    np.savez_compressed(os.path.join(out_dir, "ref_dequant.npz"), packed=pw, scales=sw, g=np.float32(g), out=out)

    # fp4_linear (W4A16 fallback), with and without pre_quant_scale
    for tag, M, N, K, pre in (("a", 24, 32, 64, False), ("b", 40, 128, 256, True)):
        pw, sw, g = o.seeded_weight(N, K, 10)
        x = o.seeded_activation(M, K, 11)
        pb = o.f32_to_bf16_bits(rng.uniform(0.5, 2.0, K).astype(np.float32)) if pre else None
        out = bits_of(ref.fp4_linear(to_dev_bf16(x), to_dev_u8(pw), to_dev_u8(sw), g,
                                     to_dev_bf16(pb) if pre else None))
        np.savez_compressed(os.path.join(out_dir, f"ref_fp4_linear_{tag}.npz"), x=x, packed=pw, scales=sw,
                            g=np.float32(g), pre=pb if pre else np.zeros(0, np.uint16), out=out)

    # nvfp4_linear (W4A4, cuBLASLt FP4), M multiple of 16 and not (padding path)
    for tag, M, N, K, pre in (("a", 32, 128, 256, False), ("b", 24, 256, 512, True)):
        pw, sw, g = o.seeded_weight(N, K, 20)
        x = o.seeded_activation(M, K, 21)
        isc = o.default_input_scale(x)
        pb = o.f32_to_bf16_bits(rng.uniform(0.5, 2.0, K).astype(np.float32)) if pre else None
        rc, out = ref.nvfp4_linear(to_dev_bf16(x), to_dev_u8(pw), to_dev_u8(sw), isc, g,
                                   to_dev_bf16(pb) if pre else None)
        if rc != 0:
            print(f"reference nvfp4_linear returned {rc} for case {tag}: not recorded")
            continue
        np.savez_compressed(os.path.join(out_dir, f"ref_nvfp4_linear_{tag}.npz"), x=x, packed=pw, scales=sw,
                            g=np.float32(g), input_scale=np.float32(isc),
                            pre=pb if pre else np.zeros(0, np.uint16), out=bits_of(out))

    # SiLU-gate, residual add, lm_head arg-max with ties
    gu = o.f32_to_bf16_bits(rng.standard_normal((16, 64)).astype(np.float32) * 4)
    a = o.f32_to_bf16_bits(rng.standard_normal(512).astype(np.float32))
    b = o.f32_to_bf16_bits(rng.standard_normal(512).astype(np.float32))
    h = np.zeros((3, 64), np.float32)
    w = (rng.standard_normal((1024, 64)) * 0.1).astype(np.float32)
    h[:, 0] = 1.0
    w[:, 0] = 0.0
    w[[300, 5, 900], 0] = 3.0
    h[2] = rng.standard_normal(64)
    hb, wb = o.f32_to_bf16_bits(h), o.f32_to_bf16_bits(w)
    np.savez_compressed(
        os.path.join(out_dir, "ref_elementwise.npz"), gate_up=gu,
        silu=bits_of(ref.silu_mul_split_packed(to_dev_bf16(gu))), a=a, b=b,
        residual=bits_of(ref.residual_add(to_dev_bf16(a), to_dev_bf16(b))), hidden=hb, lm_weight=wb,
        logits=bits_of(_bf16_linear(ref, hb, wb)),
        tokens=ref.lm_head_argmax_batched(to_dev_bf16(hb), to_dev_bf16(wb)).numpy())
    print("wrote", sorted(os.listdir(out_dir)))


def _bf16_linear(ref, hb, wb):
    import torch
    M, K = hb.shape
    out = torch.empty((M, wb.shape[0]), dtype=torch.bfloat16, device="cuda")
    ref.lib.bf16_linear(ref.handle, ref._p(out), ref._p(to_dev_bf16(hb)), ref._p(to_dev_bf16(wb)), None, M,
                        wb.shape[0], K)
    torch.cuda.synchronize()
    return out


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
