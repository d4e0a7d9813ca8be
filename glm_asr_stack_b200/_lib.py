"""ctypes loader for ``libglmasr_fp4.so`` (the C-ABI library built from ``csrc/``).

There is no CPU fallback and no alternative backend: if the shared library is missing or
does not export a symbol that ``include/glmasr_fp4.h`` declares, importing fails loudly.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libglmasr_fp4.so")


class Fp4Weight(Structure):
    """``glmasr_fp4_weight`` of include/glmasr_fp4.h."""

    _fields_ = [("w_packed", c_void_p), ("w_scales", c_void_p), ("w_global_scale", c_float), ("N", c_int)]


class LayerWeights(Structure):
    """``glmasr_layer_weights`` of include/glmasr_fp4.h."""

    _fields_ = [("q", Fp4Weight), ("k", Fp4Weight), ("v", Fp4Weight), ("o", Fp4Weight),
                ("gate", Fp4Weight), ("up", Fp4Weight), ("down", Fp4Weight),
                ("in_qkv", c_float), ("in_o", c_float), ("in_gate_up", c_float), ("in_down", c_float),
                ("hidden", c_int), ("ffn", c_int)]


P = c_void_p
#: symbol -> (restype, argtypes); must list every function include/glmasr_fp4.h declares
SIGNATURES = {
    "fp4_dequant_to_bf16": (None, [P, P, P, c_float, c_int, c_int]),
    "fp4_linear": (None, [P, P, P, P, P, P, P, c_float, P, P, c_int, c_int, c_int]),
    "nvfp4_cutlass_available": (c_int, []),
    "nvfp4_linear": (c_int, [P, P, P, P, P, P, c_float, c_float, P, P, c_int, c_int, c_int]),
    "bf16_linear": (None, [P, P, P, P, P, c_int, c_int, c_int]),
    "silu_mul_split_packed": (None, [P, P, c_int, c_int]),
    "silu_elementwise_mul": (None, [P, P, c_int]),
    "residual_add": (None, [P, P, P, c_int]),
    "lm_head_argmax_batched": (None, [P, P, P, c_int, c_int, c_int, P]),
    "lm_head_cleanup": (None, []),
    "rmsnorm": (None, [P, P, P, c_float, c_int, c_int]),
    "embedding_lookup": (None, [P, P, P, c_int, c_int]),
    "reshape_and_cache": (None, [P, P, P, P, P, c_int, c_int, c_int, c_int]),
    "paged_decode_attention": (None, [P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int]),
    "decoder_decode_step_batched": (None, [P, P, P, P, P, P, P, c_int, P, P, P]),
    "decoder_prefill_paged_batched": (None, [P, P, P, c_int, c_int, P, P, P, P, P, P]),
    "flash_fwd_vllm_gqa_available": (c_int, []),
    "flash_fwd_vllm_gqa_launch": (c_int, [P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, c_int]),
    "layernorm": (None, [P, P, P, P, c_float, c_int, c_int]),
    "gelu_inplace": (None, [P, c_int]),
    "rope_encoder": (None, [P, P, c_int, c_int, c_int, c_float]),
    "residual_add_bias": (None, [P, P, P, P, c_int, c_int]),
    "concat_4frames": (None, [P, P, c_int, c_int]),
    "conv1d_forward": (None, [P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int]),
    "transpose_2d": (None, [P, P, c_int, c_int]),
    "bf16_linear_gelu": (None, [P, P, P, P, P, c_int, c_int, c_int]),
    "encoder_forward": (None, [P, P, P, c_int, P]),
    "encoder_forward_packed": (None, [P, P, P, c_int, c_int, P, P, P]),
    "encoder_cleanup": (None, []),
    "glmasr_audio_encode_batched": (c_int, [P, P, P, c_longlong, P, c_int, P, c_longlong, P]),
    "mel_spectrogram": (None, [P, c_int, P, P, P]),
    "mel_cleanup": (None, []),
    "glmasr_mel_spectrogram_batched": (c_int, [P, c_longlong, P, c_int, P, P, c_longlong, c_int, P]),
    "safetensors_load": (c_int, [ctypes.c_char_p, P]),
    "safetensors_free": (None, [P]),
    "glmasr_safetensors_inspect": (c_int, [ctypes.c_char_p, P, POINTER(ctypes.c_size_t)]),
    "glmasr_safetensors_release_index": (None, [P]),
    "glmasr_rope_single_token": (None, [P, P, c_int, c_int, c_int]),
    "glmasr_rope_qk_cache": (c_int, [P, c_int, c_int, c_int, P, P, P, P, c_int, c_int, c_int, c_int]),
    "glmasr_rmsnorm_quant": (c_int, [P, P, P, P, c_float, c_float, c_int, c_int]),
    "glmasr_decode_layer_tail": (c_int, [P, c_int, P, P, P, P, P, P, P, P, P, P, P, c_int]),
    "glmasr_fp4_linear_quantized": (c_int, [c_int, P, c_int, P, P, P, c_int, c_float, c_int, P, c_int, c_int, P, P, c_float]),
    "glmasr_decoder_forget_weights": (None, []),
    "glmasr_fp4_linear_fused": (c_int, [c_int, P, c_int, P, c_int, POINTER(Fp4Weight), c_int, c_float, P, P,
                                        c_int, P, c_int, c_int]),
    "glmasr_fp4_prepack": (c_int, [P, c_int, c_int]),
    "glmasr_fp4_forget": (None, [P]),
    "glmasr_quantize_bf16_to_fp4": (c_int, [P, P, P, P, c_float, c_int, c_int]),
    "glmasr_swizzle_rowwise_scales": (c_int, [P, P, c_int, c_int]),
    "glmasr_argmax_rows": (c_int, [P, P, c_int, c_int]),
    "glmasr_fp4_layer_proj": (c_int, [c_int, P, P, POINTER(LayerWeights), c_int]),
    "glmasr_fp4_layer_proj_host": (c_int, [c_int, P, P, POINTER(LayerWeights), c_int]),
    "glmasr_nvfp4_linear_noalloc": (c_int, [P, P, P, P, c_float, c_float, c_int, c_int, c_int]),
    "glmasr_fp4_status": (c_int, []),
    "glmasr_launch_count": (c_longlong, []),
    "glmasr_profile_enable": (None, [c_int]),
    "glmasr_profile_read": (c_int, [c_int, P, P, P]),
    "glmasr_set_stream": (None, [P]),
    "glmasr_fp4_cleanup": (None, []),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "or `make -C glm_asr_stack_b200/csrc` (there is no CPU or PyTorch fallback for this path)")
    lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_LOCAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the export is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
