"""B200-native (sm_100a) drop-in for the FP4-weight linear path of the GLM-ASR Infer-engine.

``ops``      the reference operator interface (fp4_linear, nvfp4_linear, ...) on torch CUDA tensors
``weights``  WeightStore + linear_proj dispatcher mirror
``synth``    seeded synthetic FP4 weights / activations for tests and benchmarks
``_lib``     ctypes binding of libglmasr_fp4.so (include/glmasr_fp4.h); no fallback exists
"""
from . import _lib  # noqa: F401

__all__ = ["ops", "weights", "synth", "_lib"]
