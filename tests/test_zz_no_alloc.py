"""GPU: the allocation-free W4A4 entry point against the regular one.

glmasr_nvfp4_linear_noalloc exists for callers that cannot grow a device workspace when they
call -- typically the decode loop, which runs after the engine has given every free byte to the
paged-KV pool -- so its temporaries sit in a fixed array inside the library.  Both entry points
launch the same kernels, so their outputs must agree to the last bit; the array is shared by all
calls and keeps the previous call's bytes, hence two different calls in a row.
Collected last on purpose: a run that stops at the first failure has then run every other test.
"""
import numpy as np
import pytest
import torch

import fp4_oracle as o
from gpu_util import REL_TOL_TIGHT, bits_of, to_dev_bf16, to_dev_u8

pytestmark = pytest.mark.gpu


def _case(ops, M, N, K, seed):
    pw, sw, g = o.seeded_weight(N, K, seed)
    x = o.seeded_activation(M, K, seed + 1)
    isc = o.default_input_scale(x)
    xd, wd, sd = to_dev_bf16(x), to_dev_u8(pw), to_dev_u8(sw)
    want = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    assert ops.nvfp4_linear(want, xd, wd, sd, isc, g) == 0
    got = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    assert ops.nvfp4_linear_noalloc(got, xd, wd, sd, isc, g) == 0
    torch.cuda.synchronize()
    return bits_of(got), bits_of(want), o.nvfp4_linear(x, pw, sw, isc, g)


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    from glm_asr_stack_b200 import ops
    assert torch.cuda.is_available()
    # second call is smaller in every dimension, so stale bytes of the first would show
    for M, N, K, seed in [(256, 2048, 2048, 900), (130, 200, 512, 910)]:
        got, want, oracle = _case(ops, M, N, K, seed)
        assert o.rel_err(got, want) <= REL_TOL_TIGHT
        assert np.array_equal(got, want)
        assert o.rel_err(got, oracle) <= REL_TOL_TIGHT
    assert ops.status() == 0


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from glm_asr_stack_b200 import ops
    out = torch.full((8, 128), 3.0, dtype=torch.bfloat16, device="cuda")
    x = torch.zeros((8, 256), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((128, 128), dtype=torch.uint8, device="cuda")
    s = torch.zeros((128, 16), dtype=torch.uint8, device="cuda")
    lib = __import__("glm_asr_stack_b200._lib", fromlist=["load"]).load()
    import ctypes
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    assert lib.glmasr_nvfp4_linear_noalloc(P(out), P(x), P(w), P(s), 1.0, 1.0, 513, 128, 256) == -1     # M too large
    assert lib.glmasr_nvfp4_linear_noalloc(P(out), P(x), P(w), P(s), 1.0, 1.0, 8, 128, 8448) == -1      # K too large
    assert lib.glmasr_nvfp4_linear_noalloc(P(out), P(x), P(w), P(s), 1.0, 1.0, 8, 59264, 2048) == -1    # weight too large
    assert lib.glmasr_nvfp4_linear_noalloc(P(out), P(x), P(w), P(s), 0.0, 1.0, 8, 128, 256) == -1       # bad input_scale
    torch.cuda.synchronize()
    assert torch.all(out == 3.0)


def _cold_first_call():
    """Body of the child process below: the allocation-free entry point is the FIRST call this process makes
    into the library, so the look-up of its array, the kernels' shared-memory opt-in and the loading of the
    module that holds them all happen inside it."""
    from glm_asr_stack_b200 import ops
    M, N, K, seed = 96, 384, 512, 930
    pw, sw, g = o.seeded_weight(N, K, seed)
    x = o.seeded_activation(M, K, seed + 1)
    isc = o.default_input_scale(x)
    xd, wd, sd = to_dev_bf16(x), to_dev_u8(pw), to_dev_u8(sw)
    got = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    assert ops.launch_count() == 0
    assert ops.nvfp4_linear_noalloc(got, xd, wd, sd, isc, g) == 0
    torch.cuda.synchronize()
    assert ops.status() == 0                  # reads the status word inside the library image as well
    err = o.rel_err(bits_of(got), o.nvfp4_linear(x, pw, sw, isc, g))
    assert err <= REL_TOL_TIGHT, err
    print("COLD_OK", err)


def test_noalloc_as_the_first_library_call_of_a_process():
    import os
    import subprocess
    import sys
    from conftest import ROOT
    code = ("import sys; sys.path[:0]=[%r,%r,%r]; import test_zz_no_alloc as t; t._cold_first_call()"
            % (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "COLD_OK" in r.stdout
