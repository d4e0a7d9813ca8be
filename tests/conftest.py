import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def reference_root():
    """Directory of the reference project (the one that holds Infer-engine/), or None.  GLMASR_REFERENCE_ROOT names
    it; by default it is looked for beside this repository."""
    cand = os.environ.get("GLMASR_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
    return cand if os.path.isdir(os.path.join(cand, "Infer-engine", "include")) else None


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle_libs():
    """Build (if needed) the test-only checker libraries under oracle/."""
    odir = os.path.join(ROOT, "oracle")
    need = [os.path.join(odir, "libfp4_oracle.so"), os.path.join(odir, "libnv_cvt_host.so")]
    if not all(os.path.exists(p) for p in need):
        subprocess.run(["make", "-C", odir, need[0], need[1]], check=True, capture_output=True)
    return {"c": need[0], "nv": need[1]}


@pytest.fixture(scope="session")
def product_lib():
    """libglmasr_fp4.so must exist; build it if the tree is fresh."""
    lib = os.path.join(ROOT, "glm_asr_stack_b200", "libglmasr_fp4.so")
    if not os.path.exists(lib):
        subprocess.run(["make", "-C", os.path.join(ROOT, "glm_asr_stack_b200", "csrc")], check=True,
                       capture_output=True)
    return lib
