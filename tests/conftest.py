import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    # The shared libraries are build products (not in the history): make a fresh checkout
    # testable.  nvcc cross-compiles sm_100a without a GPU; nothing is rebuilt when up to date.
    from ctensor_b200 import build as b
    b.build()
    b.build_host()
    b.build_gen1()


@pytest.fixture(scope="session")
def oracle():
    from oracle_lib import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The real reference compiled by oracle/build_ref.sh; skipped where it was not built."""
    from oracle_lib import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/libctensor_ref.so not built on this machine")
    ref = Reference()
    if not (ref.has_avx2 and ref.has_avx512):
        pytest.skip("host CPU lacks AVX2/AVX-512F needed by the reference's SIMD back-ends")
    return ref


@pytest.fixture(scope="session")
def ct():
    """The product binding, with the library loaded and a CUDA device present."""
    import torch
    import ctensor_b200
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    ctensor_b200.lib()
    return ctensor_b200
