"""CPU tests of the C-ABI library: it loads, exports every symbol the header declares, and its
host-side validation answers with the reference's error texts (no compute call needs a GPU)."""
import ctypes
import os
import re

import numpy as np
import pytest

import ctensor_b200 as ct

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    return ct.lib()


def test_header_symbols_exported(L):
    header = open(os.path.join(ROOT, "include", "ctb200.h")).read()
    declared = sorted(set(re.findall(r"\b(ctb_[a-z0-9_]+)\s*\(", header)))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(L, name), f"{name} declared in ctb200.h but not exported"
    assert sorted(ct.EXPORTED_SYMBOLS) == declared


def test_version_and_struct_layout(L):
    assert L.ctb_abi_version() == 1
    assert ctypes.sizeof(ct.View) == 8 + 8 + 4 + 4 + 8 * 8 + 8 * 8


def _host_view(arr):
    return ct.make_view(arr.ctypes.data, ct.F32, arr.shape, [s // 4 for s in arr.strides])


def test_null_and_shape_errors_match_reference_messages(L):
    a = np.zeros((4, 3), np.float32)
    b = np.zeros((4, 2), np.float32)
    o = np.zeros((4, 3), np.float32)
    va, vb, vo = _host_view(a), _host_view(b), _host_view(o)
    assert L.ctb_binary(ct.ADD, None, vb, vo, None) == 1
    assert L.ctb_last_error() == b"binary_op: null input"            # src/core/opsmp.cpp:138
    assert L.ctb_binary(ct.ADD, va, vb, vo, None) == 2
    assert L.ctb_last_error() == b"Shape mismatch in binary op"      # src/core/opsmp.cpp:144
    assert L.ctb_unary(ct.RELU, None, 0.0, vo, None) == 1
    assert L.ctb_last_error() == b"unary_op: null input"             # src/core/opsmp.cpp:274
    assert L.ctb_reduce(ct.SUM, None, 0, vo, None) == 1
    assert L.ctb_last_error() == b"reduction: null input"            # src/core/opsmp.cpp:595
    assert L.ctb_reduce(ct.ARGMAX, va, 5, vo, None) == 4
    assert L.ctb_last_error() == b"argmax: dim out of range"         # src/core/ops_dispatch.cpp:433
    assert L.ctb_binary(99, va, va, vo, None) == 5
    bad = _host_view(a)
    bad.dtype = 11
    assert L.ctb_binary(ct.ADD, bad, bad, vo, None) == 3


def test_output_checks(L):
    a = np.zeros((4, 3), np.float32)
    o = np.zeros((5, 3), np.float32)
    assert L.ctb_unary(ct.RELU, _host_view(a), 0.0, _host_view(o), None) == 2
    ot = np.zeros((3, 4), np.float32).T            # right size, not contiguous
    assert L.ctb_unary(ct.RELU, _host_view(a), 0.0, _host_view(ot), None) == 2
    assert b"contiguous" in L.ctb_last_error()


def test_no_cpu_fallback(L):
    """Without a CUDA device a well-formed call must fail loudly, not compute on the host."""
    if L.ctb_device_count() > 0:
        pytest.skip("a CUDA device is present")
    a = np.ones((8,), np.float32)
    o = np.full((8,), 7.0, np.float32)
    st = L.ctb_unary(ct.RELU, _host_view(a), 0.0, _host_view(o), None)
    assert st == 6 and b"CUDA" in L.ctb_last_error()
    assert np.all(o == 7.0)
    with pytest.raises(ct.CtbError):
        ct.check(st)


def test_no_cpu_fallback_for_the_caller_side_entry_points(L):
    """matmul, cat, accumulate_grad, gather, optimizer steps, BatchNorm and the fused rows also
    refuse to run without a CUDA device and leave their outputs untouched."""
    if L.ctb_device_count() > 0:
        pytest.skip("a CUDA device is present")
    a = np.ones((8, 8), np.float32)
    o = np.full((8, 8), 7.0, np.float32)
    idx = np.zeros((8, 1), np.int32)
    oi = np.full((8, 1), 7.0, np.float32)
    vi = ct.make_view(idx.ctypes.data, ct.I32, idx.shape, [1, 1])
    va, vo = _host_view(a), _host_view(o)
    views = (ctypes.POINTER(ct.View) * 1)(ctypes.pointer(va))
    calls = [
        lambda: L.ctb_matmul(va, va, vo, None),
        lambda: L.ctb_cat(views, 1, 0, vo, None),
        lambda: L.ctb_accumulate_grad(vo, va, None),
        lambda: L.ctb_gather(va, 1, vi, _host_view(oi), None, None),
        lambda: L.ctb_sgd_step(vo, va, 0.1, None),
        lambda: L.ctb_softmax_lastdim(va, None, 0, vo, None),
        lambda: L.ctb_log_softmax_lastdim(va, None, vo, None),
        lambda: L.ctb_layernorm_lastdim(va, None, None, 1e-5, vo, None),
        lambda: L.ctb_copy_into(va, vo, None),
    ]
    for i, call in enumerate(calls):
        assert call() == 6, (i, L.ctb_last_error())
    assert np.all(o == 7.0) and np.all(oi == 7.0)
