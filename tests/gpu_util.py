"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import ctensor_b200 as ct
from oracle_lib import HostView


def to_device(hv: HostView, device="cuda:0") -> ct.DView:
    """Upload the whole storage buffer of a HostView; keep offset/shape/strides."""
    buf = torch.from_numpy(np.ascontiguousarray(hv.buf)).to(device)
    return ct.DView(buf, tuple(hv.shape), tuple(hv.strides), hv.offset)


def bits(a: np.ndarray) -> np.ndarray:
    if a.dtype == np.float32:
        return a.view(np.uint32)
    if a.dtype == np.float64:
        return a.view(np.uint64)
    return a


def assert_bits_equal(got, ref: np.ndarray, what="", nan_payload_free=True):
    """Bit-exact comparison; NaNs compare equal to NaNs whatever their payload (x86 and the GPU
    propagate different payloads)."""
    got = got.detach().cpu().numpy() if isinstance(got, torch.Tensor) else got
    assert got.shape == ref.shape, f"{what}: shape {got.shape} != {ref.shape}"
    if got.dtype.kind == "f" and nan_payload_free:
        gn, rn = np.isnan(got), np.isnan(ref)
        assert np.array_equal(gn, rn), f"{what}: NaN positions differ"
        ok = np.array_equal(bits(got)[~gn], bits(ref)[~rn])
    else:
        ok = np.array_equal(bits(got), bits(ref))
    if not ok:
        bad = np.flatnonzero((bits(got) != bits(ref)).reshape(-1))
        i = bad[0]
        raise AssertionError(f"{what}: {bad.size} of {got.size} elements differ; first at {i}: "
                             f"got {got.reshape(-1)[i]!r} want {ref.reshape(-1)[i]!r}")


def assert_close(got, ref: np.ndarray, rtol=1e-5, what="", atol=0.0):
    got = got.detach().cpu().numpy() if isinstance(got, torch.Tensor) else got
    assert got.shape == ref.shape, f"{what}: shape {got.shape} != {ref.shape}"
    np.testing.assert_allclose(got, ref, rtol=rtol, atol=atol, err_msg=what, equal_nan=True)
