"""The C++ host layer (ctensor_b200/host): it must compile and link everywhere (CPU test) and
its known-answer program — written like the reference's test/test_ops.cpp — must pass on a GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "ctensor_b200")
EXE = os.path.join(ROOT, "tests", "cpp", "test_host_api.bin")


def _build():
    from ctensor_b200 import build as b
    b.build()
    b.build_host()
    src = os.path.join(ROOT, "tests", "cpp", "test_host_api.cpp")
    if not os.path.exists(EXE) or os.path.getmtime(EXE) < max(os.path.getmtime(src), os.path.getmtime(b.HOST_LIB)):
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-o", EXE, src,
                               "-I", os.path.join(PKG, "host", "include"), "-L", PKG, "-lctensor_host", "-lctb200",
                               f"-Wl,-rpath,{PKG}"])
    return EXE


def test_host_layer_compiles_and_links():
    assert os.path.exists(_build())


def test_host_layer_refuses_to_run_without_gpu():
    import ctensor_b200
    if ctensor_b200.lib().ctb_device_count() > 0:
        pytest.skip("a CUDA device is present")
    r = subprocess.run([_build()], capture_output=True, text=True)
    assert r.returncode != 0 and "no CUDA device" in (r.stderr + r.stdout)


@pytest.mark.gpu
def test_host_layer_known_answers():
    r = subprocess.run([_build()], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ALL PASSED" in r.stdout
