"""Runs the C++ drop-in test (tests/cpp/dropin_test.cpp): the reference's operator signatures
(Kokkos::View arguments, exceptions, decline -> fallback) on top of the C ABI, on the GPU."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def test_cpp_dropin_layer(kd):
    import __graft_entry__ as ge
    exe = ge.build_cpp_dropin_test()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "all checks passed" in res.stdout
