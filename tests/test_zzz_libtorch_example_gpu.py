"""examples/libtorch_linear.cpp on a device: the C++ program's GEMM (bias and GELU in the epilogue) agrees with libtorch's
own matmul and the status word stays clear."""
import os
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir("/usr/local/cuda/include"), reason="needs g++ and the CUDA headers")
def test_cpp_program_on_libtorch_and_the_device_library(tmp_path):
    from test_native_build_cpu import _build_libtorch_example
    exe = _build_libtorch_example(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "device status 0" in r.stdout, r.stdout + r.stderr
