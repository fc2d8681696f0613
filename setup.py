"""Build script: `pip install .` (or `python setup.py build_py`) compiles the two native libraries in-tree first -
`liblt_cuda.so` with nvcc for sm_100a (`-gencode arch=compute_100a,code=sm_100a`) and `liblt_host.so` with g++ - and
ships them as package data under `litetorch_b200/_lib`.  The reference builds one pybind11 module plus a dlopen'ed GPU
library from its setup.py (setup.py:21-143); here the Python side binds plain C symbols through ctypes, so no
extension module is compiled against the Python headers."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class BuildNativeThenPy(build_py):
    def run(self):
        from litetorch_b200 import _native
        _native.build_all(verbose=True)
        super().run()


setup(cmdclass={"build_py": BuildNativeThenPy})
