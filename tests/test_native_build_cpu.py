"""The C++ side without Python in the loop: the CMake project builds the host runtime and the demo program of
examples/native_demo.cpp, the demo passes its own checks, and the public header declares every exported function of the
runtime."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("cmake") is None, reason="cmake not installed")
def test_cmake_builds_the_host_runtime_and_the_demo_runs(tmp_path):
    build = str(tmp_path / "b")
    cfg = subprocess.run(["cmake", "-S", ROOT, "-B", build, "-DLT_BUILD_CUDA=OFF", "-DLT_OUTPUT_DIR=" + build + "/lib"],
                         capture_output=True, text=True, timeout=300)
    assert cfg.returncode == 0, cfg.stdout[-2000:] + cfg.stderr[-2000:]
    mk = subprocess.run(["cmake", "--build", build, "-j", "4"], capture_output=True, text=True, timeout=900)
    assert mk.returncode == 0, mk.stdout[-3000:] + mk.stderr[-3000:]
    assert os.path.exists(os.path.join(build, "lib", "liblt_host.so"))
    run = subprocess.run([os.path.join(build, "lt_native_demo"), str(tmp_path)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "all checks passed" in run.stdout, run.stdout + run.stderr


def test_the_public_header_declares_every_exported_function():
    header = open(os.path.join(ROOT, "csrc", "runtime", "lt_host.h")).read()
    declared = set(re.findall(r"\b(lt_[a-z0-9_]+)\(", header))
    defined = set()
    for name in os.listdir(os.path.join(ROOT, "csrc", "runtime")):
        if name.endswith(".cpp"):
            src = open(os.path.join(ROOT, "csrc", "runtime", name)).read()
            assert '#include "lt_host.h"' in src, name          # a drifting definition then fails to compile
            defined |= set(re.findall(r"^[A-Za-z_][A-Za-z0-9_ ]*\**\s+(lt_[a-z0-9_]+)\([^;{]*\)\s*\{", src, re.M))
    assert defined and defined <= declared, sorted(defined - declared)
    # and the library really exports them
    from litetorch_b200._native import host_lib
    lib = host_lib()
    for fn in sorted(declared):
        assert hasattr(lib, fn), fn


def test_the_device_library_header_covers_every_bound_kernel_and_is_plain_c(tmp_path):
    header_path = os.path.join(ROOT, "csrc", "kernels", "lt_cuda.h")
    header = open(header_path).read()
    declared = set(re.findall(r"\b(lt_[a-z0-9_]+)\(", header))
    bound = set(re.findall(r'"(lt_[a-z0-9_]+)"', open(os.path.join(ROOT, "litetorch_b200", "ops", "kernels.py")).read()))
    assert bound and bound <= declared, sorted(bound - declared)
    for folder, inc in (("kernels", '#include "lt_cuda.h"'), ("kernels/common", '#include "lt_cuda.h"'),
                        ("cuda_runtime", '#include "kernels/lt_cuda.h"')):
        for name in os.listdir(os.path.join(ROOT, "csrc", folder)):
            if name.endswith(".cu"):
                assert inc in open(os.path.join(ROOT, "csrc", folder, name)).read(), name
    # usable from a host compiler without the CUDA toolkit's headers, as C and as C++
    for ext, cc in ((".c", "gcc"), (".cpp", "g++")):
        if shutil.which(cc) is None:
            continue
        src = tmp_path / ("use" + ext)
        src.write_text('#include "lt_cuda.h"\n#include "lt_host.h"\nint main(void) { return lt_pool_threads() < 0; }\n')
        r = subprocess.run([cc, "-fsyntax-only", "-I", os.path.join(ROOT, "csrc", "kernels"), "-I",
                            os.path.join(ROOT, "csrc", "runtime"), str(src)], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr[-2000:]


def _build_libtorch_example(tmp_path):
    import torch
    from torch.utils.cpp_extension import include_paths
    from litetorch_b200 import _native
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    lt_dir = os.path.join(ROOT, "litetorch_b200", "_lib")
    if not os.path.exists(os.path.join(lt_dir, "liblt_cuda.so")):
        _native.build_cuda()
    exe = str(tmp_path / "lt_libtorch_linear")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    cmd = (["g++", "-std=c++17", "-O1"] + ["-I" + p for p in include_paths("cuda")] + ["-I" + cuda_inc,
           "-I" + os.path.join(ROOT, "csrc", "kernels"), os.path.join(ROOT, "examples", "libtorch_linear.cpp"),
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI), "-L" + lib_dir, "-L" + lt_dir,
           "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-llt_cuda",
           "-Wl,-rpath," + lib_dir, "-Wl,-rpath," + lt_dir, "-o", exe])
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-4000:]
    return exe


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir("/usr/local/cuda/include"), reason="needs g++ and the CUDA headers")
def test_libtorch_example_compiles_and_links_against_the_device_library(tmp_path):
    """examples/libtorch_linear.cpp: libtorch as the tensor layer, `lt_gemm_bf16` for the math.  Without a GPU the program
    says so and exits 0; tests/test_zzz_libtorch_example_gpu.py runs it on a device."""
    exe = _build_libtorch_example(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
