"""The host runtime's shared structures (memory pool, LRU list, thread pool, TCP store) under AddressSanitizer +
UndefinedBehaviorSanitizer and under ThreadSanitizer: the stress driver of tests/native is compiled together with the
runtime sources and must exit 0 with no sanitizer report."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCES = [os.path.join(ROOT, "csrc", "runtime", f) for f in ("threadpool.cpp", "allocator.cpp", "store.cpp")]
DRIVER = os.path.join(ROOT, "tests", "native", "runtime_stress.cpp")


@pytest.mark.parametrize("flags,env", [
    (["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0"}),
    (["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=1"}),
])
def test_runtime_stress_under_sanitizers(tmp_path, flags, env):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "runtime_stress")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-pthread"] + flags + [DRIVER] + SOURCES + ["-o", exe]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if b.returncode != 0 and "sanitize" in b.stderr and "cannot find" in b.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert b.returncode == 0, b.stderr[-3000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=dict(os.environ, **env))
    assert r.returncode == 0 and "OK" in r.stdout, (r.stdout[-1000:], r.stderr[-4000:])
    assert "Sanitizer" not in r.stderr, r.stderr[-4000:]
