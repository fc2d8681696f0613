"""The host runtime (memory pool, LRU list, thread pool, TCP store; serving scheduler, prefix cache, data loader,
checkpoint files, JIT tree) under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer: the drivers
of tests/native are compiled together with the runtime sources and must exit 0 with no sanitizer report."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNTIME = os.path.join(ROOT, "csrc", "runtime")
DRIVERS = {
    "runtime_stress": ["threadpool.cpp", "allocator.cpp", "store.cpp"],
    "services_stress": ["scheduler.cpp", "dataloader.cpp", "tokenstream.cpp", "io.cpp", "jit.cpp", "threadpool.cpp", "allocator.cpp"],
}


@pytest.mark.parametrize("driver", sorted(DRIVERS))
@pytest.mark.parametrize("flags,env", [
    (["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0"}),
    (["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=1"}),
])
def test_runtime_stress_under_sanitizers(tmp_path, flags, env, driver):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path / driver)
    sources = [os.path.join(ROOT, "tests", "native", driver + ".cpp")] + [os.path.join(RUNTIME, f) for f in DRIVERS[driver]]
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-pthread"] + flags + sources + ["-o", exe]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if b.returncode != 0 and "sanitize" in b.stderr and "cannot find" in b.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert b.returncode == 0, b.stderr[-3000:]
    r = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True, timeout=600, env=dict(os.environ, **env))
    assert r.returncode == 0 and "OK" in r.stdout, (r.stdout[-1000:], r.stderr[-4000:])
    assert "Sanitizer" not in r.stderr, r.stderr[-4000:]
