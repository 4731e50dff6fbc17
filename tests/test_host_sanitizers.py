"""The C++ host runtime (sequence packers, paged-KV scheduler) under AddressSanitizer +
UndefinedBehaviorSanitizer and under ThreadSanitizer: a standalone driver (no Python, no GPU) stresses
the packers on random inputs and the scheduler from a client thread and an engine thread at once."""
import os
import shutil
import subprocess

import pytest

HOST = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "areal_b200", "csrc", "host")
SRCS = ["selftest.cpp", "seqpack.cpp", "rollout_scheduler.cpp"]


@pytest.mark.parametrize("name,flags", [("asan_ubsan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]),
                                        ("tsan", ["-fsanitize=thread"])])
def test_host_runtime_under_sanitizers(tmp_path, name, flags):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / f"selftest_{name}")
    build = subprocess.run([cxx, "-std=c++17", "-O1", "-g", "-pthread", *flags, *SRCS, "-o", exe], cwd=HOST,
                           capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr.lower():
        pytest.skip(f"sanitizer runtime not available: {build.stderr[-200:]}")
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1",
               UBSAN_OPTIONS="print_stacktrace=1")
    for seed in ("1", "2"):
        run = subprocess.run([exe, seed], capture_output=True, text=True, timeout=600, env=env)
        assert run.returncode == 0, (run.stdout[-1500:], run.stderr[-3000:])
        assert "host selftest ok" in run.stdout
