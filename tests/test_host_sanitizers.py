"""The host runtime's C++ under AddressSanitizer + UBSan and under ThreadSanitizer: `tests/host_walk.cpp`
(a random walk over scheduler, prefix cache, layout and the worker loop with client threads) is built
with g++ against the same sources the library is built from, and must run clean.  The reference leans on
Rust's ownership for this; the C++ port gets the sanitizers instead."""

import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "qwencore_b200", "csrc", "host")
SOURCES = [os.path.join(ROOT, "tests", "host_walk.cpp"), os.path.join(HOST, "runtime.cpp"),
           os.path.join(HOST, "worker.cpp")]


@pytest.mark.parametrize("sanitizers", ["address,undefined", "thread"])
def test_host_runtime_runs_clean_under_sanitizers(tmp_path, sanitizers):
    binary = str(tmp_path / "host_walk")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizers}", "-fno-sanitize-recover=all",
                            "-fno-omit-frame-pointer", "-I", HOST, "-I", os.path.join(ROOT, "include"), *SOURCES,
                            "-o", binary, "-lpthread"], capture_output=True, text=True)
    if build.returncode != 0 and ("cannot find -l" in build.stderr or "unrecognized" in build.stderr):
        pytest.skip(f"this g++ has no runtime for -fsanitize={sanitizers}")
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1",
               UBSAN_OPTIONS="print_stacktrace=1")
    run = subprocess.run([binary], capture_output=True, text=True, timeout=300, env=env)
    assert run.returncode == 0, (run.stdout[-1000:], run.stderr[-3000:])
    assert run.stdout.startswith("ok ") and "failed=0" in run.stdout
    assert "Sanitizer" not in run.stderr and "runtime error" not in run.stderr
