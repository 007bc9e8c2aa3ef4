"""The host runtime (cache manager and scheduler, csrc/cache_runtime.cpp and csrc/scheduler_runtime.cpp) compiled with the
address and undefined-behaviour sanitizers, and the tests that drive it (random orders of calls against the Python twins,
the golden batches, the engine loop) run against that build in a child process.  A heap overflow, a use after free or an
undefined operation in the C++ code ends the child with the sanitizer's report."""
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "cppvllm_b200", "csrc")


def _file_of(compiler, name):
    out = subprocess.run([compiler, f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip()
    return out if os.path.isabs(out) and os.path.isfile(out) else None


def test_host_runtime_is_clean_under_the_sanitizers(tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++ on this machine")
    asan, ubsan = _file_of(cxx, "libasan.so"), _file_of(cxx, "libubsan.so")
    if asan is None or ubsan is None:
        pytest.skip("this g++ has no sanitizer runtimes")
    so = str(tmp_path / "libcvb_runtime_san.so")
    build = subprocess.run([cxx, "-std=c++17", "-O1", "-g", "-fPIC", "-shared", "-fsanitize=address,undefined",
                            "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-I", SRC,
                            os.path.join(SRC, "cache_runtime.cpp"), os.path.join(SRC, "scheduler_runtime.cpp"), "-o", so],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, CVB_LIBRARY_RUNTIME=so, LD_PRELOAD=f"{asan}:{ubsan}",
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    run = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "not gpu", "-p", "no:cacheprovider",
                          os.path.join(ROOT, "tests", "test_cache_native.py"), os.path.join(ROOT, "tests", "test_scheduler_native.py"),
                          os.path.join(ROOT, "tests", "test_scheduler.py"), os.path.join(ROOT, "tests", "test_engine_loop.py")],
                         capture_output=True, text=True, env=env, cwd=ROOT, timeout=900)
    tail = (run.stdout + run.stderr)[-4000:]
    assert run.returncode == 0, tail
    assert "passed" in run.stdout and "ERROR: AddressSanitizer" not in tail and "runtime error" not in tail, tail
