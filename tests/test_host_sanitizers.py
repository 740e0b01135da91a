"""The C++ host under AddressSanitizer and UndefinedBehaviorSanitizer.

The host library is built once more with `-fsanitize=address,undefined` (the kernels' objects are taken over as they
are) into a temporary folder, and the host-side tests of configuration, weights, cache manager, scheduler and logging
run against it in a child process with the sanitizers' runtimes loaded first.  A heap overflow, a use after free, a
signed overflow or a misaligned access anywhere on those paths ends the child with a report.  Skipped where the
compiler has no sanitizer runtimes."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FILES = ["test_cache.py", "test_scheduler.py", "test_weights.py", "test_config.py", "test_logging.py"]


def _runtime(cxx: str, name: str):
    try:
        path = subprocess.run([cxx, f"-print-file-name={name}"], capture_output=True, text=True, timeout=30).stdout.strip()
    except (OSError, subprocess.TimeoutExpired):
        return None
    return path if os.path.isabs(path) and os.path.isfile(path) else None


def _compiler_with_runtimes():
    for cxx in ("/usr/bin/g++", shutil.which("g++"), shutil.which("c++")):
        if cxx and os.path.isfile(cxx):
            asan, ubsan = _runtime(cxx, "libasan.so"), _runtime(cxx, "libubsan.so")
            if asan and ubsan:
                return cxx, asan, ubsan
    return None


def test_host_side_tests_pass_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    found = _compiler_with_runtimes()
    if found is None:
        pytest.skip("no C++ compiler with libasan.so and libubsan.so here")
    if os.environ.get("LIYAB_B200_SANITIZE"):
        pytest.skip("already running under the sanitizers")
    cxx, asan, ubsan = found
    env = dict(os.environ, LIYAB_B200_SANITIZE="address,undefined", LIYAB_CXX=cxx, LIYAB_B200_BUILD_DIR=str(tmp_path / "build"),
               LD_PRELOAD=f"{asan} {ubsan}", ASAN_OPTIONS="detect_leaks=0:halt_on_error=1",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider", "-m", "not gpu"] + [os.path.join("tests", f) for f in FILES]
    proc = subprocess.run(cmd, cwd=REPO, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    tail = proc.stdout[-6000:]
    assert proc.returncode == 0, tail
    assert "runtime error" not in proc.stdout and "AddressSanitizer" not in proc.stdout, tail
    assert " passed" in proc.stdout, tail
