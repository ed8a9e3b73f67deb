"""CPU: the library's host side (argument checks, size and chunk arithmetic, error strings) under
AddressSanitizer and UndefinedBehaviorSanitizer.

The host-only ABI tests run once more in a child interpreter that preloads the sanitizer runtimes and
loads a build of the library whose host code is instrumented.  Any report fails the test."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _runtime(name):
    r = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True)
    path = r.stdout.strip()
    return path if r.returncode == 0 and os.path.isabs(path) and os.path.exists(path) else None


def test_host_side_is_clean_under_asan_and_ubsan():
    asan, ubsan = _runtime("libasan.so"), _runtime("libubsan.so")
    if asan is None or ubsan is None:
        pytest.skip("gcc's sanitizer runtimes are not installed")
    from moe_gen_b200.build import build_sanitized_library
    lib = build_sanitized_library()
    env = dict(os.environ, LD_PRELOAD=f"{asan}:{ubsan}", MOEGEN_B200_LIB=lib,
               ASAN_OPTIONS="detect_leaks=0:halt_on_error=1", UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_abi_cpu.py"), "-x", "-q",
                        "-p", "no:cacheprovider"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    out = r.stdout + r.stderr
    assert "AddressSanitizer" not in out and "runtime error:" not in out, out[-4000:]
    assert r.returncode == 0, out[-4000:]
    assert " passed" in out
