"""The C++ runtime core under AddressSanitizer + UBSan and under ThreadSanitizer (host only): block pool / table,
batch scheduler with concurrent submitters and cancellation, command channel between threads, JSON parser on hostile
input, host sampler, HTTP server under hostile and concurrent requests, file readers on damaged files, tokenizer; and
the AVX2 host kernels under AddressSanitizer + UBSan with every operand in a heap block of exactly its size.  Skipped
where the toolchain has no sanitizer runtime."""
import os
import subprocess

import pytest

from deepseek_v4_2080ti_b200 import build


@pytest.mark.parametrize("sanitizer", ["", "address", "thread"])
def test_core_selftest(sanitizer):
    try:
        exe = build.build_selftest(sanitizer)
    except RuntimeError:
        if sanitizer:
            pytest.skip(f"no {sanitizer} sanitizer runtime in this toolchain")
        raise
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="halt_on_error=1",
               TSAN_OPTIONS="halt_on_error=1")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "CORE_SELFTEST_OK" in r.stdout, (r.stdout[-500:], r.stderr[-3000:])
    assert "ERROR: AddressSanitizer" not in r.stderr and "WARNING: ThreadSanitizer" not in r.stderr and "runtime error" not in r.stderr


@pytest.mark.parametrize("sanitizer", ["", "address"])
def test_cpu_kernel_selftest(sanitizer):
    try:
        exe = build.build_cpu_selftest(sanitizer)
    except RuntimeError:
        if sanitizer:
            pytest.skip(f"no {sanitizer} sanitizer runtime in this toolchain")
        raise
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="halt_on_error=1")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "CPU_SELFTEST_OK" in r.stdout, (r.stdout[-500:], r.stderr[-3000:])
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr
