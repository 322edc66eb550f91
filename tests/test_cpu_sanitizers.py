"""The host runtime under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer: the
self-test driver exercises every exported entry point (multi-threaded blob reads included)."""
import shutil
import subprocess

import pytest

from momijo_b200._C import build


@pytest.mark.parametrize("kind", ["asan_ubsan", "tsan"])
def test_host_runtime_selftest_under_sanitizer(tmp_path, kind):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = build.build_sanitized(kind, out_dir=tmp_path)
    env = {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "halt_on_error=1",
           "TSAN_OPTIONS": "halt_on_error=1", "PATH": "/usr/bin:/bin"}
    r = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    assert "selftest ok" in r.stdout
    assert "ERROR: " not in r.stderr and "WARNING: ThreadSanitizer" not in r.stderr, r.stderr[-3000:]
