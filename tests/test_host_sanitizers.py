"""The host runtime under ThreadSanitizer and AddressSanitizer: a native driver (csrc/host/sanitize_main.cc) runs
allocator storms, PEs as threads with per-thread contexts, atomics, collectives and the reverse-offload ring with
several producers; any report from the sanitizer fails the test."""
import os
import subprocess

import pytest

from roc_shmem_b200 import build


@pytest.mark.parametrize("kind", ["thread", "address"])
def test_host_runtime_is_clean_under_sanitizer(kind):
    try:
        exe = build.build_sanitizer_driver(kind)
    except RuntimeError as e:
        if "cannot find" in str(e) or "unrecognized" in str(e):
            pytest.skip(f"this toolchain has no -fsanitize={kind} runtime")
        raise
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 second_deadlock_stack=1", ASAN_OPTIONS="detect_leaks=1 abort_on_error=0")
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode == 0 and "SANITIZE_OK" in p.stdout, p.stdout[-2000:] + p.stderr[-6000:]
    assert "WARNING: ThreadSanitizer" not in p.stderr and "ERROR: AddressSanitizer" not in p.stderr, p.stderr[-6000:]
