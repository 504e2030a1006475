"""The C++ host runtime compiled with AddressSanitizer + UndefinedBehaviorSanitizer and driven by a
small C++ program (random packing problems, delta encode / apply round trips, truncated streams)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_host_runtime_is_clean_under_asan_and_ubsan(tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("g++ not available")
    host = os.path.join(ROOT, "xorl_b200", "csrc", "host")
    srcs = [os.path.join(host, f) for f in sorted(os.listdir(host)) if f.endswith(".cpp")]
    exe = str(tmp_path / "host_sanitize")
    cmd = [cxx, "-O1", "-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
           "-fno-omit-frame-pointer", "-pthread", "-o", exe,
           os.path.join(ROOT, "tests", "native", "host_sanitize_main.cpp"), *srcs]
    b = subprocess.run(cmd, capture_output=True, text=True)
    if b.returncode != 0 and "asan" in (b.stderr + b.stdout).lower() and "cannot find" in b.stderr:
        pytest.skip("sanitizer runtime libraries not installed")
    assert b.returncode == 0, b.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    env.pop("LD_PRELOAD", None)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-4000:])
    assert "clean under asan+ubsan" in r.stdout
