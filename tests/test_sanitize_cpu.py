"""Host runtime under AddressSanitizer + UBSan: the C++ self-test is compiled together with the
runtime sources with -fsanitize=address,undefined and must exit cleanly (no leaks, overflows or UB)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "kharon_b200", "csrc", "runtime")


def test_runtime_selftest_under_asan_ubsan(tmp_path):
    exe = str(tmp_path / "rt_selftest")
    b = None
    for cand in ("/usr/bin/g++", "g++", os.environ.get("CXX", "")):      # the first one that ships libasan
        cxx = shutil.which(cand) if cand else None
        if not cxx:
            continue
        cmd = [cxx, "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-o", exe,
               os.path.join(SRC, "rt_selftest.cpp"), os.path.join(SRC, "kharon_rt.cpp")]
        b = subprocess.run(cmd, capture_output=True, text=True)
        if b.returncode == 0:
            break
    if b is None or (b.returncode != 0 and "asan" in (b.stderr + b.stdout).lower()):
        pytest.skip("no compiler with the sanitizer runtime")
    assert b.returncode == 0, b.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="halt_on_error=1")
    r = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "runtime selftest ok" in r.stdout, (r.stdout[-500:], r.stderr[-3000:])
