"""Host-side native code under AddressSanitizer + UndefinedBehaviorSanitizer."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.skipif(shutil.which("g++") is None, reason="g++ not available")
def test_cpu_library_is_clean_under_asan_ubsan(tmp_path):
    exe = tmp_path / "sanitize_main"
    srcs = [str(ROOT / "tests/native/sanitize_main.cpp")] + \
        [str(p) for p in sorted((ROOT / "csrc/cpu").glob("*.cpp"))]
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
           "-ffp-contract=off", "-I", str(ROOT / "csrc/include"), "-o", str(exe)] + srcs
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    assert "sanitize ok" in r.stdout
