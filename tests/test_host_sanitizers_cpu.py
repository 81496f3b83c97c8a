"""The library's host-only C++ (the per-thread error channel, csrc/error.cpp) under AddressSanitizer and
UndefinedBehaviorSanitizer: built with g++ here, no GPU involved.  Device code is checked by other means (bounded
waits with status words, index checks before launches, canaries)."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

CSRC = Path(__file__).resolve().parents[1] / "tensorsharp_b200" / "csrc"
FLAGS = ["-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-fno-omit-frame-pointer", "-pthread"]


def _cuda_include():
    for d in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if d and (Path(d) / "include" / "cuda_runtime.h").exists():
            return str(Path(d) / "include")
    return None


def test_error_channel_under_asan_and_ubsan(tmp_path):
    gxx, inc = shutil.which("g++"), _cuda_include()
    if gxx is None or inc is None:
        pytest.skip("needs g++ and the CUDA headers")
    probe = tmp_path / "probe.cpp"
    probe.write_text("int main() { return 0; }\n")
    if subprocess.run([gxx, *FLAGS, str(probe), "-o", str(tmp_path / "probe")], capture_output=True).returncode != 0:
        pytest.skip("this g++ has no sanitizer runtime")
    exe = tmp_path / "host_check"
    build = subprocess.run([gxx, *FLAGS, "-I", inc, str(CSRC / "error.cpp"), str(CSRC / "tests" / "host_check.cpp"), "-o", str(exe)],
                           capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    env.pop("TSB_DISABLE_PDL", None)
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120, env=env)
    assert run.returncode == 0 and run.stdout.strip().endswith("OK"), run.stdout + run.stderr[-3000:]
    assert "runtime error" not in run.stderr and "AddressSanitizer" not in run.stderr, run.stderr[-3000:]
    off = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120, env=dict(env, TSB_DISABLE_PDL="1"))
    assert off.returncode == 0, off.stdout + off.stderr[-2000:]
