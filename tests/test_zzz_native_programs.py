"""The stand-alone C++ test program (csrc/tests/native_check.cu): it builds against the library without Python, skips
itself on a machine without a GPU, and on a B200 every case passes."""
import subprocess

import pytest
import torch

from tensorsharp_b200.ops import native


def _exe():
    exes = {p.name: p for p in native.build_tests()}
    assert "native_check" in exes
    return str(exes["native_check"])


def test_native_check_builds_and_skips_without_a_gpu():
    exe = _exe()
    bad = subprocess.run([exe, "8", "33"], capture_output=True, text=True, timeout=120)
    assert bad.returncode == 2 and "usage" in bad.stdout            # K must be whole blocks
    if torch.cuda.is_available():
        pytest.skip("GPU present: covered by the gpu test")
    p = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert p.returncode == 77 and "SKIP" in p.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [("512", "1024"), ("300", "4096")])
def test_native_check_passes_on_the_gpu(shape):
    p = subprocess.run([_exe(), *shape], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "FAIL" not in p.stdout and p.stdout.strip().endswith("OK"), p.stdout + p.stderr
