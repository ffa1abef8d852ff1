"""Compile-only check of the class layer's interface: a caller written in the style of code that targets the
upstream project's headers (tests/api_compile/reference_style_user.cu) must compile against deepfuse_b200/dnn
with nothing but the include path changed.  nvcc cross-compiles for sm_100a without a GPU."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "api_compile" / "reference_style_user.cu"


def test_reference_style_caller_compiles(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc not found")
    cmd = [nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(ROOT / "deepfuse_b200"),
           "-I", str(ROOT / "include"), "-c", str(SRC), "-o", str(tmp_path / "user.o")]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert proc.returncode == 0, proc.stdout
