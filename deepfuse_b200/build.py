"""In-tree build of the native libraries (nvcc, sm_100a only).

    python -m deepfuse_b200.build            # build what is out of date
    python -m deepfuse_b200.build --force    # rebuild everything

Produces, under ``deepfuse_b200/lib/``:

* ``libdf8.so``      the C-ABI kernel library declared in ``include/df8.h``
* ``libdf8_dnn.so``  the C++17 ``dnn::`` classes built on it, plus the small C harness
                     (``include/df8_dnn.h``) that the Python tests and ``bench.py`` drive

nvcc cross-compiles for sm_100a without a GPU, so this runs anywhere the CUDA toolkit is installed.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
DNN = PKG / "dnn"
LIB = PKG / "lib"
OBJ = ROOT / "build" / "obj"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
    "-I", str(ROOT / "include"), "-I", str(CSRC), "-I", str(PKG),
]


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout)
    if proc.stdout.strip() and os.environ.get("DF8_BUILD_VERBOSE"):
        print(proc.stdout)


def _newest_header_mtime() -> float:
    newest = 0.0
    for pattern, base in (("*.cuh", CSRC), ("*.h", ROOT / "include"), ("**/*.cuh", DNN), ("**/*.h", DNN)):
        for f in base.glob(pattern):
            newest = max(newest, f.stat().st_mtime)
    return newest


def _compile(src: Path, obj: Path, extra: list[str], force: bool, hdr_mtime: float) -> bool:
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_mtime):
        return False
    obj.parent.mkdir(parents=True, exist_ok=True)
    _run([NVCC, *ARCH_FLAGS, *COMMON_FLAGS, *extra, "-c", str(src), "-o", str(obj)])
    return True


def _link(objs: list[Path], out: Path, extra: list[str]) -> None:
    out.parent.mkdir(parents=True, exist_ok=True)
    # link beside the target and rename: a reader never sees a half-written library
    tmp = out.with_name(out.name + ".linking")
    _run([NVCC, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs), *extra])
    os.replace(tmp, out)


def _build_lib(name: str, sources: list[Path], extra_cc: list[str], extra_ld: list[str], force: bool) -> Path:
    out = LIB / name
    hdr_mtime = _newest_header_mtime()
    objs = [OBJ / name / (s.stem + ".o") for s in sources]
    with ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as pool:
        changed = list(pool.map(lambda so: _compile(so[0], so[1], extra_cc, force, hdr_mtime), zip(sources, objs)))
    if force or any(changed) or not out.exists():
        _link(objs, out, extra_ld)
    return out


def build_all(force: bool = False) -> dict[str, Path]:
    """Compile every CUDA source for sm_100a and link the shared libraries. Returns their paths."""
    built = {}
    kernel_srcs = sorted(CSRC.glob("*.cu"))
    built["df8"] = _build_lib("libdf8.so", kernel_srcs, [], ["-ldl"], force)
    dnn_srcs = sorted(DNN.glob("**/*.cu"))
    if dnn_srcs:
        built["df8_dnn"] = _build_lib(
            "libdf8_dnn.so", dnn_srcs, [],
            ["-L", str(LIB), "-ldf8", "-Xlinker", "-rpath=$ORIGIN"], force)
    return built


if __name__ == "__main__":
    libs = build_all(force="--force" in sys.argv)
    for k, v in libs.items():
        print(f"{k}: {v}")
