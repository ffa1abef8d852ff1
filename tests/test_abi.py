"""The C-ABI library builds for sm_100a, loads, and exports every symbol include/*.h declares.
No compute call is made here (no GPU needed)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared(header: Path):
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(df8_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(df8):
    names = _declared(ROOT / "include" / "df8.h")
    assert "df8_amax_f32" in names and "df8_last_error" in names
    handle = ctypes.CDLL(str(df8.LIB_DIR / "libdf8.so"))
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, f"declared in include/df8.h but not exported: {missing}"


def test_python_signatures_cover_the_header(df8):
    names = set(_declared(ROOT / "include" / "df8.h"))
    bound = set(df8._SIGNATURES) | set(df8._RESTYPES)
    assert names == bound, f"unbound: {sorted(names - bound)}; stale: {sorted(bound - names)}"


def test_error_reporting_without_a_gpu(df8):
    lib = df8.lib()
    assert lib.df8_version().decode().startswith("df8")
    # argument validation happens before any CUDA call
    rc = lib.df8_quantize_f32(None, 16, 7, None, None, None, None)
    assert rc == 1
    assert b"kind" in lib.df8_last_error()
    rc = lib.df8_amax_f32(None, 4, None, None)
    assert rc == 1 and b"null" in lib.df8_last_error()


def test_missing_library_fails_loudly(df8, monkeypatch, tmp_path):
    import deepfuse_b200 as pkg

    monkeypatch.setattr(pkg, "_lib", None)
    monkeypatch.setattr(pkg, "LIB_DIR", tmp_path)
    try:
        pkg.lib()
    except pkg.Df8Error as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")


def test_dnn_harness_exports_every_declared_symbol(df8):
    """libdf8_dnn.so (the C++ dnn:: classes + their C harness) loads without a GPU and exports what
    include/df8_dnn.h declares."""
    text = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / "df8_dnn.h").read_text(), flags=re.S)
    names = sorted(set(re.findall(r"\b(dnn_[a-z0-9_]+)\s*\(", text)))
    assert "dnn_gpt2_create" in names and "dnn_selftest_tensor" in names
    handle = df8.dnn_lib()
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, f"declared in include/df8_dnn.h but not exported: {missing}"


def test_dnn_harness_reports_errors_without_a_gpu(df8):
    lib = df8.dnn_lib()
    assert lib.dnn_set_fp8_policy(3, 0) != 0
    assert b"fp8 kind" in lib.dnn_last_error()
