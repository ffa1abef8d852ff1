"""deepfuse_b200 — Python loader for the B200 fp8 kernel library (``libdf8.so``).

The product is the native code: CUDA kernels behind the C-ABI of ``include/df8.h`` and the C++17
``dnn::`` classes above it.  This module only loads the shared libraries with ``ctypes`` and gives the
tests and ``bench.py`` typed access to the entry points.  PyTorch is used by callers for device memory
and streams only; tensors are passed as raw device pointers.

There is no CPU fallback: if the library has not been built, or an entry point fails, an exception
is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

__all__ = ["lib", "dnn_lib", "check", "Df8Error", "E4M3", "E5M2", "LIB_DIR", "ptr", "stream_ptr"]

LIB_DIR = Path(__file__).resolve().parent / "lib"

E4M3, E5M2 = 0, 1
FP8_MAX = {E4M3: 448.0, E5M2: 57344.0}

# GEMM epilogue flags (include/df8.h)
GELU, RESIDUAL, AMAX = 1, 2, 4
# attention mask modes
MASK_NONE, MASK_CAUSAL, MASK_ADDITIVE = 0, 1, 2


class Df8Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""


_lib = None
_dnn = None

_vp, _sz, _i, _f = C.c_void_p, C.c_size_t, C.c_int, C.c_float

# name -> argtypes; every entry returns df8_status (int) unless listed in _RESTYPES
_SIGNATURES = {
    "df8_amax_f32": [_vp, _sz, _vp, _vp],
    "df8_quantize_f32": [_vp, _sz, _i, _vp, _vp, _vp, _vp],
    "df8_dequantize_f32": [_vp, _sz, _i, _vp, _vp, _vp],
    "df8_gemm_fp8_tn": [_vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp],
    "df8_layernorm_f32": [_vp, _i, _i, _vp, _vp, _f, _vp, _vp, _vp],
    "df8_layernorm_quantize_f32": [_vp, _i, _i, _vp, _vp, _f, _i, _vp, _vp, _vp, _vp, _vp],
    "df8_embed_pe_f32": [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "df8_attention_fp8": [_vp, _i, _vp, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp, _vp],
    "df8_softmax_masked_f32": [_vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "df8_status_word_read": [_vp, _vp],
    "df8_status_word_reset": [],
}
_RESTYPES = {"df8_last_error": C.c_char_p, "df8_version": C.c_char_p}


def lib() -> C.CDLL:
    """The C-ABI kernel library. Raises if it has not been built (python -m deepfuse_b200.build)."""
    global _lib
    if _lib is None:
        path = LIB_DIR / "libdf8.so"
        if not path.exists():
            raise Df8Error(f"{path} is missing: build it with `python -m deepfuse_b200.build` "
                           "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
        for name, rt in _RESTYPES.items():
            fn = getattr(handle, name)
            fn.restype = rt
            fn.argtypes = []
        for name, args in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                raise Df8Error(f"libdf8.so does not export {name}")
            fn.argtypes = args
            fn.restype = C.c_int
        _lib = handle
    return _lib


def check(status: int, what: str = "") -> None:
    """Raise Df8Error carrying df8_last_error() if `status` is non-zero."""
    if status != 0:
        msg = lib().df8_last_error().decode("utf-8", "replace")
        raise Df8Error(f"{what or 'df8 call'} failed (status {status}): {msg}")


def ptr(t) -> int:
    """Device pointer of a torch tensor (or None)."""
    return None if t is None else t.data_ptr()


def stream_ptr(stream=None) -> int:
    """cudaStream_t of a torch stream (default: torch's current stream)."""
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


# ---- thin typed wrappers over torch tensors (used by tests and bench.py) -----------------------

def amax_f32(x, amax_out, stream=None) -> None:
    check(lib().df8_amax_f32(ptr(x), x.numel(), ptr(amax_out), stream_ptr(stream)), "df8_amax_f32")


def quantize_f32(x, kind: int, amax_in, codes_out, scale_out, stream=None) -> None:
    check(lib().df8_quantize_f32(ptr(x), x.numel(), kind, ptr(amax_in), ptr(codes_out), ptr(scale_out),
                                 stream_ptr(stream)), "df8_quantize_f32")


def dequantize_f32(codes, kind: int, scale, y_out, stream=None) -> None:
    check(lib().df8_dequantize_f32(ptr(codes), codes.numel(), kind, ptr(scale), ptr(y_out), stream_ptr(stream)),
          "df8_dequantize_f32")


def gemm_fp8_tn(a_codes, kind_a, scale_a, w_codes, kind_w, scale_w, bias, residual, M, N, K, flags, out,
                out_amax=None, stream=None) -> None:
    check(lib().df8_gemm_fp8_tn(ptr(a_codes), kind_a, ptr(scale_a), ptr(w_codes), kind_w, ptr(scale_w), ptr(bias),
                                ptr(residual), M, N, K, flags, ptr(out), ptr(out_amax), stream_ptr(stream)),
          "df8_gemm_fp8_tn")


def status_word() -> tuple[int, int]:
    """(first timeout code, number of timeouts) recorded by bounded device-side waits; (0, 0) when clean."""
    code, count = C.c_uint(0), C.c_uint(0)
    check(lib().df8_status_word_read(C.byref(code), C.byref(count)), "df8_status_word_read")
    return code.value, count.value


def status_word_reset() -> None:
    check(lib().df8_status_word_reset(), "df8_status_word_reset")


def layernorm_f32(x, rows, cols, gamma, beta, eps, y, amax_out=None, stream=None) -> None:
    check(lib().df8_layernorm_f32(ptr(x), rows, cols, ptr(gamma), ptr(beta), eps, ptr(y), ptr(amax_out),
                                  stream_ptr(stream)), "df8_layernorm_f32")


def layernorm_quantize_f32(x, rows, cols, gamma, beta, eps, kind, codes_out, scale_out, amax_out, row_stats,
                           stream=None) -> None:
    check(lib().df8_layernorm_quantize_f32(ptr(x), rows, cols, ptr(gamma), ptr(beta), eps, kind, ptr(codes_out),
                                           ptr(scale_out), ptr(amax_out), ptr(row_stats), stream_ptr(stream)),
          "df8_layernorm_quantize_f32")


def embed_pe_f32(ids, B, T, E, V, table, bias, pe, out, bad_ids=None, stream=None) -> None:
    check(lib().df8_embed_pe_f32(ptr(ids), B, T, E, V, ptr(table), ptr(bias), ptr(pe), ptr(out), ptr(bad_ids),
                                 stream_ptr(stream)), "df8_embed_pe_f32")


def attention_fp8(qkv_codes, kind, scale, B, T, H, D, mask_mode, mask, out, out_amax=None, stream=None) -> None:
    mask_b = 0 if mask is None else mask.shape[0]
    check(lib().df8_attention_fp8(ptr(qkv_codes), kind, ptr(scale), B, T, H, D, mask_mode, ptr(mask), mask_b,
                                  ptr(out), ptr(out_amax), stream_ptr(stream)), "df8_attention_fp8")


def softmax_masked_f32(x, mask, B, H, T, out, stream=None) -> None:
    mask_b = 0 if mask is None else mask.shape[0]
    check(lib().df8_softmax_masked_f32(ptr(x), ptr(mask), mask_b, B, H, T, ptr(out), stream_ptr(stream)),
          "df8_softmax_masked_f32")
