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
    "df8_gemm_fp8_tn_ex": [_vp, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp],
    "df8_gemm_fp8_tn_amax_ex": [_vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "df8_gemm_fp8_tn_codes_ex": [_vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "df8_gemm_fp8_tn_part": [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp],
    "df8_gemm_fp8_tn_amax_part": [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "df8_gemm_fp8_tn_codes_part": [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "df8_gemv_fp8_tn": [_vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp],
    "df8_embed_pe_pos_f32": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "df8_kv_cache_append_pos": [_vp, _vp, _i, _i, _i, _vp, _i, _vp, _vp, _vp, _vp],
    "df8_attention_decode_fp8_pos": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp, _vp],
    "df8_attention_decode_fused_f32": [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp, _vp],
    "df8_position_advance": [_vp, _vp],
    "df8_quantize_transpose_f32": [_vp, _i, _i, _i, _vp, _vp, _i, _vp, _vp],
    "df8_quantize_both_layouts_f32": [_vp, _i, _i, _i, _vp, _vp, _i, _vp, _i, _vp, _vp],
    "df8_transpose_u8": [_vp, _i, _i, _i, _vp, _i, _vp],
    "df8_colsum_f32": [_vp, _i, _i, _i, _vp, _vp, _vp],
    "df8_colsum_amax_f32": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp],
    "df8_colsum_partial_floats": [_i],
    "df8_cross_entropy_f32": [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp],
    "df8_cross_entropy_grad_f32": [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _i, _vp],
    "df8_cross_entropy_bad_indices": [_vp, _i],
    "df8_kv_cache_append": [_vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "df8_attention_decode_fp8": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp],
    "df8_layernorm_f32": [_vp, _i, _i, _vp, _vp, _f, _vp, _vp, _vp],
    "df8_layernorm_quantize_f32": [_vp, _i, _i, _vp, _vp, _f, _i, _vp, _vp, _vp, _vp, _vp],
    "df8_layernorm_quantize_f32_noalloc": [_vp, _i, _i, _vp, _vp, _f, _i, _vp, _vp, _vp, _vp],
    "df8_layernorm_shard_stats_f32": [_vp, _i, _i, _vp, _vp],
    "df8_layernorm_shard_amax_f32": [_vp, _i, _i, _vp, _i, _vp, _vp, _f, _vp, _vp, _vp],
    "df8_layernorm_shard_quantize_f32": [_vp, _i, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp],
    "df8_embed_pe_f32": [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "df8_attention_fp8": [_vp, _i, _vp, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp, _vp],
    "df8_softmax_masked_f32": [_vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "df8_gemm_fp8_tn_q": [_vp, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "df8_streamer_create": [_sz, _i, _i, _vp],
    "df8_streamer_create_sharded": [_sz, _i, _i, _vp, _vp],
    "df8_streamer_resize": [_vp, _i],
    "df8_streamer_traffic": [_vp, _vp, _vp],
    "df8_streamer_time_uploads": [_vp, _vp],
    "df8_streamer_destroy": [_vp],
    "df8_streamer_host_ptr": [_vp, _i, _vp],
    "df8_streamer_prefetch": [_vp, _i],
    "df8_streamer_acquire": [_vp, _i, _vp, _vp],
    "df8_streamer_release": [_vp, _i, _vp],
    "df8_streamer_stats": [_vp, _vp, _vp, _vp],
    "df8_comm_available": [_vp],
    "df8_comm_unique_id": [_vp],
    "df8_comm_init_rank": [_vp, _i, _i, _vp],
    "df8_comm_destroy": [_vp],
    "df8_comm_abort": [_vp],
    "df8_comm_rank": [_vp, _vp, _vp],
    "df8_comm_allgather_u8": [_vp, _vp, _vp, _sz, _vp],
    "df8_comm_symm_alloc": [_vp, _sz, _vp],
    "df8_comm_p2p_enabled": [_vp, _vp],
    "df8_comm_allgather_symm": [_vp, _vp, _sz, _sz, _vp],
    "df8_comm_push_symm": [_vp, _vp, _sz, _sz, _vp, _vp],
    "df8_comm_wait_symm": [_vp, C.c_uint, _i, _vp],
    "df8_comm_allreduce_max_p2p": [_vp, _vp, _vp],
    "df8_comm_bytes_pushed": [_vp, _vp],
    "df8_comm_allreduce_max_f32": [_vp, _vp, _sz, _vp],
    "df8_gemm_fp8_tn_amax": [_vp, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "df8_gemm_fp8_tn_codes": [_vp, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "df8_fc_fp8_column_sharded": [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "df8_interleave_gathered_u8": [_vp, _i, _i, _i, _vp, _vp],
    "df8_status_word_read": [_vp, _vp],
    "df8_status_word_reset": [],
    "df8_status_word_check": [],
    "df8_set_amax_preclear": [C.c_int],
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


def gemm_fp8_tn_ex(a_codes, kind_a, scale_a, a_slabs, w_codes, kind_w, scale_w, bias, residual, M, N, K, flags, out, ldc,
                   out_amax=None, stream=None) -> None:
    check(lib().df8_gemm_fp8_tn_ex(ptr(a_codes), kind_a, ptr(scale_a), a_slabs, ptr(w_codes), kind_w, ptr(scale_w),
                                   ptr(bias), ptr(residual), M, N, K, flags, ptr(out), ldc, ptr(out_amax),
                                   stream_ptr(stream)), "df8_gemm_fp8_tn_ex")


def gemm_fp8_tn_q(a_codes, kind_a, scale_a, w_codes, kind_w, scale_w, bias, M, N, K, flags, out_kind, out_codes,
                  out_scale, out_amax, stream=None) -> None:
    check(lib().df8_gemm_fp8_tn_q(ptr(a_codes), kind_a, ptr(scale_a), ptr(w_codes), kind_w, ptr(scale_w), ptr(bias),
                                  M, N, K, flags, out_kind, ptr(out_codes), ptr(out_scale), ptr(out_amax),
                                  stream_ptr(stream)), "df8_gemm_fp8_tn_q")


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


def layernorm_quantize_f32_noalloc(x, rows, cols, gamma, beta, eps, kind, codes_out, scale_out, amax_out,
                                   stream=None) -> None:
    check(lib().df8_layernorm_quantize_f32_noalloc(ptr(x), rows, cols, ptr(gamma), ptr(beta), eps, kind,
                                                   ptr(codes_out), ptr(scale_out), ptr(amax_out),
                                                   stream_ptr(stream)), "df8_layernorm_quantize_f32_noalloc")


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


# ---- libdf8_dnn.so: the C++ dnn:: classes behind their C harness (include/df8_dnn.h) -----------------

_DNN_SIGNATURES = {
    "dnn_init": [_i],
    "dnn_set_stream": [_vp],
    "dnn_set_fp8_policy": [_i, _i],
    "dnn_gpt2_destroy": [_vp],
    "dnn_gpt2_set_options": [_vp, _i, _i],
    "dnn_gpt2_num_params": [_vp],
    "dnn_gpt2_param_info": [_vp, _i, _vp, _i, _vp, _vp],
    "dnn_gpt2_param_upload": [_vp, _i, _vp],
    "dnn_gpt2_param_download": [_vp, _i, _vp],
    "dnn_gpt2_prepare": [_vp],
    "dnn_gpt2_set_stage_timing": [_vp, _i],
    "dnn_gpt2_last_head_ms": [_vp, _vp],
    "dnn_gpt2_initialize_on_device": [_vp, C.c_ulonglong, _f],
    "dnn_gpt2_forward_logits": [_vp, _vp, _i, _i, _i, _vp],
    "dnn_gpt2_forward_logits_host": [_vp, _vp, _i, _i, _vp],
    "dnn_gpt2_forward_hidden": [_vp, _vp, _i, _i, _vp],
    "dnn_gpt2_forward_logits_pitched": [_vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "dnn_gpt2_copy_logits_host": [_vp, _vp],
    "dnn_gpt2_serve_step": [_vp, _vp, _i, _i, _vp],
    "dnn_gpt2_serve_flush": [_vp],
    "dnn_gpt2_forward_ids": [_vp, _vp, _i, _vp],
    "dnn_gpt2_save": [_vp, C.c_char_p],
    "dnn_gpt2_enable_streaming": [_vp, _i, _i],
    "dnn_gpt2_disable_streaming": [_vp],
    "dnn_gpt2_enable_streaming_sharded": [_vp, _i, _i, _vp],
    "dnn_gpt2_resize_streaming_slots": [_vp, _i],
    "dnn_gpt2_streaming_traffic": [_vp, _vp, _vp],
    "dnn_gpt2_time_layer_uploads": [_vp, _vp],
    "dnn_fc_forward": [_i, _i, _vp, _vp, _vp, _i, _vp],
    "dnn_fc_backward": [_i, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp],
    "dnn_layernorm_forward": [_i, _i, _vp, _vp, _f, _vp, _vp],
    "dnn_softmax_forward": [_i, _i, _i, _vp, _vp, _i, _vp],
    "dnn_mha_forward": [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp],
    "dnn_block_forward": [_i, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _vp],
    "dnn_embedding_forward": [_i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp],
    "dnn_selftest_tensor": [_vp, _i],
    "dnn_selftest_context": [_vp, _i],
    "dnn_selftest_errors": [_vp, _i],
    "dnn_selftest_bounded_wait": [_vp, _i],
    "dnn_selftest_tokenizer": [C.c_char_p, _vp, _i],
    "dnn_tokenizer_encode": [C.c_char_p, C.c_char_p, C.c_char_p, _i, _vp, _i],
    "dnn_tokenizer_decode": [C.c_char_p, C.c_char_p, _vp, _i, _i, _vp, _i],
    "dnn_tokenizer_save": [C.c_char_p, C.c_char_p],
    "dnn_cross_entropy": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp],
    "dnn_gpt2_prefill": [_vp, _vp, _i, _i, _i, _vp],
    "dnn_gpt2_decode_step": [_vp, _vp, _i, _i, _vp],
    "dnn_gpt2_end_decode": [_vp],
    "dnn_gpt2_decode_graph_active": [_vp, _vp],
    "dnn_gpt2_save_upstream": [_vp, C.c_char_p],
    "dnn_gpt2_save_quantized": [_vp, C.c_char_p],
    "dnn_gpt2_forward_text": [_vp, C.c_char_p, _vp, _i, _vp],
    "dnn_file_roundtrip": [_i, C.c_char_p, C.c_char_p, _vp, _i, _vp],
    "dnn_set_host_init": [_i],
    "dnn_gpt2cs_destroy": [_vp],
    "dnn_gpt2cs_set_options": [_vp, _i, _i],
    "dnn_gpt2cs_vocab_range": [_vp, _vp, _vp],
    "dnn_gpt2cs_num_params": [_vp],
    "dnn_gpt2cs_param_info": [_vp, _i, _vp, _i, _vp, _vp],
    "dnn_gpt2cs_param_upload": [_vp, _i, _vp],
    "dnn_gpt2cs_initialize_on_device": [_vp, C.c_ulonglong],
    "dnn_gpt2cs_prepare": [_vp],
    "dnn_gpt2cs_forward_logits_shard": [_vp, _vp, _i, _i, _i, _vp],
    "dnn_gpt2cs_forward_logits_shard_host": [_vp, _vp, _i, _i, _vp],
    "dnn_gpt2cs_forward_logits_shard_pitched": [_vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "dnn_gpt2cs_forward_hidden": [_vp, _vp, _i, _i, _vp],
}


def dnn_lib() -> C.CDLL:
    """The C++ dnn:: class library behind its C harness. Raises if it has not been built."""
    global _dnn
    if _dnn is None:
        lib()  # libdf8.so first (RTLD_GLOBAL), libdf8_dnn.so links against it
        path = LIB_DIR / "libdf8_dnn.so"
        if not path.exists():
            raise Df8Error(f"{path} is missing: build it with `python -m deepfuse_b200.build`")
        handle = C.CDLL(str(path))
        handle.dnn_last_error.restype = C.c_char_p
        handle.dnn_last_error.argtypes = []
        handle.dnn_gpt2_create.restype = C.c_void_p
        handle.dnn_gpt2_create.argtypes = [_i] * 6
        handle.dnn_gpt2_streamed_bytes.restype = C.c_ulonglong
        handle.dnn_gpt2_streamed_bytes.argtypes = [_vp]
        handle.dnn_gpt2_load.restype = C.c_void_p
        handle.dnn_gpt2_load.argtypes = [C.c_char_p]
        for fn in ("dnn_gpt2_load_upstream", "dnn_gpt2_load_quantized"):
            getattr(handle, fn).restype = C.c_void_p
            getattr(handle, fn).argtypes = [C.c_char_p]
        handle.dnn_gpt2_create_with_tokenizer.restype = C.c_void_p
        handle.dnn_gpt2_create_with_tokenizer.argtypes = [C.c_char_p] + [_i] * 6
        handle.dnn_gpt2cs_bytes_pushed.restype = C.c_ulonglong
        handle.dnn_gpt2cs_bytes_pushed.argtypes = [_vp]
        handle.dnn_gpt2cs_create.restype = C.c_void_p
        handle.dnn_gpt2cs_create.argtypes = [_vp] + [_i] * 6
        for name, args in _DNN_SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = args
            fn.restype = None if name in ("dnn_gpt2_destroy", "dnn_gpt2cs_destroy") else C.c_int
        _dnn = handle
    return _dnn


def dnn_check(rc: int, what: str = "dnn call") -> None:
    if rc != 0:
        raise Df8Error(f"{what} failed (code {rc}): {dnn_lib().dnn_last_error().decode('utf-8', 'replace')}")


class Gpt2:
    """dnn::Gpt2<float> driven through the C harness (tests and bench.py)."""

    def __init__(self, vocab, max_seq_len, layers, heads, hidden, ffn, device: int = 0, vocab_json: str | None = None):
        d = dnn_lib()
        dnn_check(d.dnn_init(device), "dnn_init")
        self.cfg = dict(vocab=vocab, max_seq_len=max_seq_len, layers=layers, heads=heads, hidden=hidden, ffn=ffn)
        if vocab_json is not None:  # with a BpeTokenizer over that vocabulary file
            self.h = d.dnn_gpt2_create_with_tokenizer(vocab_json.encode(), vocab, max_seq_len, layers, heads, hidden, ffn)
        else:
            self.h = d.dnn_gpt2_create(vocab, max_seq_len, layers, heads, hidden, ffn)
        if not self.h:
            raise Df8Error("dnn_gpt2_create failed: " + d.dnn_last_error().decode())

    @classmethod
    def from_file(cls, path: str, layout: str = "upstream", device: int = 0) -> "Gpt2":
        """A model read from a file: layout 'upstream' (what upstream's Gpt2::save writes), 'quantized' (the
        quantise-once cache of save_quantized) or 'native' (Gpt2::save of this build)."""
        d = dnn_lib()
        dnn_check(d.dnn_init(device), "dnn_init")
        fn = {"upstream": d.dnn_gpt2_load_upstream, "quantized": d.dnn_gpt2_load_quantized, "native": d.dnn_gpt2_load}[layout]
        h = fn(path.encode())
        if not h:
            raise Df8Error(f"loading {path} failed: " + d.dnn_last_error().decode())
        self = cls.__new__(cls)
        self.h = h
        self.cfg = None
        return self

    def save_file(self, path: str, layout: str = "upstream"):
        d = dnn_lib()
        fn = {"upstream": d.dnn_gpt2_save_upstream, "quantized": d.dnn_gpt2_save_quantized, "native": d.dnn_gpt2_save}[layout]
        dnn_check(fn(self.h, path.encode()), f"saving {path}")

    def forward_text(self, text: str):
        """Gpt2::forward_from_text: numpy hidden states [T, E] of the tokenised text."""
        import numpy as np

        cap = 1 << 24
        out = np.empty(cap, np.float32)
        t = C.c_int(0)
        dnn_check(dnn_lib().dnn_gpt2_forward_text(self.h, text.encode(), out.ctypes.data_as(C.c_void_p), cap, C.byref(t)),
                  "dnn_gpt2_forward_text")
        hidden = self.cfg["hidden"] if self.cfg else None
        if hidden is None:
            raise Df8Error("forward_text needs the model's configuration (models made by from_file: use the harness call)")
        return out[: t.value * hidden].reshape(t.value, hidden).copy()

    def close(self):
        if self.h:
            dnn_lib().dnn_gpt2_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def param_names(self):
        d = dnn_lib()
        out = []
        buf = C.create_string_buffer(128)
        shape = (C.c_int * 8)()
        ndim = C.c_int(0)
        for i in range(d.dnn_gpt2_num_params(self.h)):
            dnn_check(d.dnn_gpt2_param_info(self.h, i, buf, 128, shape, C.byref(ndim)), "dnn_gpt2_param_info")
            out.append((buf.value.decode(), tuple(shape[k] for k in range(ndim.value))))
        return out

    def load_params(self, params: dict):
        import numpy as np

        d = dnn_lib()
        for i, (name, shape) in enumerate(self.param_names()):
            a = np.ascontiguousarray(params[name], dtype=np.float32)
            n = 1
            for s in shape:
                n *= s
            if a.size != n:
                raise ValueError(f"{name}: expected {shape}, got {a.shape}")
            dnn_check(d.dnn_gpt2_param_upload(self.h, i, a.ctypes.data_as(C.c_void_p)), "dnn_gpt2_param_upload")
        dnn_check(d.dnn_gpt2_prepare(self.h), "dnn_gpt2_prepare")

    def initialize_on_device(self, seed: int, std: float = 0.02):
        dnn_check(dnn_lib().dnn_gpt2_initialize_on_device(self.h, seed, std), "dnn_gpt2_initialize_on_device")
        dnn_check(dnn_lib().dnn_gpt2_prepare(self.h), "dnn_gpt2_prepare")

    def set_stage_timing(self, on: bool):
        dnn_check(dnn_lib().dnn_gpt2_set_stage_timing(self.h, int(on)), "dnn_gpt2_set_stage_timing")

    def last_head_ms(self) -> float:
        ms = C.c_float(0)
        dnn_check(dnn_lib().dnn_gpt2_last_head_ms(self.h, C.byref(ms)), "dnn_gpt2_last_head_ms")
        return ms.value

    def set_options(self, gelu=True, causal=False):
        dnn_check(dnn_lib().dnn_gpt2_set_options(self.h, int(gelu), int(causal)), "dnn_gpt2_set_options")

    def enable_streaming(self, slots=2, release_fp32=False, comm=None):
        """comm: a Comm of more than one rank -> every rank uploads 1/world of each layer and an all-gather over
        NVLink completes the slot (all ranks then run the same sequence of forwards)."""
        if comm is not None and comm.h:
            dnn_check(dnn_lib().dnn_gpt2_enable_streaming_sharded(self.h, slots, int(release_fp32), comm.h),
                      "dnn_gpt2_enable_streaming_sharded")
        else:
            dnn_check(dnn_lib().dnn_gpt2_enable_streaming(self.h, slots, int(release_fp32)), "dnn_gpt2_enable_streaming")
        self._streaming = True

    def resize_streaming_slots(self, slots: int):
        dnn_check(dnn_lib().dnn_gpt2_resize_streaming_slots(self.h, slots), "dnn_gpt2_resize_streaming_slots")

    def streaming_traffic(self) -> tuple[int, int]:
        """(bytes this rank copied from host memory, bytes it received from its peers) since streaming began."""
        a, b = C.c_ulonglong(0), C.c_ulonglong(0)
        dnn_check(dnn_lib().dnn_gpt2_streaming_traffic(self.h, C.byref(a), C.byref(b)), "dnn_gpt2_streaming_traffic")
        return a.value, b.value

    def time_uploads(self) -> float:
        """Device time (ms) of uploading every layer once with nothing else running."""
        ms = C.c_float(0)
        dnn_check(dnn_lib().dnn_gpt2_time_layer_uploads(self.h, C.byref(ms)), "dnn_gpt2_time_layer_uploads")
        return ms.value

    def disable_streaming(self):
        dnn_check(dnn_lib().dnn_gpt2_disable_streaming(self.h), "dnn_gpt2_disable_streaming")

    def streamed_bytes(self) -> int:
        return int(dnn_lib().dnn_gpt2_streamed_bytes(self.h))

    def set_stream(self, stream=None):
        """The stream every dnn:: object of this process launches on from now on (as upstream's Cuda context holds
        one stream): not a property of this model.  None = torch's current stream.  Hand the default back before the
        stream is destroyed."""
        dnn_check(dnn_lib().dnn_set_stream(stream_ptr(stream)), "dnn_set_stream")

    def forward_logits(self, ids_dev, check_ids=True) -> int:
        """ids_dev: torch int32 CUDA tensor [B,T]; returns the device pointer of fp32 logits [B*T, V]."""
        out = C.c_void_p(0)
        B, T = ids_dev.shape
        dnn_check(dnn_lib().dnn_gpt2_forward_logits(self.h, ptr(ids_dev), B, T, int(check_ids), C.byref(out)),
                  "dnn_gpt2_forward_logits")
        return out.value

    def forward_logits_host(self, ids_host) -> int:
        """ids_host: pinned torch int32 CPU tensor [B,T]; the upload happens inside the call."""
        out = C.c_void_p(0)
        B, T = ids_host.shape
        dnn_check(dnn_lib().dnn_gpt2_forward_logits_host(self.h, ids_host.data_ptr(), B, T, C.byref(out)),
                  "dnn_gpt2_forward_logits_host")
        return out.value

    def forward_logits_pitched(self, ids, check_ids=True) -> tuple[int, int]:
        """ids: torch int32 tensor [B,T] on the device, or pinned on the host (uploaded inside the call).  Returns
        (device pointer, pitch): fp32 logits [B*T, pitch] whose first `vocab` columns of every row are valid."""
        out, pitch = C.c_void_p(0), C.c_int(0)
        B, T = ids.shape
        on_host = 0 if ids.is_cuda else 1
        dnn_check(dnn_lib().dnn_gpt2_forward_logits_pitched(self.h, ids.data_ptr(), on_host, B, T, int(check_ids),
                                                            C.byref(out), C.byref(pitch)),
                  "dnn_gpt2_forward_logits_pitched")
        return out.value, pitch.value

    def copy_logits_host(self, dst_host) -> None:
        """Enqueues the copy of the last logits into the dense (pinned) host tensor [B*T, vocab]."""
        dnn_check(dnn_lib().dnn_gpt2_copy_logits_host(self.h, dst_host.data_ptr()), "dnn_gpt2_copy_logits_host")

    def serve_step(self, ids_host, dst_host) -> None:
        """One step of a serving loop: pinned host ids [B,T] in, the full logits into the pinned host tensor
        [B*T, vocab]; the copy back runs on a stream of its own under the next step's forward.  dst_host must not be
        reused before the next-but-one call (alternate two buffers) or serve_flush()."""
        B, T = ids_host.shape
        dnn_check(dnn_lib().dnn_gpt2_serve_step(self.h, ids_host.data_ptr(), B, T, dst_host.data_ptr()), "dnn_gpt2_serve_step")

    def serve_flush(self) -> None:
        """The current stream waits for every copy serve_step has issued."""
        dnn_check(dnn_lib().dnn_gpt2_serve_flush(self.h), "dnn_gpt2_serve_flush")

    def forward_hidden(self, ids_dev) -> int:
        out = C.c_void_p(0)
        B, T = ids_dev.shape
        dnn_check(dnn_lib().dnn_gpt2_forward_hidden(self.h, ptr(ids_dev), B, T, C.byref(out)),
                  "dnn_gpt2_forward_hidden")
        return out.value

    def prefill(self, ids_dev, max_len: int = 0) -> int:
        """Prompt [B,T] (int32, device) -> device pointer of the last position's logits [B, vocab]; fills the KV cache."""
        out = C.c_void_p(0)
        B, T = ids_dev.shape
        dnn_check(dnn_lib().dnn_gpt2_prefill(self.h, ptr(ids_dev), B, T, max_len, C.byref(out)), "dnn_gpt2_prefill")
        return out.value

    def decode_step(self, next_ids_dev, check_ids=True) -> int:
        """One new token id per sequence [B] (int32, device) -> device pointer of its logits [B, vocab]."""
        out = C.c_void_p(0)
        dnn_check(dnn_lib().dnn_gpt2_decode_step(self.h, ptr(next_ids_dev), next_ids_dev.numel(), int(check_ids),
                                                 C.byref(out)), "dnn_gpt2_decode_step")
        return out.value

    def end_decode(self):
        dnn_check(dnn_lib().dnn_gpt2_end_decode(self.h), "dnn_gpt2_end_decode")

    def decode_graph_active(self):
        """True once decode steps are replayed from a CUDA graph (never on the legacy default stream)."""
        v = C.c_int(0)
        dnn_check(dnn_lib().dnn_gpt2_decode_graph_active(self.h, C.byref(v)), "dnn_gpt2_decode_graph_active")
        return bool(v.value)


class Comm:
    """One df8_comm (NCCL communicator, one process per GPU).  The 128-byte id made on rank 0 reaches the other ranks
    through torch.distributed when a process group exists, otherwise through the file `id_path`."""

    def __init__(self, rank: int, world: int, id_path: str | None = None):
        import os
        import time

        l = lib()
        buf = C.create_string_buffer(128)
        self.h = C.c_void_p(0)
        self.rank, self.world = rank, world
        if world == 1:
            return  # a single rank needs no communicator: the sharded model takes NULL
        use_dist = False
        try:
            import torch.distributed as dist

            use_dist = dist.is_available() and dist.is_initialized() and id_path is None
        except Exception:
            pass
        if use_dist:
            import torch

            if rank == 0:
                check(l.df8_comm_unique_id(buf), "df8_comm_unique_id")
            dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
            t = torch.tensor(list(buf.raw), dtype=torch.uint8, device=dev)
            dist.broadcast(t, src=0)
            buf.raw = bytes(t.cpu().tolist())
        else:
            if id_path is None:
                raise Df8Error("Comm needs an initialised torch.distributed group or an id_path")
            if rank == 0:
                check(l.df8_comm_unique_id(buf), "df8_comm_unique_id")
                with open(id_path + ".tmp", "wb") as f:
                    f.write(buf.raw)
                os.replace(id_path + ".tmp", id_path)
            else:
                for _ in range(1200):
                    if os.path.exists(id_path):
                        break
                    time.sleep(0.05)
                buf.raw = open(id_path, "rb").read()
        check(l.df8_comm_init_rank(buf, world, rank, C.byref(self.h)), "df8_comm_init_rank")

    def close(self):
        if self.h:
            check(lib().df8_comm_destroy(self.h), "df8_comm_destroy")
            self.h = C.c_void_p(0)

    def abort(self):
        """df8_comm_abort: give the communicator up without talking to the peers (one of them is gone).  Close every
        model built on it first; nothing of this rank may be in flight on it."""
        if self.h:
            h, self.h = self.h, C.c_void_p(0)
            check(lib().df8_comm_abort(h), "df8_comm_abort")


class Gpt2ColumnSharded:
    """dnn::Gpt2ColumnSharded<float> through the C harness: this rank's shard of a GPT-2 whose fully-connected
    weights are split by output columns over the ranks of `comm`."""

    def __init__(self, comm: Comm, vocab, max_seq_len, layers, heads, hidden, ffn, device: int = 0):
        d = dnn_lib()
        dnn_check(d.dnn_init(device), "dnn_init")
        self.comm = comm
        self.cfg = dict(vocab=vocab, max_seq_len=max_seq_len, layers=layers, heads=heads, hidden=hidden, ffn=ffn)
        self.h = d.dnn_gpt2cs_create(comm.h, vocab, max_seq_len, layers, heads, hidden, ffn)
        if not self.h:
            raise Df8Error("dnn_gpt2cs_create failed: " + d.dnn_last_error().decode())
        b, n = C.c_int(0), C.c_int(0)
        dnn_check(d.dnn_gpt2cs_vocab_range(self.h, C.byref(b), C.byref(n)), "dnn_gpt2cs_vocab_range")
        self.vocab_begin, self.vocab_rows = b.value, n.value

    def close(self):
        if self.h:
            dnn_lib().dnn_gpt2cs_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def param_names(self):
        d = dnn_lib()
        out = []
        buf = C.create_string_buffer(128)
        shape = (C.c_int * 8)()
        ndim = C.c_int(0)
        for i in range(d.dnn_gpt2cs_num_params(self.h)):
            dnn_check(d.dnn_gpt2cs_param_info(self.h, i, buf, 128, shape, C.byref(ndim)), "dnn_gpt2cs_param_info")
            out.append((buf.value.decode(), tuple(shape[k] for k in range(ndim.value))))
        return out

    def load_full_params(self, params: dict, prepare: bool = True):
        """Slices this rank's shards out of a full parameter dictionary and uploads them (collective).  prepare=False
        leaves the re-quantisation of the weights to the next forward (what a C++ caller that only uploads gets)."""
        import numpy as np

        from .sharding import shard_gpt2_params

        d = dnn_lib()
        mine = shard_gpt2_params(params, self.cfg, self.comm.world, self.comm.rank)
        for i, (name, shape) in enumerate(self.param_names()):
            a = np.ascontiguousarray(mine[name], dtype=np.float32)
            n = 1
            for s in shape:
                n *= s
            if a.size != n:
                raise ValueError(f"{name}: expected {shape}, got {a.shape}")
            dnn_check(d.dnn_gpt2cs_param_upload(self.h, i, a.ctypes.data_as(C.c_void_p)), "dnn_gpt2cs_param_upload")
        if prepare:
            dnn_check(d.dnn_gpt2cs_prepare(self.h), "dnn_gpt2cs_prepare")

    def initialize_on_device(self, seed: int):
        dnn_check(dnn_lib().dnn_gpt2cs_initialize_on_device(self.h, seed), "dnn_gpt2cs_initialize_on_device")
        dnn_check(dnn_lib().dnn_gpt2cs_prepare(self.h), "dnn_gpt2cs_prepare")

    def set_options(self, gelu=True, causal=False):
        dnn_check(dnn_lib().dnn_gpt2cs_set_options(self.h, int(gelu), int(causal)), "dnn_gpt2cs_set_options")

    def set_stream(self, stream=None):
        dnn_check(dnn_lib().dnn_set_stream(stream_ptr(stream)), "dnn_set_stream")

    def forward_logits_shard(self, ids_dev, check_ids=True) -> int:
        """ids_dev: torch int32 CUDA tensor [B,T] (the same on every rank); returns the device pointer of this rank's
        fp32 logits [B*T, vocab_rows]."""
        out = C.c_void_p(0)
        B, T = ids_dev.shape
        dnn_check(dnn_lib().dnn_gpt2cs_forward_logits_shard(self.h, ptr(ids_dev), B, T, int(check_ids), C.byref(out)),
                  "dnn_gpt2cs_forward_logits_shard")
        return out.value

    def forward_logits_shard_pitched(self, ids, check_ids=True) -> tuple[int, int]:
        """ids on the device or pinned on the host; returns (device pointer, pitch) of fp32 logits [B*T, pitch]."""
        out, pitch = C.c_void_p(0), C.c_int(0)
        B, T = ids.shape
        dnn_check(dnn_lib().dnn_gpt2cs_forward_logits_shard_pitched(self.h, ids.data_ptr(), 0 if ids.is_cuda else 1, B, T,
                                                                    int(check_ids), C.byref(out), C.byref(pitch)),
                  "dnn_gpt2cs_forward_logits_shard_pitched")
        return out.value, pitch.value

    def forward_hidden(self, ids_dev) -> int:
        out = C.c_void_p(0)
        B, T = ids_dev.shape
        dnn_check(dnn_lib().dnn_gpt2cs_forward_hidden(self.h, ptr(ids_dev), B, T, C.byref(out)), "dnn_gpt2cs_forward_hidden")
        return out.value

    def bytes_pushed(self) -> int:
        return int(dnn_lib().dnn_gpt2cs_bytes_pushed(self.h))

    def forward_logits_shard_host(self, ids_host) -> int:
        out = C.c_void_p(0)
        B, T = ids_host.shape
        dnn_check(dnn_lib().dnn_gpt2cs_forward_logits_shard_host(self.h, ids_host.data_ptr(), B, T, C.byref(out)),
                  "dnn_gpt2cs_forward_logits_shard_host")
        return out.value


def device_view(torch, data_ptr: int, shape, dtype=None):
    """A torch tensor viewing device memory owned by the native side (no copy)."""
    import numpy as np

    dtype = dtype or torch.float32
    n = int(np.prod(shape))
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Holder:
        __cuda_array_interface__ = {"shape": (n,), "typestr": {4: "<f4", 1: "|u1"}[itemsize] if dtype != torch.int32 else "<i4",
                                    "data": (data_ptr, False), "version": 3}

    return torch.as_tensor(_Holder(), device=f"cuda:{torch.cuda.current_device()}").view(*shape)
