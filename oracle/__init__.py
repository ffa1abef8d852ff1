"""ctypes front end of the CPU oracle (``oracle/df8_oracle.cpp``).  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this module; the product package never does.  All arrays are numpy, C-contiguous.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libdf8_oracle.so"

E4M3, E5M2 = 0, 1
FP8_MAX = {E4M3: 448.0, E5M2: 57344.0}
GELU, RESIDUAL = 1, 2
MASK_NONE, MASK_CAUSAL, MASK_ADDITIVE = 0, 1, 2


def build(force: bool = False) -> Path:
    """Compile the oracle with the Makefile beside this file (g++, no GPU needed)."""
    src = _HERE / "df8_oracle.cpp"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE)] + (["-B"] if force else []), check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(_LIB_PATH))
        _lib.orc_amax_f32.restype = C.c_float
        _lib.orc_code_value.restype = C.c_float
        _lib.orc_get_threads.restype = C.c_int
        _lib.orc_embed_pe_f32.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def set_threads(n: int) -> None:
    lib().orc_set_threads(C.c_int(n))


def get_threads() -> int:
    return int(lib().orc_get_threads())


def fill_normal(n: int, seed: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_fill_normal(_p(out), C.c_int64(n), C.c_uint64(seed), C.c_float(mean), C.c_float(std))
    return out


def fill_normal_outliers(n: int, seed: int, frac: float = 1e-3, outlier_scale: float = 100.0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_fill_normal_outliers(_p(out), C.c_int64(n), C.c_uint64(seed), C.c_float(frac), C.c_float(outlier_scale))
    return out


def fill_token_ids(n: int, seed: int, vocab: int) -> np.ndarray:
    out = np.empty(n, dtype=np.int32)
    lib().orc_fill_token_ids(_p(out), C.c_int64(n), C.c_uint64(seed), C.c_int32(vocab))
    return out


def amax(x: np.ndarray) -> float:
    x = _f32(x)
    return float(lib().orc_amax_f32(_p(x), C.c_int64(x.size)))


def scales_from_amax(amax_v: float, kind: int) -> np.ndarray:
    s = np.empty(2, dtype=np.float32)
    lib().orc_scales_from_amax(C.c_float(amax_v), C.c_int(kind), _p(s))
    return s


def quantize(x: np.ndarray, kind: int, amax_v: float | None = None):
    """Returns (codes uint8, scale float32[2] = {q, dq})."""
    x = _f32(x)
    if amax_v is None:
        amax_v = amax(x)
    codes = np.empty(x.shape, dtype=np.uint8)
    s = np.empty(2, dtype=np.float32)
    lib().orc_quantize_f32(_p(x), C.c_int64(x.size), C.c_int(kind), C.c_float(amax_v), _p(codes), _p(s))
    return codes, s


def dequantize(codes: np.ndarray, kind: int, dq: float) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    y = np.empty(codes.shape, dtype=np.float32)
    lib().orc_dequantize_f32(_p(codes), C.c_int64(codes.size), C.c_int(kind), C.c_float(dq), _p(y))
    return y


def code_value(code: int, kind: int) -> float:
    return float(lib().orc_code_value(C.c_uint8(code), C.c_int(kind)))


def fc_forward_f32(x, w, b) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    b = None if b is None else _f32(b)
    M, K = x.shape
    N = w.shape[0]
    y = np.empty((M, N), dtype=np.float32)
    lib().orc_fc_forward_f32(_p(x), _p(w), _p(b), C.c_int(M), C.c_int(K), C.c_int(N), _p(y))
    return y


def fc_forward_fp8(xc, kind_x, dqx, wc, kind_w, dqw, bias=None, residual=None, flags=0) -> np.ndarray:
    xc = np.ascontiguousarray(xc, dtype=np.uint8)
    wc = np.ascontiguousarray(wc, dtype=np.uint8)
    M, K = xc.shape
    N = wc.shape[0]
    bias = None if bias is None else _f32(bias)
    residual = None if residual is None else _f32(residual)
    y = np.empty((M, N), dtype=np.float32)
    lib().orc_fc_forward_fp8(_p(xc), C.c_int(kind_x), C.c_float(dqx), _p(wc), C.c_int(kind_w), C.c_float(dqw),
                             _p(bias), _p(residual), C.c_int(M), C.c_int(N), C.c_int(K), C.c_int(flags), _p(y))
    return y


def softmax_masked(x, mask=None) -> np.ndarray:
    x = _f32(x)
    B, H, T, _ = x.shape
    mask_b = 0
    if mask is not None:
        mask = _f32(mask)
        mask_b = mask.shape[0]
    out = np.empty_like(x)
    lib().orc_softmax_masked(_p(x), _p(mask), C.c_int(mask_b), C.c_int(B), C.c_int(H), C.c_int(T), _p(out))
    return out


def fc_backward_f32(dy, x, w):
    """Upstream's fully-connected backward in fp32 (dnn/layers/fully_connected_layer.cu:43-107): dX = dY W,
    dW = dY^T X, db = sum_n dY, each a sequential fp32 sum in upstream; float64 accumulation here (the comparison
    tolerances are far above the difference)."""
    dy, x, w = _f32(dy), _f32(x), _f32(w)
    dx = (dy.astype(np.float64) @ w.astype(np.float64)).astype(np.float32)
    dw = (dy.astype(np.float64).T @ x.astype(np.float64)).astype(np.float32)
    db = dy.astype(np.float64).sum(axis=0).astype(np.float32)
    return dx, dw, db


def fc_backward_fp8(dy, x, w, act_kind: int = E4M3, grad_kind: int = E5M2, w_kind: int = E4M3):
    """The same through the 8-bit path: dY quantised per tensor to e5m2, X to the activation kind, W to e4m3; products of
    the dequantised codes accumulated exactly; db from the unquantised dY."""
    dy, x, w = _f32(dy), _f32(x), _f32(w)
    dyc, dys = quantize(dy, grad_kind)
    xc, xs = quantize(x, act_kind)
    wc, ws = quantize(w, w_kind)
    dyq = dequantize(dyc, grad_kind, dys[1]).astype(np.float64)
    xq = dequantize(xc, act_kind, xs[1]).astype(np.float64)
    wq = dequantize(wc, w_kind, ws[1]).astype(np.float64)
    return (dyq @ wq).astype(np.float32), (dyq.T @ xq).astype(np.float32), dy.astype(np.float64).sum(axis=0).astype(np.float32)


def cross_entropy(logits, targets=None, target_idx=None):
    """Upstream's softmax cross-entropy (dnn/losses/cross_entropy.cu:12-74 loss, :77-139 gradient, :142-170 the mean),
    restated in float32 with its order of operations: per row the maximum, the sum of expf(x - max) accumulated class
    by class, log(sum + 1e-7); loss_i = -sum_j t_ij (x_ij - max - lse); the mean is a float accumulated row by row;
    grad_ij = expf(x_ij - max) / (sum + 1e-7) - t_ij.  Targets: dense [rows, C] or class indices [rows]
    (upstream turns indices into a one-hot matrix first, utils/common.cuh:123).  Returns (mean loss, row losses, grad)."""
    x = _f32(logits)
    rows, Cn = x.shape
    if (targets is None) == (target_idx is None):
        raise ValueError("give dense targets or class indices, one of the two")
    if targets is None:
        t = np.zeros((rows, Cn), np.float32)
        t[np.arange(rows), np.asarray(target_idx, np.int64)] = 1.0
    else:
        t = _f32(targets)
    mx = x.max(axis=1, keepdims=True)
    e = np.exp((x - mx).astype(np.float32)).astype(np.float32)
    s = np.zeros(rows, np.float32)
    for j in range(Cn):  # class by class, as the kernel's loop
        s = (s + e[:, j]).astype(np.float32)
    lse = np.log((s + np.float32(1e-7)).astype(np.float32)).astype(np.float32)
    term = (t * ((x - mx).astype(np.float32) - lse[:, None]).astype(np.float32)).astype(np.float32)
    total = np.zeros(rows, np.float32)
    for j in range(Cn):
        total = (total + term[:, j]).astype(np.float32)
    row_loss = (-total).astype(np.float32)
    acc = np.float32(0.0)
    for v in row_loss:
        acc = np.float32(acc + v)
    mean = np.float32(acc / np.float32(rows))
    grad = (e / (s + np.float32(1e-7))[:, None]).astype(np.float32) - t
    return float(mean), row_loss, grad.astype(np.float32)


def layernorm(x, gamma=None, beta=None, eps: float = 1e-5) -> np.ndarray:
    x = _f32(x)
    cols = x.shape[-1]
    rows = x.size // cols
    gamma = None if gamma is None else _f32(gamma)
    beta = None if beta is None else _f32(beta)
    y = np.empty_like(x)
    lib().orc_layernorm_f32(_p(x), C.c_int64(rows), C.c_int(cols), _p(gamma), _p(beta), C.c_float(eps), _p(y))
    return y


def gelu(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_gelu_f32(_p(x), C.c_int64(x.size), _p(y))
    return y


def pe_table(max_len: int, E: int) -> np.ndarray:
    pe = np.empty((max_len, E), dtype=np.float32)
    lib().orc_pe_table(C.c_int(max_len), C.c_int(E), _p(pe))
    return pe


def embed_pe(ids, table, bias, pe) -> np.ndarray:
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    table = _f32(table)
    B, T = ids.shape
    V, E = table.shape
    bias = None if bias is None else _f32(bias)
    pe = None if pe is None else _f32(pe)
    out = np.empty((B, T, E), dtype=np.float32)
    rc = lib().orc_embed_pe_f32(_p(ids), C.c_int(B), C.c_int(T), C.c_int(E), C.c_int(V), _p(table), _p(bias), _p(pe),
                                _p(out))
    if rc != 0:
        raise RuntimeError("Invalid token ID")
    return out


def attention_fp8(qkv_codes, kind: int, dq: float, B: int, T: int, H: int, D: int, mask_mode: int = MASK_NONE,
                  mask=None) -> np.ndarray:
    qkv_codes = np.ascontiguousarray(qkv_codes, dtype=np.uint8)
    E = H * D
    assert qkv_codes.size == B * T * 3 * E
    mask_b = 0
    if mask is not None:
        mask = _f32(mask)
        mask_b = mask.shape[0]
    out = np.empty((B * T, E), dtype=np.float32)
    lib().orc_attention_fp8(_p(qkv_codes), C.c_int(kind), C.c_float(dq), C.c_int(B), C.c_int(T), C.c_int(H),
                            C.c_int(D), C.c_int(mask_mode), _p(mask), C.c_int(mask_b), _p(out))
    return out
