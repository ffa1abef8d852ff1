"""Pins the CPU oracle to OUTPUTS OF THE UPSTREAM IMPLEMENTATION ITSELF, run on the GPU.

oracle/_ref/libdnn_ref.so is the upstream project's own fp32 FullyConnectedLayer / SoftmaxLayer / LayerNormLayer /
TokenEmbedding / PositionalEncoding compiled for sm_100a from the upstream sources (recipe: oracle/ref_build.sh,
wrapper: oracle/ref_wrap.cu).  It is built where the upstream tree is available and travels as a prebuilt file;
when it is absent these tests skip.  Tolerance 1e-5, the one upstream's own tests use."""
import ctypes as C
import os
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REF_LIB = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libdnn_ref.so"


@pytest.fixture(scope="module")
def ref(cuda):
    if not REF_LIB.exists():
        pytest.skip("oracle/_ref/libdnn_ref.so not built (needs the upstream sources at build time)")
    lib = C.CDLL(str(REF_LIB), mode=os.RTLD_LOCAL | getattr(os, "RTLD_DEEPBIND", 0))
    lib.ref_last_error.restype = C.c_char_p
    return lib


def p(a):
    return None if a is None else np.ascontiguousarray(a).ctypes.data_as(C.c_void_p)


def ok(lib, rc):
    assert rc == 0, lib.ref_last_error().decode()


@pytest.mark.parametrize("M,K,N", [(1, 4, 3), (64, 768, 3072), (5, 100, 37)])
def test_fc_oracle_matches_upstream_kernel(ref, oracle, M, K, N):
    x = oracle.fill_normal(M * K, seed=0).reshape(M, K)
    w = oracle.fill_normal(N * K, seed=100, std=0.02).reshape(N, K)
    b = oracle.fill_normal(N, seed=3, std=0.1)
    y = np.zeros((M, N), np.float32)
    ok(ref, ref.ref_fc_forward(K, N, p(w), p(b), p(x), M, p(y)))
    assert np.abs(y - oracle.fc_forward_f32(x, w, b)).max() <= 1e-5


def test_softmax_oracle_matches_upstream_kernel(ref, oracle):
    """Only rows of at most one warp (T <= 32): upstream's kernel overwrites the shared row with the exponentials
    (softmax_layer.cu:62-64) without a barrier after every thread's max scan (:57-61), so with several warps per
    row a fast warp corrupts the maximum a slow warp is still computing (observed: 1.5e-2 error at T = 1024)."""
    rng = np.random.default_rng(1)
    for B, H, T in [(2, 4, 8), (3, 2, 32), (1, 1, 17)]:
        x = rng.standard_normal((B, H, T, T)).astype(np.float32)
        y = np.zeros_like(x)
        ok(ref, ref.ref_softmax_forward(B, H, T, p(x), None, 0, p(y)))
        assert np.abs(y - oracle.softmax_masked(x)).max() <= 1e-5
        i, j = np.meshgrid(np.arange(T), np.arange(T), indexing="ij")
        mask = np.where(j <= i, 0.0, -1e9).astype(np.float32)[None, None].repeat(B, axis=0)
        ok(ref, ref.ref_softmax_forward(B, H, T, p(x), p(mask), B, p(y)))
        assert np.abs(y - oracle.softmax_masked(x, mask)).max() <= 1e-5


def test_layernorm_oracle_matches_upstream_kernel(ref, oracle):
    for rows, cols in [(7, 48), (64, 768), (33, 1024)]:
        x = oracle.fill_normal(rows * cols, seed=rows, mean=0.5, std=2.0).reshape(rows, cols)
        g = oracle.fill_normal(cols, seed=1, mean=1.0, std=0.2)
        b = oracle.fill_normal(cols, seed=2, std=0.2)
        y = np.zeros_like(x)
        ok(ref, ref.ref_layernorm_forward(rows, cols, p(g), p(b), C.c_float(1e-5), p(x), p(y)))
        assert np.abs(y - oracle.layernorm(x, g, b, 1e-5)).max() <= 2e-5


def test_embedding_oracle_matches_upstream_kernels(ref, oracle):
    V, E, T, B = 50, 48, 9, 2
    table = oracle.fill_normal(V * E, seed=8, std=0.02).reshape(V, E)
    bias = oracle.fill_normal(E, seed=9, std=0.01)
    ids = oracle.fill_token_ids(B * T, seed=2, vocab=V).reshape(B, T)
    y = np.zeros((B, T, E), np.float32)
    ok(ref, ref.ref_embedding_forward(V, E, 16, p(table), p(bias), p(ids), B, T, 0, p(y)))
    assert np.array_equal(y, oracle.embed_pe(ids, table, bias, None))
    # with positions: upstream builds its sinusoidal table with device intrinsics, the oracle on the host
    ok(ref, ref.ref_embedding_forward(V, E, 16, p(table), p(bias), p(ids), B, T, 1, p(y)))
    assert np.abs(y - oracle.embed_pe(ids, table, bias, oracle.pe_table(16, E))).max() <= 1e-5
