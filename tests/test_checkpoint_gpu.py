"""Checkpoint files.

1. Records written by the UPSTREAM classes' own save() code (oracle/_ref/libdnn_ref.so: tensor, FullyConnectedLayer,
   LayerNormLayer, TokenEmbedding compiled from the upstream sources) are read by this build's load(), give back the
   values that were put in, and this build's save() writes the same bytes.
2. A whole model in the layout upstream's Gpt2::save writes (header, tokenizer state, every layer preceded by the raw
   bytes of its name) round-trips through save_upstream / load_upstream, and a TransformerBlock record does through
   the block's own load / save.
3. The quantise-once cache (e4m3 codes + scales) gives a model that computes bit for bit what the model that wrote
   it computes, without fp32 weight matrices on the device.
"""
import ctypes as C
import json
import os
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REF_LIB = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libdnn_ref.so"


def p(a):
    return None if a is None else np.ascontiguousarray(a).ctypes.data_as(C.c_void_p)


@pytest.fixture(scope="module")
def dnn(df8, cuda):
    lib = df8.dnn_lib()
    df8.dnn_check(lib.dnn_init(0), "dnn_init")
    df8.dnn_check(lib.dnn_set_fp8_policy(0, 0))
    return lib


@pytest.fixture(scope="module")
def ref(cuda):
    if not REF_LIB.exists():
        pytest.skip("oracle/_ref/libdnn_ref.so not built (needs the upstream sources at build time)")
    lib = C.CDLL(str(REF_LIB), mode=os.RTLD_LOCAL | getattr(os, "RTLD_DEEPBIND", 0))
    lib.ref_last_error.restype = C.c_char_p
    if not hasattr(lib, "ref_fc_save"):
        pytest.skip("oracle/_ref/libdnn_ref.so predates the save wrappers: rebuild it with oracle/ref_build.sh")
    return lib


def roundtrip(df8, dnn, what, src, dst, cap):
    got = np.full(cap, np.nan, np.float32)
    n = C.c_int(0)
    df8.dnn_check(dnn.dnn_file_roundtrip(what, str(src).encode(), str(dst).encode(), p(got), cap, C.byref(n)),
                  "dnn_file_roundtrip")
    return got[: n.value]


def test_records_written_by_upstream_load_here(df8, dnn, ref, oracle, tmp_path):
    # tensor<float> [3, 5, 7]
    t = oracle.fill_normal(105, seed=1).reshape(3, 5, 7)
    shape = (C.c_int * 3)(3, 5, 7)
    assert ref.ref_tensor_save_f32(str(tmp_path / "t.bin").encode(), 3, shape, p(t)) == 0, ref.ref_last_error()
    got = roundtrip(df8, dnn, 0, tmp_path / "t.bin", tmp_path / "t2.bin", 1000)
    assert np.array_equal(got, t.ravel())
    assert (tmp_path / "t.bin").read_bytes() == (tmp_path / "t2.bin").read_bytes()
    # FullyConnectedLayer 100 -> 37 (in_features not a multiple of 16: the fp8 path pads K; the file does not)
    w = oracle.fill_normal(37 * 100, seed=2, std=0.05)
    b = oracle.fill_normal(37, seed=3, std=0.1)
    assert ref.ref_fc_save(str(tmp_path / "fc.bin").encode(), 100, 37, p(w), p(b)) == 0, ref.ref_last_error()
    got = roundtrip(df8, dnn, 1, tmp_path / "fc.bin", tmp_path / "fc2.bin", 10000)
    assert np.array_equal(got, np.concatenate([w, b]))
    assert (tmp_path / "fc.bin").read_bytes() == (tmp_path / "fc2.bin").read_bytes()
    # LayerNormLayer 64
    g = oracle.fill_normal(64, seed=4, mean=1.0, std=0.1)
    be = oracle.fill_normal(64, seed=5, std=0.1)
    assert ref.ref_layernorm_save(str(tmp_path / "ln.bin").encode(), 64, p(g), p(be)) == 0, ref.ref_last_error()
    got = roundtrip(df8, dnn, 2, tmp_path / "ln.bin", tmp_path / "ln2.bin", 1000)
    assert np.array_equal(got, np.concatenate([g, be]))
    # upstream also writes its two gradient tensors, whose contents it never initialises: compare the layout
    # (sizes) and the parameter part of the bytes
    a, c = (tmp_path / "ln.bin").read_bytes(), (tmp_path / "ln2.bin").read_bytes()
    assert len(a) == len(c) and a[: 4 + 2 * (8 + 64 * 4)] == c[: 4 + 2 * (8 + 64 * 4)]
    # TokenEmbedding 50 x 32, context 16
    tab = oracle.fill_normal(50 * 32, seed=6, std=0.02)
    eb = oracle.fill_normal(32, seed=7, std=0.01)
    assert ref.ref_embedding_save(str(tmp_path / "emb.bin").encode(), 50, 32, 16, p(tab), p(eb)) == 0, ref.ref_last_error()
    got = roundtrip(df8, dnn, 3, tmp_path / "emb.bin", tmp_path / "emb2.bin", 10000)
    assert np.array_equal(got, np.concatenate([tab, eb]))
    assert (tmp_path / "emb.bin").read_bytes() == (tmp_path / "emb2.bin").read_bytes()


def test_fc_loaded_from_an_upstream_file_computes_like_an_uploaded_one(df8, dnn, ref, oracle, tmp_path):
    """The imported layer goes through the fp8 path like any other: same output as a layer given the same parameters
    directly, and within 5e-2 of upstream's own fp32 forward of the layer that wrote the file."""
    M, K, N = 32, 256, 96
    w = oracle.fill_normal(N * K, seed=8, std=0.05).reshape(N, K)
    b = oracle.fill_normal(N, seed=9, std=0.1)
    x = oracle.fill_normal(M * K, seed=10).reshape(M, K)
    assert ref.ref_fc_save(str(tmp_path / "fc.bin").encode(), K, N, p(w), p(b)) == 0
    got = roundtrip(df8, dnn, 1, tmp_path / "fc.bin", tmp_path / "fc2.bin", N * K + N)
    y_loaded, y_direct, y_ref = (np.zeros((M, N), np.float32) for _ in range(3))
    df8.dnn_check(dnn.dnn_fc_forward(K, N, p(got[: N * K]), p(got[N * K:]), p(x), M, p(y_loaded)))
    df8.dnn_check(dnn.dnn_fc_forward(K, N, p(w), p(b), p(x), M, p(y_direct)))
    assert np.array_equal(y_loaded, y_direct)
    ref.ref_fc_forward.argtypes = None
    assert ref.ref_fc_forward(K, N, p(w), p(b), p(x), M, p(y_ref)) == 0
    assert np.abs(y_loaded - y_ref).max() / np.abs(y_ref).max() <= 5e-2


def test_gpt2_upstream_layout_round_trip(df8, dnn, oracle, cuda, tmp_path):
    import torch

    vocab = {"<|endoftext|>": 0, "<|unk|>": 1, "<|pad|>": 2, "hello": 3, "world": 4, "h": 5, "i": 6}
    (tmp_path / "vocab.json").write_text(json.dumps(vocab))
    cfg = dict(vocab=64, max_seq_len=32, layers=2, heads=1, hidden=64, ffn=128)
    model = df8.Gpt2(**cfg, vocab_json=str(tmp_path / "vocab.json"))
    path = str(tmp_path / "gpt2_upstream.bin")
    model.save_file(path, "upstream")
    raw = Path(path).read_bytes()
    assert np.frombuffer(raw[:16], np.int32).tolist() == [64, 32, 2, 64]
    for name in (b"TokenEmbedding", b"PositionalEncoding", b"TransformerBlock", b"FullyConnected"):
        assert name in raw
    assert raw.count(b"TransformerBlock") == 2
    back = df8.Gpt2.from_file(path, "upstream")
    n = dnn.dnn_gpt2_num_params(model.h)
    assert dnn.dnn_gpt2_num_params(back.h) == n
    for i, (name, shape) in enumerate(model.param_names()):
        a = np.zeros(int(np.prod(shape)), np.float32)
        b = np.ones_like(a)
        df8.dnn_check(dnn.dnn_gpt2_param_download(model.h, i, p(a)))
        df8.dnn_check(dnn.dnn_gpt2_param_download(back.h, i, p(b)))
        assert np.array_equal(a, b), name
    back.save_file(str(tmp_path / "again.bin"), "upstream")  # the tokenizer came back with the model
    # same bytes except for the order in which the tokenizer's hash maps are written
    assert len(Path(tmp_path / "again.bin").read_bytes()) == len(raw)
    # text in, hidden states out, on both models
    back.cfg = cfg
    h1, h2 = model.forward_text("hello world hi"), back.forward_text("hello world hi")
    assert h1.shape == (6, 64) and np.array_equal(h1, h2)  # BOS hello world h i EOS
    # a TransformerBlock record cut out of the file loads through the block's own load() and saves identically
    start = raw.index(b"TransformerBlock") + len(b"TransformerBlock")
    end = raw.index(b"TransformerBlock", start)
    (tmp_path / "block.bin").write_bytes(raw[start:end])
    got = roundtrip(df8, dnn, 4, tmp_path / "block.bin", tmp_path / "block2.bin", 1 << 20)
    assert got.size == 2 * 2 * 64 + (3 * 64 * 64 + 3 * 64) + (64 * 64 + 64) + (128 * 64 + 128) + (64 * 128 + 64)
    assert (tmp_path / "block2.bin").read_bytes() == raw[start:end]
    with pytest.raises(df8.Df8Error):
        df8.Gpt2.from_file(str(tmp_path / "block.bin"), "upstream")
    model.close()
    back.close()


@pytest.mark.parametrize("act_kind", [0, 1])
def test_quantised_cache_reproduces_the_model(df8, dnn, oracle, cuda, tmp_path, act_kind):
    import torch
    from oracle import gpt2_ref

    cfg = dict(vocab=300, max_seq_len=64, layers=2, heads=2, hidden=128, ffn=256)
    prm = gpt2_ref.make_params(cfg, seed=21, std=0.05)
    df8.dnn_check(dnn.dnn_set_fp8_policy(0, act_kind))
    try:
        model = df8.Gpt2(**cfg)
        model.load_params(prm)
        ids = torch.from_numpy(oracle.fill_token_ids(2 * 64, seed=3, vocab=300).reshape(2, 64)).to(cuda)
        want = df8.device_view(torch, model.forward_logits(ids), (128, 300)).clone()
        path = str(tmp_path / "gpt2.df8q")
        model.save_file(path, "quantized")
        fp32_bytes = sum(int(np.prod(s)) * 4 for _, s in model.param_names())
        assert os.path.getsize(path) < 0.45 * fp32_bytes  # codes are a quarter of the fp32 matrices; the embedding stays fp32
        cached = df8.Gpt2.from_file(path, "quantized")
        got = df8.device_view(torch, cached.forward_logits(ids), (128, 300)).clone()
        assert torch.equal(got, want)
        # the fp32 weight matrices are not on the device: parameter 'block0.qkv.weight' is empty
        names = [n for n, _ in cached.param_names()]
        shape = dict(cached.param_names())["block0.qkv.weight"]
        assert "block0.qkv.weight" in names and int(np.prod(shape)) == 0
    finally:
        df8.dnn_check(dnn.dnn_set_fp8_policy(0, 0))
    with pytest.raises(df8.Df8Error):
        df8.Gpt2.from_file(str(tmp_path / "missing.df8q"), "quantized")
    model.close()
    cached.close()
