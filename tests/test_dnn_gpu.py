"""The C++ dnn:: classes (FullyConnectedLayer, LayerNormLayer, SoftmaxLayer, MultiHeadAttentionLayer,
TransformerBlock, TokenEmbedding, PositionalEncoding, Gpt2) on the GPU against the CPU oracle, through the C
harness of include/df8_dnn.h.  The cases restate the upstream project's own layer tests with fixed seeds.

Tolerances (max|y-ref| / max|ref|): fp32-only layers (LayerNorm, softmax, embedding) 2e-5 absolute; one fp8
GEMM on identical inputs 2e-4 against the fp8 oracle and 5e-2 against the fp32 layer.  Layers that re-quantise
intermediate tensors (attention layer, block, model) are compared two ways: directly against the fp8 oracle
pipeline with a loose bound (an intermediate that differs by 1e-3 flips a few fp8 codes, each flip being worth
one fp8 step, so chains cannot be held to the single-kernel 1e-2), and through their error against the
UNQUANTISED fp32 pipeline, which must not exceed the fp8 oracle's own error against it by more than 25 %."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rel_err(y, ref):
    return float(np.abs(y.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def p(a):
    return None if a is None else np.ascontiguousarray(a).ctypes.data_as(C.c_void_p)


@pytest.fixture(scope="module")
def dnn(df8, cuda):
    lib = df8.dnn_lib()
    df8.dnn_check(lib.dnn_init(0), "dnn_init")
    df8.dnn_check(lib.dnn_set_fp8_policy(0, 0))
    return lib


@pytest.mark.parametrize("which", ["tensor", "context", "errors", "bounded_wait"])
def test_cpp_selftests(df8, dnn, which):
    buf = C.create_string_buffer(1 << 14)
    failures = getattr(dnn, f"dnn_selftest_{which}")(buf, len(buf))
    assert failures == 0, buf.value.decode()


def test_fc_forward_pass_case(df8, dnn, oracle):
    """ForwardPass of fully_connected_layer_test.cu:106-148: in 4, out 3, batch 1, input i/4."""
    rng = np.random.default_rng(0)
    w = rng.uniform(-1, 1, (3, 4)).astype(np.float32)
    b = rng.uniform(-1, 1, 3).astype(np.float32)
    x = (np.arange(4, dtype=np.float32) / 4).reshape(1, 4)
    y = np.zeros((1, 3), np.float32)
    df8.dnn_check(dnn.dnn_fc_forward(4, 3, p(w), p(b), p(x), 1, p(y)))
    xc, xs = oracle.quantize(x, 0)
    wc, ws = oracle.quantize(w, 0)
    ref = oracle.fc_forward_fp8(xc, 0, xs[1], wc, 0, ws[1], b)
    assert rel_err(y, ref) <= 1e-5
    assert rel_err(y, oracle.fc_forward_f32(x, w, b)) <= 5e-2


def test_fc_known_weights_case(df8, dnn):
    """NonzeroInputGivesNonzeroOutput (:258-285): W=[[1,2],[3,4]], b=[.5,-.5], x=[1,2]; upstream only asserts
    non-zero outputs; the fp32 answer is [5.5, 10.5] and per-tensor e4m3 (3 scaled by 448/4 is not
    representable) lands within the 5e-2 bar."""
    w = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([0.5, -0.5], np.float32)
    x = np.array([[1, 2]], np.float32)
    y = np.zeros((1, 2), np.float32)
    df8.dnn_check(dnn.dnn_fc_forward(2, 2, p(w), p(b), p(x), 1, p(y)))
    assert (y != 0).all()
    assert rel_err(y, np.array([[5.5, 10.5]])) <= 5e-2


@pytest.mark.parametrize("M,K,N", [(64, 768, 3072), (5, 100, 37)])
def test_fc_layer_vs_oracle(df8, dnn, oracle, M, K, N):
    x = oracle.fill_normal(M * K, seed=0).reshape(M, K)
    w = oracle.fill_normal(N * K, seed=100, std=0.02).reshape(N, K)
    b = oracle.fill_normal(N, seed=3, std=0.1)
    y = np.zeros((M, N), np.float32)
    df8.dnn_check(dnn.dnn_fc_forward(K, N, p(w), p(b), p(x), M, p(y)))
    xc, xs = oracle.quantize(x, 0)
    wc, ws = oracle.quantize(w, 0)
    assert rel_err(y, oracle.fc_forward_fp8(xc, 0, xs[1], wc, 0, ws[1], b)) <= 2e-4
    assert rel_err(y, oracle.fc_forward_f32(x, w, b)) <= 5e-2


def test_layernorm_layer(df8, dnn, oracle):
    x = oracle.fill_normal(24 * 768, seed=5, mean=0.3, std=2.0).reshape(24, 768)
    g = oracle.fill_normal(768, seed=6, mean=1.0, std=0.1)
    b = oracle.fill_normal(768, seed=7, std=0.1)
    y = np.zeros_like(x)
    df8.dnn_check(dnn.dnn_layernorm_forward(24, 768, p(g), p(b), 1e-5, p(x), p(y)))
    assert np.abs(y - oracle.layernorm(x, g, b)).max() <= 2e-5


def test_softmax_layer_cases(df8, dnn, oracle):
    """ForwardPass / ForwardPassWithMask / MaskedSoftmaxZeroesMaskedPositions of softmax_layer_test.cu."""
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2, 4, 8, 8)).astype(np.float32)
    y = np.zeros_like(x)
    df8.dnn_check(dnn.dnn_softmax_forward(2, 4, 8, p(x), None, 0, p(y)))
    assert np.abs(y - oracle.softmax_masked(x)).max() <= 1e-5
    i, j = np.meshgrid(np.arange(8), np.arange(8), indexing="ij")
    mask = np.where(j <= i, 0.0, -1e9).astype(np.float32)[None, None].repeat(2, axis=0)
    df8.dnn_check(dnn.dnn_softmax_forward(2, 4, 8, p(x), p(mask), 2, p(y)))
    assert np.abs(y - oracle.softmax_masked(x, mask)).max() <= 1e-5
    z = np.zeros((1, 1, 3, 3), np.float32)
    m3 = np.full((1, 1, 3, 3), -1e9, np.float32)
    m3[0, 0, 0, 0] = 0
    out = np.ones_like(z)
    df8.dnn_check(dnn.dnn_softmax_forward(1, 1, 3, p(z), p(m3), 1, p(out)))
    assert abs(out.ravel()[0] - 1) <= 1e-5 and np.abs(out.ravel()[1:]).max() <= 1e-5
    # long rows (T > 1024) take the multi-pass path
    xl = rng.standard_normal((1, 1, 1100, 1100)).astype(np.float32)
    yl = np.zeros_like(xl)
    df8.dnn_check(dnn.dnn_softmax_forward(1, 1, 1100, p(xl), None, 0, p(yl)))
    assert np.abs(yl - oracle.softmax_masked(xl)).max() <= 1e-5


def test_embedding_layers(df8, dnn, oracle):
    V, E, T, B = 50, 48, 9, 2
    table = oracle.fill_normal(V * E, seed=8, std=0.02).reshape(V, E)
    bias = oracle.fill_normal(E, seed=9, std=0.01)
    ids = oracle.fill_token_ids(B * T, seed=2, vocab=V).reshape(B, T)
    y = np.zeros((B, T, E), np.float32)
    df8.dnn_check(dnn.dnn_embedding_forward(V, E, 16, p(table), p(bias), p(ids), B, T, 1, p(y)))
    assert np.array_equal(y, oracle.embed_pe(ids, table, bias, oracle.pe_table(16, E)))
    df8.dnn_check(dnn.dnn_embedding_forward(V, E, 16, p(table), p(bias), p(ids), B, T, 0, p(y)))
    assert np.array_equal(y, oracle.embed_pe(ids, table, bias, None))


def _mha_params(oracle, E, seed):
    return {
        "a.qkv.weight": oracle.fill_normal(3 * E * E, seed=seed, std=0.05).reshape(3 * E, E),
        "a.qkv.bias": oracle.fill_normal(3 * E, seed=seed + 1, std=0.02),
        "a.out.weight": oracle.fill_normal(E * E, seed=seed + 2, std=0.05).reshape(E, E),
        "a.out.bias": oracle.fill_normal(E, seed=seed + 3, std=0.02),
    }


@pytest.mark.parametrize("mask_mode", [0, 1, 2])
def test_mha_layer_vs_oracle(df8, dnn, oracle, mask_mode):
    from oracle import gpt2_ref

    B, T, E, H = 2, 96, 128, 2
    prm = _mha_params(oracle, E, 40)
    x = oracle.fill_normal(B * T * E, seed=44).reshape(B * T, E)
    mask = None
    if mask_mode == 2:  # the causal -1e9 mask upstream's MHA tests build (multi_head_attention_test.cu:50-70)
        i, j = np.meshgrid(np.arange(T), np.arange(T), indexing="ij")
        mask = np.where(j <= i, 0.0, -1e9).astype(np.float32)[None, None].repeat(B, axis=0)
    y = np.zeros((B * T, E), np.float32)
    df8.dnn_check(dnn.dnn_mha_forward(B, T, E, H, p(prm["a.qkv.weight"]), p(prm["a.qkv.bias"]), p(prm["a.out.weight"]),
                                      p(prm["a.out.bias"]), p(x), mask_mode, p(mask), B if mask is not None else 0, p(y)))
    ref = gpt2_ref.mha_forward(prm, "a", x, B, T, H, 0, 0, mask_mode, mask)
    f32 = gpt2_ref.mha_forward(prm, "a", x, B, T, H, None, None, mask_mode, mask)
    assert np.isfinite(y).all()
    assert rel_err(y, ref) <= 3e-2
    assert rel_err(y, f32) <= 1.25 * rel_err(ref, f32) + 2e-3


@pytest.mark.parametrize("gelu,causal", [(0, 0), (1, 0), (1, 1)])
def test_transformer_block_vs_oracle(df8, dnn, oracle, gelu, causal):
    from oracle import gpt2_ref

    B, T, E, H, F = 2, 64, 128, 2, 256
    cfg = dict(vocab=10, hidden=E, ffn=F, layers=1, heads=H, max_seq_len=T)
    prm = gpt2_ref.make_params(cfg, seed=7, std=0.05)
    prm["block0.ln1.gamma"] = oracle.fill_normal(E, seed=70, mean=1.0, std=0.1)
    prm["block0.ln2.beta"] = oracle.fill_normal(E, seed=71, std=0.1)
    order = ["ln1.gamma", "ln1.beta", "ln2.gamma", "ln2.beta", "qkv.weight", "qkv.bias", "out.weight", "out.bias",
             "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"]
    arrays = [np.ascontiguousarray(prm[f"block0.{n}"], dtype=np.float32) for n in order]
    ptrs = (C.c_void_p * 12)(*[a.ctypes.data for a in arrays])
    x = oracle.fill_normal(B * T * E, seed=72).reshape(B * T, E)
    y = np.zeros_like(x)
    df8.dnn_check(dnn.dnn_block_forward(B, T, E, H, F, ptrs, 12, gelu, causal, p(x), p(y)))
    ref = gpt2_ref.block_forward(prm, "block0", x, B, T, H, 0, 0, bool(gelu), 1 if causal else 0)
    f32 = gpt2_ref.block_forward(prm, "block0", x, B, T, H, None, None, bool(gelu), 1 if causal else 0)
    assert rel_err(y, ref) <= 3e-2
    assert rel_err(y, f32) <= 1.25 * rel_err(ref, f32) + 2e-3


@pytest.mark.parametrize("act_kind", [0, 1])
def test_gpt2_logits_vs_oracle(df8, dnn, oracle, cuda, act_kind):
    import torch
    from oracle import gpt2_ref

    cfg = dict(vocab=1000, max_seq_len=128, layers=2, heads=2, hidden=128, ffn=256)
    B, T = 2, 128
    prm = gpt2_ref.make_params(cfg, seed=2, std=0.05)
    ids = oracle.fill_token_ids(B * T, seed=2, vocab=cfg["vocab"]).reshape(B, T)
    df8.dnn_check(dnn.dnn_set_fp8_policy(0, act_kind))
    try:
        model = df8.Gpt2(**cfg)
        model.load_params(prm)
        ids_d = torch.from_numpy(ids).to(cuda)
        ptr = model.forward_logits(ids_d)
        logits = df8.device_view(torch, ptr, (B * T, cfg["vocab"])).cpu().numpy()
        hid = df8.device_view(torch, model.forward_hidden(ids_d), (B * T, cfg["hidden"])).cpu().numpy()
    finally:
        df8.dnn_check(dnn.dnn_set_fp8_policy(0, 0))
    ref_h = gpt2_ref.gpt2_forward(prm, ids, cfg, act_kind=act_kind, return_hidden=True)
    ref = gpt2_ref.gpt2_forward(prm, ids, cfg, act_kind=act_kind)
    f32 = gpt2_ref.gpt2_forward(prm, ids, cfg, act_kind=None, w_kind=None)
    assert np.isfinite(logits).all()
    bound = 5e-2 if act_kind == 0 else 1.5e-1  # e5m2 has 2 mantissa bits: a flipped code is a 25 % step
    assert rel_err(hid, ref_h) <= bound, rel_err(hid, ref_h)
    assert rel_err(logits, ref) <= bound, rel_err(logits, ref)
    assert rel_err(logits, f32) <= 1.25 * rel_err(ref, f32) + 2e-3, (rel_err(logits, f32), rel_err(ref, f32))
    assert df8.status_word() == (0, 0)
    model.close()


def test_gpt2_batch_rows_are_independent_and_deterministic(df8, dnn, oracle, cuda):
    """Batch sharding relies on it: a sequence's hidden states do not depend on which other sequences share
    the batch, except through the per-tensor scales — so compare a batch against itself twice (determinism)
    and the token-based batch-1 entry point against a B=1 batched call."""
    import torch

    cfg = dict(vocab=500, max_seq_len=64, layers=2, heads=2, hidden=128, ffn=256)
    from oracle import gpt2_ref

    prm = gpt2_ref.make_params(cfg, seed=5, std=0.05)
    model = df8.Gpt2(**cfg)
    model.load_params(prm)
    ids = oracle.fill_token_ids(4 * 64, seed=9, vocab=500).reshape(4, 64)
    ids_d = torch.from_numpy(ids).to(cuda)
    a = df8.device_view(torch, model.forward_hidden(ids_d), (4 * 64, 128)).clone()
    b = df8.device_view(torch, model.forward_hidden(ids_d), (4 * 64, 128)).clone()
    assert torch.equal(a, b)
    one = df8.device_view(torch, model.forward_hidden(ids_d[:1].contiguous()), (64, 128)).cpu().numpy()
    host = np.zeros((64, 128), np.float32)
    row = np.ascontiguousarray(ids[0])
    df8.dnn_check(dnn.dnn_gpt2_forward_ids(model.h, p(row), 64, p(host)))
    assert np.array_equal(one, host)
    model.close()


def test_gpt2_save_load_round_trip(df8, dnn, oracle, cuda, tmp_path):
    """SaveLoad of gpt2_test.cu:92-109: parameters equal after save -> load."""
    cfg = dict(vocab=100, max_seq_len=32, layers=1, heads=1, hidden=64, ffn=128)
    model = df8.Gpt2(**cfg)
    path = str(tmp_path / "gpt2.bin").encode()
    df8.dnn_check(dnn.dnn_gpt2_save(model.h, path))
    h2 = dnn.dnn_gpt2_load(path)
    assert h2
    n = dnn.dnn_gpt2_num_params(model.h)
    assert dnn.dnn_gpt2_num_params(h2) == n
    for i, (name, shape) in enumerate(model.param_names()):
        a = np.zeros(int(np.prod(shape)), np.float32)
        b = np.ones_like(a)
        df8.dnn_check(dnn.dnn_gpt2_param_download(model.h, i, p(a)))
        df8.dnn_check(dnn.dnn_gpt2_param_download(h2, i, p(b)))
        assert np.array_equal(a, b), name
    dnn.dnn_gpt2_destroy(h2)
    assert not dnn.dnn_gpt2_load(b"/nonexistent/file.bin")
    model.close()


@pytest.mark.parametrize("slots,release", [(2, False), (3, True), (1, False)])
def test_gpt2_layer_streaming_is_bit_identical(df8, dnn, oracle, cuda, slots, release):
    """Weights streamed per layer from pinned host memory through a ring of device slots must give exactly
    the logits of the resident-weights forward, on repeated forwards (ring wrap-around), on a side stream."""
    import torch
    from oracle import gpt2_ref

    cfg = dict(vocab=300, max_seq_len=64, layers=5, heads=2, hidden=128, ffn=512)
    prm = gpt2_ref.make_params(cfg, seed=11, std=0.05)
    model = df8.Gpt2(**cfg)
    model.load_params(prm)
    ids = torch.from_numpy(oracle.fill_token_ids(3 * 64, seed=4, vocab=300).reshape(3, 64)).to(cuda)
    want = df8.device_view(torch, model.forward_logits(ids), (3 * 64, 300)).clone()
    model.enable_streaming(slots, release)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        model.set_stream(side)
        for _ in range(3):
            got = df8.device_view(torch, model.forward_logits(ids), (3 * 64, 300)).clone()
            assert torch.equal(got, want)
        side.synchronize()
    model.set_stream(torch.cuda.current_stream())
    layer_bytes = (3 * 128 * 128 + 128 * 128 + 2 * 128 * 512)
    assert model.streamed_bytes() >= 3 * 5 * layer_bytes
    # the slots form a ring over the execution order, so a forward uploads every layer exactly once whatever
    # the ratio of layers (5) to slots (2, 3, 1): no layer that is still to be used is ever evicted
    before = model.streamed_bytes()
    with torch.cuda.stream(side):
        model.set_stream(side)
        model.forward_logits(ids)
        side.synchronize()
    model.set_stream(torch.cuda.current_stream())
    assert model.streamed_bytes() - before == 5 * layer_bytes
    h2d, gathered = model.streaming_traffic()
    assert gathered == 0 and h2d == model.streamed_bytes()  # a single rank copies everything itself
    if not release:
        model.disable_streaming()
        again = df8.device_view(torch, model.forward_logits(ids), (3 * 64, 300)).clone()
        assert torch.equal(again, want)
    assert df8.status_word() == (0, 0)
    model.close()


def test_gpt2_device_init_equals_host_generated_params(df8, dnn, oracle, cuda):
    """Gpt2::initialize_on_device(seed) draws every weight matrix on the device from the counter-based streams
    that deepfuse_b200.synthetic.make_gpt2_params (numpy) and the oracle's generator (C) use: the same model, up
    to the last bit of fp32 log / cos."""
    import torch
    from deepfuse_b200 import synthetic

    cfg = dict(vocab=300, max_seq_len=64, layers=2, heads=2, hidden=128, ffn=256)
    want = synthetic.make_gpt2_params(cfg, seed=9, std=0.02)
    df8.dnn_check(dnn.dnn_set_host_init(0))
    try:
        model = df8.Gpt2(**cfg)
    finally:
        df8.dnn_check(dnn.dnn_set_host_init(1))
    model.initialize_on_device(9, 0.02)
    for i, (name, shape) in enumerate(model.param_names()):
        got = np.zeros(int(np.prod(shape)), np.float32)
        df8.dnn_check(dnn.dnn_gpt2_param_download(model.h, i, p(got)))
        if name.endswith("gamma") or name.endswith("beta"):
            continue
        assert np.allclose(got, want[name].ravel(), rtol=0, atol=1e-7), name
    ids = torch.from_numpy(oracle.fill_token_ids(2 * 64, seed=1, vocab=300).reshape(2, 64)).to(cuda)
    ptr, pitch = model.forward_logits_pitched(ids)
    assert pitch == 320
    pitched = df8.device_view(torch, ptr, (128, pitch))[:, :300].clone()
    dense = df8.device_view(torch, model.forward_logits(ids), (128, 300)).clone()
    assert torch.equal(pitched, dense)
    host = torch.empty((128, 300), dtype=torch.float32).pin_memory()
    model.copy_logits_host(host)
    torch.cuda.synchronize()
    assert torch.equal(host, dense.cpu())
    model.set_stage_timing(True)
    model.forward_logits_pitched(ids)
    assert 0.0 < model.last_head_ms() < 50.0
    model.close()


def test_gpt2_serve_step_equals_forward_then_copy(df8, dnn, oracle, cuda):
    """Gpt2.serve_step (host ids in, full logits to pinned host memory with the copy on a stream of its own, two
    buffers alternating) returns the logits of forward_logits_pitched + copy_logits_host, step after step with
    different ids."""
    import torch
    from oracle import gpt2_ref

    cfg = dict(vocab=300, max_seq_len=32, layers=2, heads=2, hidden=128, ffn=256)
    B, T, steps = 3, 32, 5
    prm = gpt2_ref.make_params(cfg, seed=12, std=0.05)
    model = df8.Gpt2(**cfg)
    try:
        model.load_params(prm)
        ids = [torch.from_numpy(oracle.fill_token_ids(B * T, seed=20 + i, vocab=300).reshape(B, T)).pin_memory() for i in range(steps)]
        want = []
        for x in ids:
            dst = torch.empty((B * T, 300), dtype=torch.float32).pin_memory()
            model.forward_logits_pitched(x, check_ids=False)
            model.copy_logits_host(dst)
            torch.cuda.synchronize()
            want.append(dst.clone())
        bufs = [torch.full((B * T, 300), float("nan"), dtype=torch.float32).pin_memory() for _ in range(2)]
        got = []
        for i, x in enumerate(ids):
            model.serve_step(x, bufs[i % 2])
            if i >= 1:  # the copy of step i - 1 is over once step i's forward has been issued and its event waited for
                model.serve_flush()
                torch.cuda.synchronize()
                got.append(bufs[(i - 1) % 2].clone())
        model.serve_flush()
        torch.cuda.synchronize()
        got.append(bufs[(steps - 1) % 2].clone())
        for i, (g, w) in enumerate(zip(got, want)):
            assert torch.equal(g, w), i
        assert df8.status_word() == (0, 0)
    finally:
        model.close()
