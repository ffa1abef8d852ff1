"""GPU parity of LayerNorm (plain and fused with the quantiser) and of embedding + positional encoding."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _t(torch, a, dev):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(dev)


@pytest.mark.parametrize("rows,cols", [(1, 4), (7, 48), (64, 768), (33, 1024), (5, 4096), (9, 770), (3, 5000), (4, 8192)])
@pytest.mark.parametrize("affine", [True, False])
def test_layernorm_vs_oracle(df8, oracle, cuda, rows, cols, affine):
    """fp32 LayerNorm; tolerance 2e-5 absolute (reduction order differs from the serial host loop)."""
    import torch

    x = oracle.fill_normal(rows * cols, seed=rows + cols, mean=0.5, std=2.0).reshape(rows, cols)
    g = oracle.fill_normal(cols, seed=1, mean=1.0, std=0.2) if affine else None
    b = oracle.fill_normal(cols, seed=2, std=0.2) if affine else None
    y = torch.full((rows, cols), float("nan"), device=cuda)
    amax = torch.full((1,), -1.0, device=cuda)
    df8.layernorm_f32(_t(torch, x, cuda), rows, cols, _t(torch, g, cuda), _t(torch, b, cuda), 1e-5, y, amax)
    ref = oracle.layernorm(x, g, b, 1e-5)
    got = y.cpu().numpy()
    assert np.abs(got - ref).max() <= 2e-5
    assert amax.item() == np.abs(got).max()


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("rows,cols", [(64, 768), (130, 1024), (17, 4096), (9, 770), (32, 768), (5, 768), (1, 256), (17, 1024),
                                       (32, 520), (33, 768)])
def test_layernorm_quantize_vs_oracle(df8, oracle, cuda, kind, rows, cols):
    """Fused LN + quantise.  The codes are those of quantising the kernel's own LayerNorm output (bit-exact,
    checked through df8_layernorm_f32 + df8_quantize_f32); against the oracle's LayerNorm, whose row sums
    run in a different order, codes may differ by one step on a few elements.  Up to 32 rows of at most 1024
    columns take the one-CTA kernel (a decode step's shape)."""
    import torch

    x = oracle.fill_normal(rows * cols, seed=3 * rows + cols, std=1.5).reshape(rows, cols)
    g = oracle.fill_normal(cols, seed=4, mean=1.0, std=0.1)
    b = oracle.fill_normal(cols, seed=5, std=0.1)
    xd, gd, bd = _t(torch, x, cuda), _t(torch, g, cuda), _t(torch, b, cuda)
    codes = torch.full((rows, cols), 0xAA, dtype=torch.uint8, device=cuda)
    scale, amax = torch.zeros(2, device=cuda), torch.zeros(1, device=cuda)
    stats = torch.zeros(2 * rows, device=cuda)
    df8.layernorm_quantize_f32(xd, rows, cols, gd, bd, 1e-5, kind, codes, scale, amax, stats)
    # unfused chain on the GPU
    y = torch.empty((rows, cols), device=cuda)
    amax2, scale2 = torch.zeros(1, device=cuda), torch.zeros(2, device=cuda)
    codes2 = torch.empty_like(codes)
    df8.layernorm_f32(xd, rows, cols, gd, bd, 1e-5, y, amax2)
    df8.quantize_f32(y, kind, amax2, codes2, scale2)
    assert amax.item() == amax2.item()
    assert torch.equal(scale, scale2)
    assert torch.equal(codes, codes2)
    # against the oracle
    ref = oracle.layernorm(x, g, b, 1e-5)
    rc, rs = oracle.quantize(ref, kind)
    assert abs(amax.item() - oracle.amax(ref)) <= 1e-5 * oracle.amax(ref)
    got = oracle.dequantize(codes.cpu().numpy(), kind, float(scale[1].item()))
    want = oracle.dequantize(rc, kind, rs[1])
    assert (codes.cpu().numpy() != rc).mean() < 0.01
    step = 2.0 ** (-3 if kind == 0 else -2)
    assert np.all(np.abs(got - want) <= step * np.maximum(np.abs(want), 1e-3) + 1e-6)


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("rows,cols,affine", [(8192, 768, True), (4096, 1024, False), (1500, 256, True), (1024, 520, True)])
def test_layernorm_quantize_resident_path_equals_two_kernel_path(df8, oracle, cuda, monkeypatch, kind, rows, cols, affine):
    """Activations that fit the GPU's shared memory take the one-launch kernel (rows normalised into shared memory,
    grid-wide barrier, codes from shared memory); it must give the codes, scale and amax of the two-kernel path bit
    for bit, repeatedly (the barrier counters are reused) and without touching the status word."""
    import torch

    x = oracle.fill_normal(rows * cols, seed=rows + cols, std=2.0).reshape(rows, cols)
    g = oracle.fill_normal(cols, seed=4, mean=1.0, std=0.1) if affine else None
    b = oracle.fill_normal(cols, seed=5, std=0.1) if affine else None
    xd = _t(torch, x, cuda)
    gd = _t(torch, g, cuda) if affine else None
    bd = _t(torch, b, cuda) if affine else None

    def run():
        codes = torch.full((rows, cols), 0xAA, dtype=torch.uint8, device=cuda)
        scale, amax = torch.zeros(2, device=cuda), torch.zeros(1, device=cuda)
        stats = torch.zeros(2 * rows, device=cuda)
        df8.layernorm_quantize_f32(xd, rows, cols, gd, bd, 1e-5, kind, codes, scale, amax, stats)
        torch.cuda.synchronize()
        return codes, scale, amax

    monkeypatch.setenv("DF8_LN_RESIDENT", "0")
    c0, s0, a0 = run()
    monkeypatch.delenv("DF8_LN_RESIDENT")
    for _ in range(3):
        c1, s1, a1 = run()
        assert a1.item() == a0.item() and torch.equal(s1, s0) and torch.equal(c1, c0)
    assert df8.status_word() == (0, 0)


@pytest.mark.parametrize("B,T,E,V", [(2, 5, 8, 11), (8, 64, 768, 50257), (1, 7, 30, 100)])
def test_embed_pe_vs_oracle(df8, oracle, cuda, B, T, E, V):
    import torch

    table = oracle.fill_normal(V * E, seed=6, std=0.02).reshape(V, E)
    bias = oracle.fill_normal(E, seed=7, std=0.01)
    pe = oracle.pe_table(T + 3, E)
    ids = oracle.fill_token_ids(B * T, seed=2, vocab=V).reshape(B, T)
    out = torch.full((B, T, E), float("nan"), device=cuda)
    bad = torch.full((1,), 99, dtype=torch.int32, device=cuda)
    df8.embed_pe_f32(_t(torch, ids, cuda), B, T, E, V, _t(torch, table, cuda), _t(torch, bias, cuda),
                     _t(torch, pe, cuda), out, bad)
    assert bad.item() == 0
    assert np.array_equal(out.cpu().numpy(), oracle.embed_pe(ids, table, bias, pe))  # same fp32 adds, same order


def test_embed_counts_invalid_ids(df8, oracle, cuda):
    import torch

    V, E = 10, 8
    table = torch.ones(V, E, device=cuda)
    ids = torch.tensor([[0, 3, V, -1]], dtype=torch.int32, device=cuda)
    out = torch.full((1, 4, E), float("nan"), device=cuda)
    bad = torch.zeros(1, dtype=torch.int32, device=cuda)
    df8.embed_pe_f32(ids, 1, 4, E, V, table, None, None, out, bad)
    assert bad.item() == 2
    assert out[0, 2].abs().sum().item() == 0 and out[0, 3].abs().sum().item() == 0 and out[0, 1].sum().item() == E
