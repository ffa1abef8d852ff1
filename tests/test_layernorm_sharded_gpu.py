"""LayerNorm + quantise of a tensor whose columns are split across ranks (df8_layernorm_shard_*), on ONE GPU: the
pieces of g emulated ranks are processed one after the other and the two exchanges (row statistics, maximum) are
done by hand.  The result must agree with the single-GPU fused kernel and with the oracle up to the order of the
additions: the scale to 1e-6, all but a few codes identical, those few one step apart."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,g,kind", [(300, 512, 2, 0), (1024, 4096, 8, 0), (77, 1024, 4, 1), (129, 256, 2, 0)])
def test_sharded_layernorm_matches_the_unsharded_kernel(df8, oracle, cuda, rows, cols, g, kind):
    import torch

    n = cols // g
    x = oracle.fill_normal(rows * cols, seed=rows + g, mean=0.3, std=1.7).reshape(rows, cols)
    x[:, :n] += 2.0  # pieces with different means: the combination formula has something to do
    gam = oracle.fill_normal(cols, seed=5, mean=1.0, std=0.1)
    bet = oracle.fill_normal(cols, seed=6, std=0.1)
    xd, gd, bd = (torch.from_numpy(a).to(cuda) for a in (x, gam, bet))
    lib, st = df8.lib(), df8.stream_ptr()
    pieces = [xd[:, r * n:(r + 1) * n].contiguous() for r in range(g)]
    partial_all = torch.zeros((g, rows, 2), device=cuda)
    for r in range(g):
        df8.check(lib.df8_layernorm_shard_stats_f32(df8.ptr(pieces[r]), rows, n, df8.ptr(partial_all[r]), st))
    row_stats = torch.zeros((rows, 2), device=cuda)
    amaxes = torch.zeros(g, device=cuda)
    for r in range(g):
        df8.check(lib.df8_layernorm_shard_amax_f32(df8.ptr(pieces[r]), rows, n, df8.ptr(partial_all), g,
                                                   df8.ptr(gd[r * n:]), df8.ptr(bd[r * n:]), 1e-5, df8.ptr(row_stats),
                                                   df8.ptr(amaxes[r:]), st))
    amax = amaxes.max().reshape(1).clone()
    codes = torch.zeros((rows, cols), dtype=torch.uint8, device=cuda)
    scale = torch.zeros(2, device=cuda)
    for r in range(g):
        piece_codes = torch.zeros((rows, n), dtype=torch.uint8, device=cuda)
        df8.check(lib.df8_layernorm_shard_quantize_f32(df8.ptr(pieces[r]), rows, n, df8.ptr(row_stats), df8.ptr(gd[r * n:]),
                                                       df8.ptr(bd[r * n:]), kind, df8.ptr(amax), df8.ptr(piece_codes),
                                                       df8.ptr(scale), st))
        codes[:, r * n:(r + 1) * n] = piece_codes
    # the single-GPU fused kernel
    want = torch.zeros((rows, cols), dtype=torch.uint8, device=cuda)
    wscale, wamax, stats = torch.zeros(2, device=cuda), torch.zeros(1, device=cuda), torch.zeros(2 * rows, device=cuda)
    df8.layernorm_quantize_f32(xd, rows, cols, gd, bd, 1e-5, kind, want, wscale, wamax, stats)
    torch.cuda.synchronize()
    assert abs(amax.item() / wamax.item() - 1) <= 2e-6
    assert abs(scale[0].item() / wscale[0].item() - 1) <= 2e-6
    a, b = codes.cpu().numpy(), want.cpu().numpy()
    diff = a != b
    assert diff.mean() <= 2e-3, f"{diff.mean():.2e} of the codes differ"
    if diff.any():
        assert (np.abs(a[diff].astype(np.int16) - b[diff].astype(np.int16)) == 1).all()
    # and the oracle: LayerNorm rows, per-tensor quantiser
    ref_codes, ref_scale = oracle.quantize(oracle.layernorm(x, gam, bet, 1e-5), kind)
    assert abs(scale[1].item() / ref_scale[1] - 1) <= 1e-5
    assert (a != ref_codes).mean() <= 2e-3
