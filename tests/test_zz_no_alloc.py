"""The allocation-free LayerNorm + quantise entry point (df8_layernorm_quantize_f32_noalloc).

It serves callers that cannot hand the library a scratch buffer because they cannot allocate on the device
when they call (everything already sits in their own arena, or they may not block on the allocator): the
per-row scratch is a fixed array inside the library.  The result must be identical to the entry point that
takes a caller-provided scratch buffer, also on a second call that reuses the same built-in array with
different data.  This file sorts last on purpose: the array is shared by every call in the process, so the test
also shows that whatever the earlier tests ran has left it usable."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _both(df8, torch, dev, x, g, b, kind):
    rows, cols = x.shape
    xd, gd, bd = (torch.from_numpy(a).to(dev) for a in (x, g, b))
    out = []
    for use_builtin in (False, True):
        codes = torch.full((rows, cols), 0xAA, dtype=torch.uint8, device=dev)
        scale, amax = torch.zeros(2, device=dev), torch.full((1,), -1.0, device=dev)
        if use_builtin:
            df8.layernorm_quantize_f32_noalloc(xd, rows, cols, gd, bd, 1e-5, kind, codes, scale, amax)
        else:
            stats = torch.zeros(2 * rows, device=dev)
            df8.layernorm_quantize_f32(xd, rows, cols, gd, bd, 1e-5, kind, codes, scale, amax, stats)
        torch.cuda.synchronize()
        out.append((codes, scale, amax))
    return out


@pytest.mark.parametrize("kind", [0, 1])
def test_noalloc_matches_scratch_variant_twice_in_a_row(df8, oracle, cuda, kind):
    import torch

    for call, (rows, cols, seed) in enumerate([(300, 768, 1), (129, 1024, 2)]):  # second call: other shape and data
        x = oracle.fill_normal(rows * cols, seed=seed, mean=0.2, std=1.7).reshape(rows, cols)
        g = oracle.fill_normal(cols, seed=seed + 10, mean=1.0, std=0.1)
        b = oracle.fill_normal(cols, seed=seed + 20, std=0.1)
        (c0, s0, a0), (c1, s1, a1) = _both(df8, torch, cuda, x, g, b, kind)
        assert a0.item() == a1.item() and a1.item() > 0, f"call {call}"
        assert torch.equal(s0, s1), f"call {call}"
        assert torch.equal(c0, c1), f"call {call}: {(c0 != c1).sum().item()} codes differ"


def test_noalloc_rejects_more_rows_than_the_builtin_scratch(df8, cuda, monkeypatch):
    import torch

    # 65536 rows of 4 columns would qualify for the one-launch kernel that keeps the rows in shared memory and
    # needs no row scratch at all; switch it off (the variable is read at every call) so that both entry points
    # take the two-kernel path and the built-in array is written and read over its whole extent
    monkeypatch.setenv("DF8_LN_RESIDENT", "0")

    x = torch.zeros(16, device=cuda)
    codes = torch.zeros(16, dtype=torch.uint8, device=cuda)
    s, a = torch.zeros(2, device=cuda), torch.zeros(1, device=cuda)
    with pytest.raises(df8.Df8Error, match="exceed the built-in scratch"):
        df8.layernorm_quantize_f32_noalloc(x, 65537, 16, None, None, 1e-5, 0, codes, s, a)
    # the limit itself is accepted (rows = 65536 of 4 columns)
    n = 65536
    xb = torch.randn(n, 4, device=cuda)
    cb = torch.zeros(n, 4, dtype=torch.uint8, device=cuda)
    df8.layernorm_quantize_f32_noalloc(xb, n, 4, None, None, 1e-5, 0, cb, s, a)
    stats = torch.zeros(2 * n, device=cuda)
    cb2, s2, a2 = torch.zeros_like(cb), torch.zeros(2, device=cuda), torch.zeros(1, device=cuda)
    df8.layernorm_quantize_f32(xb, n, 4, None, None, 1e-5, 0, cb2, s2, a2, stats)
    assert torch.equal(cb, cb2) and torch.equal(s, s2)
