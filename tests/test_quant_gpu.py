"""GPU parity of amax / quantise / dequantise against the CPU oracle: bit-exact codes."""
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _run_quant(df8, torch, x_host, kind, dev):
    x = torch.from_numpy(x_host).to(dev)
    amax = torch.full((1,), -1.0, device=dev)
    codes = torch.full((max(x.numel(), 1),), 0xAA, dtype=torch.uint8, device=dev)
    scale = torch.zeros(2, device=dev)
    df8.amax_f32(x, amax)
    df8.quantize_f32(x, kind, amax, codes, scale)
    y = torch.full((max(x.numel(), 1),), float("nan"), device=dev)
    df8.dequantize_f32(codes[: x.numel()], kind, scale, y)
    torch.cuda.synchronize()
    n = x.numel()
    return amax.item(), codes.cpu().numpy()[:n], scale.cpu().numpy(), y.cpu().numpy()[:n]


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 15, 16, 17, 1023, 4096 + 7, 1 << 20, (1 << 22) + 3])
def test_quantise_bit_exact_vs_oracle(df8, oracle, cuda, kind, n):
    import torch

    x = oracle.fill_normal_outliers(n, seed=1)
    amax, codes, scale, y = _run_quant(df8, torch, x, kind, cuda)
    assert amax == oracle.amax(x)
    ref_codes, ref_scale = oracle.quantize(x, kind)
    assert np.array_equal(scale, ref_scale)
    assert np.array_equal(codes, ref_codes), f"{(codes != ref_codes).sum()} code mismatches"
    assert np.array_equal(y, oracle.dequantize(ref_codes, kind, ref_scale[1]))


@pytest.mark.parametrize("kind,name", [(0, "e4m3"), (1, "e5m2")])
def test_quantise_matches_committed_golden(df8, cuda, kind, name):
    import torch

    g = np.load(GOLDEN / "quant_golden.npz")
    amax, codes, scale, y = _run_quant(df8, torch, g["x"], kind, cuda)
    assert np.array_equal(codes, g[f"codes_{name}"])
    assert np.array_equal(scale, g[f"scale_{name}"])
    assert np.array_equal(y, g[f"deq_{name}"])


@pytest.mark.parametrize("kind,name", [(0, "e4m3"), (1, "e5m2")])
def test_decode_of_every_code(df8, cuda, kind, name):
    import torch

    table = np.load(GOLDEN / "fp8_code_values.npz")[name]
    codes = torch.arange(256, dtype=torch.uint8, device=cuda)
    scale = torch.ones(2, device=cuda)
    y = torch.zeros(256, device=cuda)
    df8.dequantize_f32(codes, kind, scale, y)
    got = y.cpu().numpy()
    assert np.array_equal(np.isnan(got), np.isnan(table))
    ok = ~np.isnan(table)
    assert np.array_equal(got[ok], table[ok])


@pytest.mark.parametrize("kind", [0, 1])
def test_special_values(df8, oracle, cuda, kind):
    """Saturation, signed zero, subnormals, infinities and NaN follow cuda_fp8.h."""
    import torch

    fmax = oracle.FP8_MAX[kind]
    x = np.array([0.0, -0.0, fmax, -fmax, fmax * 1.0001, 1e30, -1e30, np.inf, -np.inf, np.nan, 2.0 ** -9, 2.0 ** -10,
                  2.0 ** -16, 2.0 ** -17, 1.5 * 2.0 ** -16, 17, 18, 19, 0.3], dtype=np.float32)
    xd = torch.from_numpy(x).to(cuda)
    amax = torch.tensor([fmax], device=cuda)  # q == 1: conversion alone
    codes = torch.zeros(x.size, dtype=torch.uint8, device=cuda)
    scale = torch.zeros(2, device=cuda)
    df8.quantize_f32(xd, kind, amax, codes, scale)
    ref, _ = oracle.quantize(x, kind, amax_v=fmax)
    assert np.array_equal(codes.cpu().numpy(), ref)


def test_amax_ignores_nan_and_zero_tensor(df8, cuda):
    import torch

    x = torch.tensor([1.0, float("nan"), -3.0, 2.0], device=cuda)
    amax = torch.zeros(1, device=cuda)
    df8.amax_f32(x, amax)
    assert amax.item() == 3.0
    z = torch.zeros(1000, device=cuda)
    codes = torch.ones(1000, dtype=torch.uint8, device=cuda)
    scale = torch.zeros(2, device=cuda)
    df8.amax_f32(z, amax)
    df8.quantize_f32(z, 0, amax, codes, scale)
    assert amax.item() == 0.0 and scale.tolist() == [1.0, 1.0] and not codes.any().item()


def test_amax_preclear_switch(df8, cuda):
    """With the per-call clearing off the caller owns the zeroing: a slot keeps accumulating the maximum
    until the caller clears it; the switch is per thread and returns the previous setting."""
    import torch

    a = torch.tensor([1.0, -2.0, 0.5, 0.25], device=cuda)
    b = torch.tensor([0.5, 0.25, -1.5, 1.0], device=cuda)
    slot = torch.zeros(1, device=cuda)
    lib = df8.lib()
    assert lib.df8_set_amax_preclear(0) == 1
    try:
        df8.amax_f32(a, slot)
        df8.amax_f32(b, slot)
        assert slot.item() == 2.0  # not cleared in between
        slot.zero_()
        df8.amax_f32(b, slot)
        assert slot.item() == 1.5
    finally:
        assert lib.df8_set_amax_preclear(1) == 0
    df8.amax_f32(b, slot)
    df8.amax_f32(torch.zeros(4, device=cuda), slot)
    assert slot.item() == 0.0  # cleared by the call again


@pytest.mark.parametrize("kind", [0, 1])
def test_large_tensor_properties(df8, oracle, cuda, kind):
    """2^28 elements: amax equals torch's, the round trip is idempotent, and a strided sample of the
    codes matches the oracle bit for bit."""
    import torch

    n = 1 << 28
    g = torch.Generator(device=cuda)
    g.manual_seed(1)
    x = torch.randn(n, device=cuda, generator=g)
    idx = torch.randint(0, n, (n // 1000,), device=cuda, generator=g)
    x[idx] = 100.0 * torch.randn(idx.numel(), device=cuda, generator=g)
    amax = torch.zeros(1, device=cuda)
    codes = torch.empty(n, dtype=torch.uint8, device=cuda)
    scale = torch.zeros(2, device=cuda)
    y = torch.empty(n, device=cuda)
    df8.amax_f32(x, amax)
    df8.quantize_f32(x, kind, amax, codes, scale)
    df8.dequantize_f32(codes, kind, scale, y)
    assert amax.item() == x.abs().max().item()
    codes2 = torch.empty_like(codes)
    df8.quantize_f32(y, kind, amax, codes2, scale)
    assert torch.equal(codes, codes2)
    sample = slice(12345, n, 4099)
    xs = x[sample].cpu().numpy()
    ref, _ = oracle.quantize(xs, kind, amax_v=amax.item())
    assert np.array_equal(codes[sample].cpu().numpy(), ref)
    # relative error of the round trip is bounded by half an ulp of the format for normal values
    rel = ((y - x).abs() / x.abs().clamp_min(1e-30))[x.abs() > amax.item() * 2.0 ** -5]
    assert rel.max().item() <= (2.0 ** -4 if kind == 0 else 2.0 ** -3) * 1.0001
