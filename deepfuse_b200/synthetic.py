"""Seeded synthetic inputs for the benchmark and the examples: weights ~N(0, std), token ids uniform in [0, vocab),
activations ~N(0,1) with a fraction of outliers.  Counter-based (splitmix64 of (seed, index) -> Box-Muller), so any
slice of a tensor can be generated on its own and every rank of a multi-GPU run can make exactly its share.

numpy only.  The test suite's CPU oracle carries the same generator in C; tests/test_synthetic.py holds the two to
each other (token ids bit for bit, normals to fp32 rounding of log / cos).
"""
from __future__ import annotations

import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_SEED_MUL = np.uint64(0xD1342543DE82EF95)
_ID_MUL = np.uint64(0x2545F4914F6CDD1D)
_CHUNK = 1 << 22


def _mix64(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z + _GOLD
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def _u01(bits: np.ndarray) -> np.ndarray:
    return ((bits >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)


def _normal_at(seed: int, idx: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        base = np.uint64(seed) * _SEED_MUL
        a = _mix64(base + np.uint64(2) * idx)
        b = _mix64(base + np.uint64(2) * idx + np.uint64(1))
    r = np.sqrt(np.float32(-2.0) * np.log(_u01(a)))
    return (r * np.cos(np.float32(6.28318530718) * _u01(b))).astype(np.float32)


def fill_normal(n: int, seed: int, mean: float = 0.0, std: float = 1.0, offset: int = 0) -> np.ndarray:
    """n values ~N(mean, std): elements offset .. offset+n-1 of the stream `seed`."""
    out = np.empty(n, dtype=np.float32)
    for lo in range(0, n, _CHUNK):
        hi = min(n, lo + _CHUNK)
        idx = np.arange(offset + lo, offset + hi, dtype=np.uint64)
        out[lo:hi] = np.float32(mean) + np.float32(std) * _normal_at(seed, idx)
    return out


def fill_normal_outliers(n: int, seed: int, frac: float = 1e-3, outlier_scale: float = 100.0) -> np.ndarray:
    """N(0,1) with a fraction `frac` of the positions replaced by outlier_scale * N(0,1)."""
    out = np.empty(n, dtype=np.float32)
    for lo in range(0, n, _CHUNK):
        hi = min(n, lo + _CHUNK)
        idx = np.arange(lo, hi, dtype=np.uint64)
        v = _normal_at(seed, idx)
        with np.errstate(over="ignore"):
            pick = _u01(_mix64(np.uint64(seed) ^ np.uint64(0xA5A5A5A5) ^ (idx * _GOLD))) < np.float32(frac)
        big = np.float32(outlier_scale) * _normal_at(seed + 0x51ED27, idx)
        out[lo:hi] = np.where(pick, big, v)
    return out


def fill_token_ids(n: int, seed: int, vocab: int) -> np.ndarray:
    """n token ids uniform in [0, vocab)."""
    with np.errstate(over="ignore"):
        z = _mix64(np.uint64(seed) * _ID_MUL + np.arange(n, dtype=np.uint64))
    return (z % np.uint64(vocab)).astype(np.int32)


def make_gpt2_params(cfg: dict, seed: int, std: float = 0.02) -> dict:
    """Seeded N(0, std) weights, zero biases, LayerNorm gamma 1 / beta 0 for a GPT-2 of the given sizes
    (vocab, hidden, ffn, layers), keyed by the parameter names of include/df8_dnn.h (dnn_gpt2_param_info)."""
    V, E, F, L = cfg["vocab"], cfg["hidden"], cfg["ffn"], cfg["layers"]
    p = {}
    k = [seed * 1000]

    def normal(shape):
        k[0] += 1
        return fill_normal(int(np.prod(shape)), seed=k[0], std=std).reshape(shape)

    p["embedding.weight"] = normal((V, E))
    p["embedding.bias"] = np.zeros(E, np.float32)
    for i in range(L):
        b = f"block{i}"
        for ln in ("ln1", "ln2"):
            p[f"{b}.{ln}.gamma"] = np.ones(E, np.float32)
            p[f"{b}.{ln}.beta"] = np.zeros(E, np.float32)
        for name, shape in (("qkv", (3 * E, E)), ("out", (E, E)), ("fc1", (F, E)), ("fc2", (E, F))):
            p[f"{b}.{name}.weight"] = normal(shape)
            p[f"{b}.{name}.bias"] = np.zeros(shape[0], np.float32)
    p["final_fc.weight"] = normal((V, E))
    p["final_fc.bias"] = np.zeros(V, np.float32)
    return p
