"""The benchmark's input generator (deepfuse_b200/synthetic.py, numpy) against the oracle's (C): the same
counter-based streams.  Token ids are integers and must agree bit for bit; the normals pass through fp32 log and
cos, whose last bit may differ between numpy and libm."""
import numpy as np

from deepfuse_b200 import synthetic


def test_token_ids_equal_the_oracles(oracle):
    for seed, vocab, n in [(2, 50257, 8192), (100, 50257, 1000), (4, 1000, 77)]:
        assert np.array_equal(synthetic.fill_token_ids(n, seed, vocab), oracle.fill_token_ids(n, seed=seed, vocab=vocab))


def test_normals_equal_the_oracles(oracle):
    a = synthetic.fill_normal(100000, seed=2001, std=0.02)
    b = oracle.fill_normal(100000, seed=2001, std=0.02)
    assert np.allclose(a, b, rtol=0, atol=0.02 * 2e-6)
    assert np.array_equal(synthetic.fill_normal(1000, seed=7, offset=500), synthetic.fill_normal(1500, seed=7)[500:])
    x = synthetic.fill_normal_outliers(1 << 18, seed=1)
    y = oracle.fill_normal_outliers(1 << 18, seed=1)
    assert np.allclose(x, y, rtol=0, atol=100 * 2e-6)
    assert 1e-4 < (np.abs(x) > 6).mean() < 3e-3  # the outliers are there


def test_gpt2_params_equal_the_oracles(oracle):
    from oracle import gpt2_ref

    cfg = dict(vocab=300, max_seq_len=32, layers=2, heads=2, hidden=64, ffn=128)
    a, b = synthetic.make_gpt2_params(cfg, seed=3), gpt2_ref.make_params(cfg, seed=3)
    assert list(a) == list(b)
    for k in a:
        assert a[k].shape == b[k].shape and np.allclose(a[k], b[k], rtol=0, atol=1e-7), k
