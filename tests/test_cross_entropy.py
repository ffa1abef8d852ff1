"""Softmax cross-entropy on the logits (the training-side neighbour of the vocabulary head).

CPU: the oracle's restatement against upstream's own known-answer cases (tests/losses/cross_entropy_test.cu:68-119:
one row {2, 1, 0.1, 0.5} with class 0 as the target, loss and gradient against the textbook formula at 1e-5; :122-155
the {100, -100, 0, 0} row stays finite; :158-205 ten classes).
GPU: df8_cross_entropy_f32 / dnn::CrossEntropyLoss against the oracle at upstream's tolerance (1e-5 absolute on the
loss and on every gradient element), dense and index targets, dense and pitched rows, the head's class count; and
against upstream's own CrossEntropyLoss compiled from its sources (oracle/_ref), where that library was built."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

REF_LIB = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libdnn_ref.so"


def textbook(x, t):
    x = x.astype(np.float64)
    z = x - x.max(axis=1, keepdims=True)
    p = np.exp(z) / np.exp(z).sum(axis=1, keepdims=True)
    return float(-(t * np.log(p)).sum(axis=1).mean()), p - t


def test_oracle_reproduces_upstreams_known_answers(oracle):
    x = np.array([[2.0, 1.0, 0.1, 0.5]], np.float32)
    t = np.array([[1.0, 0.0, 0.0, 0.0]], np.float32)
    loss, rows, grad = oracle.cross_entropy(x, targets=t)
    want_loss, want_grad = textbook(x, t)
    assert abs(loss - want_loss) <= 1e-5 and np.abs(grad - want_grad).max() <= 1e-5
    assert abs(loss - 0.5542174) <= 1e-5  # -log softmax({2, 1, 0.1, 0.5})[0]
    loss_i, _, grad_i = oracle.cross_entropy(x, target_idx=[0])
    assert loss_i == loss and np.array_equal(grad_i, grad)
    # the edge case of upstream's test: finite, and the loss of an (almost) certain right answer is ~0
    x = np.array([[100.0, -100.0, 0.0, 0.0]], np.float32)
    loss, _, grad = oracle.cross_entropy(x, targets=t)
    assert np.isfinite(loss) and np.isfinite(grad).all() and abs(loss) <= 1e-6
    # ten classes, target 5
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, (1, 10)).astype(np.float32)
    t = np.zeros((1, 10), np.float32)
    t[0, 5] = 1.0
    loss, _, grad = oracle.cross_entropy(x, targets=t)
    want_loss, want_grad = textbook(x, t)
    assert abs(loss - want_loss) <= 1e-5 and np.abs(grad - want_grad).max() <= 1e-5


def test_oracle_soft_targets_and_many_rows(oracle):
    rng = np.random.default_rng(1)
    x = rng.normal(0, 3, (37, 101)).astype(np.float32)
    t = rng.dirichlet(np.ones(101), 37).astype(np.float32)
    loss, rows, grad = oracle.cross_entropy(x, targets=t)
    want_loss, want_grad = textbook(x, t)
    assert abs(loss - want_loss) <= 1e-5 * max(1.0, abs(want_loss)) and np.abs(grad - want_grad).max() <= 1e-5
    assert rows.shape == (37,)
    with pytest.raises(ValueError):
        oracle.cross_entropy(x)


def _gpu_ce(df8, torch, cuda, x, t=None, idx=None, pitch=None, want_grad=True):
    rows, Cn = x.shape
    pitch = pitch or Cn
    buf = np.full((rows, pitch), 1e30, np.float32)  # the padding must never be read
    buf[:, :Cn] = x
    xd = torch.from_numpy(buf).to(cuda)
    td = torch.from_numpy(t).to(cuda) if t is not None else None
    idd = torch.from_numpy(np.asarray(idx, np.int32)).to(cuda) if idx is not None else None
    loss = C.c_float(0)
    grad = torch.full((rows, Cn), 7.0, device=cuda) if want_grad else None
    df8.dnn_check(df8.dnn_lib().dnn_cross_entropy(df8.ptr(xd), rows, Cn, pitch, df8.ptr(td), df8.ptr(idd), C.byref(loss),
                                                  df8.ptr(grad)), "dnn_cross_entropy")
    return loss.value, (grad.cpu().numpy() if want_grad else None)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,Cn,pitch", [(1, 4, None), (5, 10, None), (64, 1000, None), (33, 1003, 1004), (7, 50257, 50272),
                                           (300, 50257, None)])
def test_cross_entropy_matches_the_oracle(df8, oracle, cuda, rows, Cn, pitch):
    import torch

    df8.dnn_check(df8.dnn_lib().dnn_init(0))
    x = oracle.fill_normal(rows * Cn, seed=rows + Cn, std=2.0).reshape(rows, Cn)
    if rows == 1:
        x = np.array([[2.0, 1.0, 0.1, 0.5]], np.float32)
    idx = oracle.fill_token_ids(rows, seed=9, vocab=Cn)
    want_loss, _, want_grad = oracle.cross_entropy(x, target_idx=idx)
    loss, grad = _gpu_ce(df8, torch, cuda, x, idx=idx, pitch=pitch)
    # upstream's tolerance (cross_entropy_test.cu:89,118); the sums run in another order here (strided + tree)
    assert abs(loss - want_loss) <= 1e-5 * max(1.0, abs(want_loss)), (loss, want_loss)
    assert np.abs(grad - want_grad).max() <= 1e-5
    if pitch is None and rows * Cn <= 100000:  # upstream's form: dense one-hot and soft targets
        t = np.zeros((rows, Cn), np.float32)
        t[np.arange(rows), idx] = 1.0
        loss_d, grad_d = _gpu_ce(df8, torch, cuda, x, t=t)
        assert abs(loss_d - loss) <= 1e-6 * max(1.0, abs(loss)) and np.abs(grad_d - grad).max() <= 1e-7
        rng = np.random.default_rng(3)
        soft = rng.dirichlet(np.ones(Cn), rows).astype(np.float32)
        want_loss, _, want_grad = oracle.cross_entropy(x, targets=soft)
        loss_s, grad_s = _gpu_ce(df8, torch, cuda, x, t=soft)
        assert abs(loss_s - want_loss) <= 1e-5 * max(1.0, abs(want_loss)) and np.abs(grad_s - want_grad).max() <= 1e-5
    assert df8.status_word() == (0, 0)


@pytest.mark.gpu
def test_cross_entropy_edge_cases(df8, oracle, cuda):
    import torch

    df8.dnn_check(df8.dnn_lib().dnn_init(0))
    x = np.array([[100.0, -100.0, 0.0, 0.0]], np.float32)
    loss, grad = _gpu_ce(df8, torch, cuda, x, idx=[0])
    assert np.isfinite(loss) and np.isfinite(grad).all() and abs(loss) <= 1e-6
    # an index outside the classes is an error, not an out-of-bounds write
    with pytest.raises(df8.Df8Error, match="outside"):
        _gpu_ce(df8, torch, cuda, np.zeros((3, 8), np.float32), idx=[1, 8, 2])
    with pytest.raises(df8.Df8Error, match="outside"):
        _gpu_ce(df8, torch, cuda, np.zeros((3, 8), np.float32), idx=[1, -1, 2])
    loss, grad = _gpu_ce(df8, torch, cuda, np.zeros((3, 8), np.float32), idx=[1, 7, 2])  # and the counter was reset
    assert abs(loss - np.log(8.0)) <= 1e-5
    # the C-ABI refuses both or neither kind of target
    xd = torch.zeros((2, 4), device=cuda)
    out = torch.zeros(2, device=cuda)
    assert df8.lib().df8_cross_entropy_f32(df8.ptr(xd), 4, None, 0, None, 2, 4, df8.ptr(out), df8.stream_ptr()) != 0


@pytest.mark.gpu
def test_oracle_matches_upstreams_cross_entropy(oracle, cuda):
    """The reference itself (its CrossEntropyLoss<float> compiled from its sources) against the restatement."""
    if not REF_LIB.exists():
        pytest.skip("oracle/_ref/libdnn_ref.so not built (needs the upstream sources at build time)")
    ref = C.CDLL(str(REF_LIB))
    if not hasattr(ref, "ref_cross_entropy"):
        pytest.skip("oracle/_ref/libdnn_ref.so predates the cross-entropy wrapper")
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    for rows, Cn in ((1, 4), (16, 257), (8, 5000)):
        x = oracle.fill_normal(rows * Cn, seed=rows * 3 + Cn, std=2.0).reshape(rows, Cn)
        idx = oracle.fill_token_ids(rows, seed=4, vocab=Cn)
        t = np.zeros((rows, Cn), np.float32)
        t[np.arange(rows), idx] = 1.0
        want_loss, _, want_grad = oracle.cross_entropy(x, targets=t)
        for kind in ("dense", "index"):
            loss = C.c_float(0)
            grad = np.zeros((rows, Cn), np.float32)
            rc = ref.ref_cross_entropy(rows, Cn, p(x), p(t) if kind == "dense" else None, p(idx) if kind == "index" else None,
                                       C.byref(loss), p(grad))
            assert rc == 0
            # same order of operations: expf / logf of the device against numpy's are the only difference
            assert abs(loss.value - want_loss) <= 2e-6 * max(1.0, abs(want_loss)), (kind, loss.value, want_loss)
            assert np.abs(grad - want_grad).max() <= 1e-6
