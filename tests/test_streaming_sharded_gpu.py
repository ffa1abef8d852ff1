"""Layer streaming across 2 GPUs (skipped on a single-GPU box): every rank holds the whole model and its own share of
the batch, uploads HALF of each layer's weight codes from its pinned host arena and gets the other half from its
peer by an all-gather on the copy stream (ncclAllGather, or with DF8_STREAM_P2P=1 copy-engine pushes into peer-mapped
slots behind a barrier).  Logits must equal the resident-weights forward bit for bit, on repeated forwards, and the
byte counters must show the split.  One process per GPU; the NCCL id travels through a file."""
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, tmp, results, p2p):
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ["DF8_STREAM_P2P"] = p2p
    import torch

    import deepfuse_b200 as df8
    from deepfuse_b200 import synthetic

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    d = df8.dnn_lib()
    df8.dnn_check(d.dnn_init(rank))
    df8.dnn_check(d.dnn_set_fp8_policy(0, 1))  # e5m2 activations, as the streamed configuration runs
    comm = df8.Comm(rank, world, id_path=os.path.join(tmp, "nccl_id.bin"))
    cfg = dict(vocab=300, max_seq_len=64, layers=5, heads=2, hidden=128, ffn=512)
    df8.dnn_check(d.dnn_set_host_init(0))
    model = df8.Gpt2(**cfg, device=rank)
    df8.dnn_check(d.dnn_set_host_init(1))
    model.initialize_on_device(11, 0.05)
    ids = torch.from_numpy(synthetic.fill_token_ids(3 * 64, seed=40 + rank, vocab=300).reshape(3, 64)).to(dev)
    want = df8.device_view(torch, model.forward_logits(ids), (3 * 64, 300)).clone()
    model.enable_streaming(slots=2, release_fp32=True, comm=comm)
    ok = True
    for _ in range(3):
        got = df8.device_view(torch, model.forward_logits(ids), (3 * 64, 300)).clone()
        ok = ok and torch.equal(got, want)
    torch.cuda.synchronize()
    h2d, gathered = model.streaming_traffic()
    ok = ok and h2d > 0 and h2d == gathered and h2d + gathered == model.streamed_bytes()
    ms = model.time_uploads()
    ok = ok and ms > 0
    got = df8.device_view(torch, model.forward_logits(ids), (3 * 64, 300)).clone()
    ok = ok and torch.equal(got, want)
    model.resize_streaming_slots(5)
    got = df8.device_view(torch, model.forward_logits(ids), (3 * 64, 300)).clone()
    ok = ok and torch.equal(got, want)
    torch.cuda.synchronize()
    results[rank] = 1 if ok and df8.status_word() == (0, 0) else 0
    model.close()
    comm.close()


@pytest.mark.parametrize("p2p", ["0", "1"])
def test_streaming_with_sharded_uploads_is_bit_identical(tmp_path, p2p):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Array("i", [0] * world)
    procs = [ctx.Process(target=_worker, args=(r, world, str(tmp_path), results, p2p)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:  # a rank that is still there would keep the box busy: end it (its exit code then fails the test)
        if p.is_alive():
            p.kill()
            p.join()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(results) == [1] * world
