"""Column-sharded GPT-2 forward (BASELINE config 5's structure at a small size): with the same weights it must
reproduce the unsharded Gpt2 forward bit for bit — each rank's logits are the matching vocabulary columns of the
single-GPU logits.  The single-rank form (no communicator) runs on any box; the 2-rank form needs 2 GPUs and runs
one process per GPU with the NCCL id passed through a file."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CFG = dict(vocab=1000, max_seq_len=128, layers=2, heads=4, hidden=256, ffn=512)
B, T = 2, 128


def _compare(rank, world, id_path, act_kind, causal):
    import torch

    import deepfuse_b200 as df8
    import oracle
    from oracle import gpt2_ref

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    df8.dnn_check(df8.dnn_lib().dnn_init(rank), "dnn_init")
    df8.dnn_check(df8.dnn_lib().dnn_set_fp8_policy(0, act_kind))
    params = gpt2_ref.make_params(CFG, seed=11)
    ids = torch.from_numpy(oracle.fill_token_ids(B * T, seed=12, vocab=CFG["vocab"]).reshape(B, T)).to(dev)

    full = df8.Gpt2(**CFG, device=rank)
    full.load_params(params)
    full.set_options(gelu=True, causal=causal)
    ref = df8.device_view(torch, full.forward_logits(ids), (B * T, CFG["vocab"])).clone()

    comm = df8.Comm(rank, world, id_path)
    try:
        model = df8.Gpt2ColumnSharded(comm, **CFG, device=rank)
        model.load_full_params(params)
        model.set_options(gelu=True, causal=causal)
        for _ in range(2):  # the second pass reuses the work space and the cached weight codes
            got = df8.device_view(torch, model.forward_logits_shard(ids), (B * T, model.vocab_rows))
            want = ref[:, model.vocab_begin:model.vocab_begin + model.vocab_rows]
            torch.cuda.synchronize()
            if not torch.equal(got, want):
                return False
        model.close()
    finally:
        comm.close()
    return df8.status_word() == (0, 0)


@pytest.mark.parametrize("act_kind,causal", [(0, False), (1, True)])
def test_single_rank_equals_unsharded_model(cuda, act_kind, causal):
    assert _compare(0, 1, None, act_kind, causal)


def _worker(rank, world, tmp, results):
    import os

    results[rank] = 1 if _compare(rank, world, os.path.join(tmp, "nccl_id.bin"), 0, False) else 0


def test_two_ranks_equal_unsharded_model(tmp_path):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Array("i", [0] * world)
    procs = [ctx.Process(target=_worker, args=(r, world, str(tmp_path), results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(results) == [1] * world
