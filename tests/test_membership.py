"""A rank that goes away between steps: the ranks that stay learn of it on the host, before their next launch.

CPU part: the board's protocol on its own, and world_size-2/3 runs with gloo collectives as the "step" (a rank
leaves, a rank goes silent, a rank dies with an exception).  GPU part (2 GPUs, child processes, NVLS off, plain peer
copies): the column-sharded forward as the step; rank 1 leaves after two steps with nothing in flight, rank 0 sees it
before launching the third, gives the communicator up with df8_comm_abort and carries on alone on a context that
still works.  Nothing here faults, traps or hangs a GPU."""
import os
import time

import numpy as np
import pytest

from deepfuse_b200.membership import PeerLeft, PeerTimeout, StepBoard


def test_board_protocol_single_process(tmp_path):
    a = StepBoard(str(tmp_path), 0, 2, timeout_s=0.2)
    with pytest.raises(PeerTimeout) as e:  # the peer has not shown up at all
        a.wait_for_peers(0)
    assert e.value.rank == 1 and e.value.seen == -1
    b = StepBoard(str(tmp_path), 1, 2, timeout_s=0.2)
    a.gone.clear()
    a.wait_for_peers(0)
    b.wait_for_peers(0)
    a.post(1)
    b.wait_for_peers(1)
    with pytest.raises(PeerTimeout) as e:
        a.wait_for_peers(1)
    assert (e.value.rank, e.value.seen, e.value.wanted) == (1, 0, 1)
    b.post(1)
    a.wait_for_peers(1)
    b.leave()
    assert b.read(1) == (1, False)
    with pytest.raises(PeerLeft) as e:
        a.wait_for_peers(1)  # it did finish step 1, but it is gone: do not launch
    assert (e.value.rank, e.value.step) == (1, 1)
    assert a.survivors() == [0]
    with pytest.raises(ValueError):
        StepBoard(str(tmp_path), 2, 2)


def _gloo_worker(rank, world, tmp, mode, results):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(29650 + {"leave": 0, "silent": 1, "raise": 2}[mode])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    board = StepBoard(os.path.join(tmp, "board"), rank, world, timeout_s=20.0 if mode != "silent" else 1.0)
    done = 0
    try:
        for step in range(6):
            board.wait_for_peers(step)
            x = torch.tensor([float(rank + step)])
            dist.all_reduce(x, op=dist.ReduceOp.MAX)  # the step: a collective every rank must join
            assert x.item() == float(world - 1 + step)
            done = step + 1
            if rank == world - 1 and done == 2:
                if mode == "leave":
                    board.leave(done)  # instead of the post: no peer may read "finished 2, alive" from this rank
                    results[rank] = 100 + done
                    return
                if mode == "silent":
                    time.sleep(3.0)  # still alive, but stuck on the host before it is ready for the next step
                    results[rank] = 100 + done
                    return
                if mode == "raise":
                    try:
                        raise RuntimeError("this rank's step failed on the host")
                    finally:
                        board.leave()
            board.post(done)
        results[rank] = done
    except PeerLeft as e:
        results[rank] = 1000 + 10 * e.rank + done
    except PeerTimeout as e:
        results[rank] = 2000 + 10 * e.rank + done
    except RuntimeError:
        results[rank] = 3000 + done
    finally:
        # no collective on the way out: the group may be short of a member
        pass


@pytest.mark.parametrize("mode,world", [("leave", 2), ("silent", 2), ("raise", 3)])
def test_rank_goes_away_between_steps_gloo(tmp_path, mode, world):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Array("i", [0] * world)
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, str(tmp_path), mode, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    got = list(results)
    last = world - 1
    stay = {"leave": 1000, "silent": 2000, "raise": 1000}[mode] + 10 * last + 2
    # every rank that stayed finished exactly two steps and launched no third one
    assert got[:last] == [stay] * last, got
    assert got[last] == {"leave": 102, "silent": 102, "raise": 3002}[mode], got


CFG = dict(vocab=1000, max_seq_len=128, layers=2, heads=4, hidden=256, ffn=512)


def _gpu_worker(rank, world, tmp, results):
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch

    import deepfuse_b200 as df8
    import oracle
    from oracle import gpt2_ref

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    df8.dnn_check(df8.dnn_lib().dnn_init(rank), "dnn_init")
    params = gpt2_ref.make_params(CFG, seed=11)
    ids = torch.from_numpy(oracle.fill_token_ids(2 * 128, seed=12, vocab=1000).reshape(2, 128)).to(dev)
    comm = df8.Comm(rank, world, os.path.join(tmp, "nccl_id.bin"))
    model = df8.Gpt2ColumnSharded(comm, **CFG, device=rank)
    model.load_full_params(params)
    board = StepBoard(os.path.join(tmp, "board"), rank, world, timeout_s=60.0)
    done = 0
    try:
        for step in range(5):
            board.wait_for_peers(step)
            model.forward_logits_shard(ids)
            torch.cuda.synchronize()  # nothing of this rank is in flight when it posts
            done = step + 1
            if rank == 1 and done == 2:
                model.close()
                board.leave(done)
                comm.abort()  # local: no goodbye collective that the peer would have to join
                results[rank] = 100 + done if df8.status_word() == (0, 0) else -1
                return
            board.post(done)
        results[rank] = done
    except PeerLeft as e:
        # before the third launch: close what was built on the communicator, give it up, carry on alone
        model.close()
        comm.abort()
        alone = df8.Gpt2(**CFG, device=rank)
        alone.load_params(params)
        logits = df8.device_view(torch, alone.forward_logits(ids), (2 * 128, 1000)).clone()
        torch.cuda.synchronize()
        want = gpt2_ref.gpt2_forward(params, ids.cpu().numpy(), CFG)
        err = float(np.abs(logits.cpu().numpy().reshape(want.shape) - want).max() / np.abs(want).max())
        ok = err <= 5e-2 and df8.status_word() == (0, 0) and board.survivors() == [0]
        results[rank] = 1000 + 10 * e.rank + done if ok else -2
        alone.close()


@pytest.mark.gpu
def test_rank_leaves_between_steps_two_gpus(tmp_path):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    results = ctx.Array("i", [0, 0])
    procs = [ctx.Process(target=_gpu_worker, args=(r, 2, str(tmp_path), results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(results) == [1012, 102]
