"""Host-side logic of the multi-GPU path, on CPU: shard arithmetic, and a world_size-2 gloo run of the
collective helpers bench.py uses (max over ranks, shard exchange)."""
import os
import socket

import numpy as np
import pytest

from deepfuse_b200 import sharding


@pytest.mark.parametrize("total,world", [(32, 1), (32, 2), (32, 4), (32, 8), (8, 8), (7, 4), (0, 3), (5, 8)])
def test_shard_range_partitions_exactly(total, world):
    covered = []
    for r in range(world):
        s, c = sharding.shard_range(total, world, r)
        covered.extend(range(s, s + c))
    assert covered == list(range(total))
    counts = [sharding.shard_range(total, world, r)[1] for r in range(world)]
    assert max(counts) - min(counts) <= 1


def test_column_shard_keeps_chunks_whole():
    for out, world in [(12288, 8), (16384, 4), (4096, 2), (3072, 8), (96, 2)]:
        cols = []
        for r in range(world):
            s, c = sharding.column_shard(out, world, r)
            assert s % 32 == 0 and c % 32 == 0
            cols.extend(range(s, s + c))
        assert cols == list(range(out))
    with pytest.raises(ValueError):
        sharding.column_shard(50257, 2, 0)
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        start, count = sharding.shard_range(32, world, rank)
        shards = sharding.gather_shards(start, count)
        slowest = sharding.max_over_ranks(10.0 + rank)
        # a column-sharded FC on CPU: every rank computes its slice, all-gather reassembles Y = X W^T
        import torch

        g = torch.Generator().manual_seed(0)
        x = torch.randn(4, 16, generator=g)
        w = torch.randn(64, 16, generator=g)
        cs, cc = sharding.column_shard(64, world, rank)
        part = x @ w[cs:cs + cc].T
        parts = [torch.zeros(4, sharding.column_shard(64, world, r)[1]) for r in range(world)]
        dist.all_gather(parts, part)
        full = torch.cat(parts, dim=1)
        ok = torch.allclose(full, x @ w.T, atol=1e-6)
        np.save(os.path.join(out_dir, f"rank{rank}.npy"),
                np.array([slowest, float(ok)] + [v for s in shards for v in s], dtype=np.float64))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_run(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        got = np.load(tmp_path / f"rank{r}.npy")
        assert got[0] == 11.0            # max over ranks of 10 + rank
        assert got[1] == 1.0             # column-sharded FC reassembled by all-gather
        assert got[2:].tolist() == [0, 16, 16, 16]


def test_vocab_shard_covers_the_vocabulary():
    from deepfuse_b200.sharding import vocab_shard

    for vocab, world in [(50257, 8), (50257, 2), (1000, 4), (7, 8), (16, 1)]:
        rows = []
        for r in range(world):
            b, n = vocab_shard(vocab, world, r)
            assert b == min(r * -(-vocab // world), vocab) and n >= 0
            rows.extend(range(b, b + n))
        assert rows == list(range(vocab))


def test_shard_gpt2_params_reassembles_to_the_full_tensors():
    import numpy as np

    from deepfuse_b200.sharding import shard_gpt2_params, vocab_shard

    cfg = dict(vocab=37, hidden=16, ffn=32, heads=4)
    E, F, V = cfg["hidden"], cfg["ffn"], cfg["vocab"]
    rng = np.random.default_rng(0)
    full = {"embedding.weight": rng.normal(size=(V, E)), "embedding.bias": rng.normal(size=(1, E, 1, 1)),
            "block0.ln1.gamma": rng.normal(size=(E,)), "block0.ln1.beta": rng.normal(size=(E,)),
            "block0.qkv.weight": rng.normal(size=(3 * E, E)), "block0.qkv.bias": rng.normal(size=(1, 3 * E, 1, 1)),
            "block0.out.weight": rng.normal(size=(E, E)), "block0.out.bias": rng.normal(size=(1, E, 1, 1)),
            "block0.fc1.weight": rng.normal(size=(F, E)), "block0.fc1.bias": rng.normal(size=(1, F, 1, 1)),
            "block0.fc2.weight": rng.normal(size=(E, F)), "block0.fc2.bias": rng.normal(size=(1, E, 1, 1)),
            "final_fc.weight": rng.normal(size=(V, E)), "final_fc.bias": rng.normal(size=(1, V, 1, 1))}
    for world in (1, 2, 4):
        shards = [shard_gpt2_params(full, cfg, world, r) for r in range(world)]
        eg = E // world
        # QKV: rank r holds [Q_r; K_r; V_r]
        qkv = np.empty((3 * E, E))
        qb = np.empty(3 * E)
        for r, s in enumerate(shards):
            for part in range(3):
                qkv[part * E + r * eg:part * E + (r + 1) * eg] = s["block0.qkv.weight"][part * eg:(part + 1) * eg]
                qb[part * E + r * eg:part * E + (r + 1) * eg] = s["block0.qkv.bias"].reshape(-1)[part * eg:(part + 1) * eg]
        assert np.array_equal(qkv, full["block0.qkv.weight"]) and np.array_equal(qb, full["block0.qkv.bias"].reshape(-1))
        for name in ("block0.out", "block0.fc1", "block0.fc2", "final_fc"):
            w = np.concatenate([s[name + ".weight"] for s in shards])
            b = np.concatenate([s[name + ".bias"].reshape(-1) for s in shards])
            assert np.array_equal(w, full[name + ".weight"]) and np.array_equal(b, full[name + ".bias"].reshape(-1))
        for r, s in enumerate(shards):
            assert s["final_fc.weight"].shape[0] == vocab_shard(V, world, r)[1]
            assert np.array_equal(s["embedding.weight"], full["embedding.weight"])
            assert np.array_equal(s["block0.ln1.gamma"], full["block0.ln1.gamma"])
    import pytest

    with pytest.raises(ValueError):
        shard_gpt2_params(full, cfg, 3, 0)
