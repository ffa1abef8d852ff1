"""Host-side partitioning of the GPT-2 forward across the GPUs of one box (one process per GPU).

Two partitions exist on this path:

* batch sharding — sequences are independent through the whole forward (attention is per sequence), so
  rank r takes a contiguous range of the batch and no activation ever crosses GPUs.  The upstream project's
  only multi-GPU scheme is of this kind: independent replicas per device under a tbb::parallel_for
  (apps/host-multi/main.cpp:157-181);
* column sharding of a fully-connected layer — W [out, in] split on `out` into world_size row blocks; every
  rank holds the full input, computes its [M, out/world] slice, and one all-gather completes the layer.

Timing of a multi-GPU step is the maximum over ranks of the per-rank device time.
"""
from __future__ import annotations


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """(start, count) of rank's contiguous share of `total` items; shares differ by at most one item."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad shard request total={total} world={world} rank={rank}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def column_shard(out_features: int, world: int, rank: int, multiple: int = 32) -> tuple[int, int]:
    """(start, count) of the output columns rank computes; every shard but the last is a multiple of
    `multiple` columns (the fp8-output GEMM epilogue works on 32-column chunks)."""
    if out_features % multiple != 0:
        raise ValueError(f"out_features={out_features} is not a multiple of {multiple}")
    start, count = shard_range(out_features // multiple, world, rank)
    return start * multiple, count * multiple


def max_over_ranks(value: float, group=None) -> float:
    """All-reduce(MAX) of a host float over the process group (identity without one)."""
    import torch
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized():
        return float(value)
    device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def gather_shards(start: int, count: int, group=None) -> list[tuple[int, int]]:
    """Every rank's (start, count), in rank order."""
    import torch
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized():
        return [(start, count)]
    device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    mine = torch.tensor([start, count], dtype=torch.int64, device=device)
    out = [torch.zeros_like(mine) for _ in range(dist.get_world_size(group))]
    dist.all_gather(out, mine, group=group)
    return [(int(t[0]), int(t[1])) for t in out]


def vocab_shard(vocab: int, world: int, rank: int) -> tuple[int, int]:
    """(first row, rows) of the vocabulary head rank owns in the column-sharded model: ceil(vocab / world) rows
    per rank, the last rank takes what is left."""
    if world <= 0 or not 0 <= rank < world or vocab <= 0:
        raise ValueError(f"bad vocabulary shard request vocab={vocab} world={world} rank={rank}")
    per = (vocab + world - 1) // world
    begin = min(rank * per, vocab)
    return begin, min(per, vocab - begin)


def shard_gpt2_params(params: dict, cfg: dict, world: int, rank: int) -> dict:
    """This rank's shards of a full GPT-2 parameter dictionary (names as dnn_gpt2_param_info gives them), in the
    layout the column-sharded model expects:

    * blockN.qkv: rows {Q, K, V} x (this rank's heads) of the fused [3E, E] weight, i.e. the three row ranges
      [r*E/g, (r+1)*E/g) + {0, E, 2E}, concatenated — so that the rank's [M, 3E/g] output is the QKV buffer of its
      own heads;
    * blockN.out / fc1 / fc2: contiguous row blocks (output columns) of [E,E], [F,E], [E,F];
    * final_fc: rows vocab_shard(...) of the head;
    * embedding and LayerNorm parameters: replicated.
    """
    import numpy as np

    E, F, H, V = cfg["hidden"], cfg["ffn"], cfg["heads"], cfg["vocab"]
    if H % world or E % world or F % world:
        raise ValueError(f"heads={H}, hidden={E}, ffn={F} must be divisible by world={world}")
    eg, fg = E // world, F // world
    out = {}
    for name, a in params.items():
        a = np.asarray(a)
        kind = name.split(".")[-2] if "." in name else name
        is_w = name.endswith(".weight")
        flat = a.reshape(a.shape[0], -1) if is_w else a.reshape(-1)
        if kind == "qkv":
            idx = np.concatenate([np.arange(rank * eg, (rank + 1) * eg) + base for base in (0, E, 2 * E)])
            out[name] = np.ascontiguousarray(flat[idx])
        elif kind in ("out", "fc2"):
            out[name] = np.ascontiguousarray(flat[rank * eg:(rank + 1) * eg])
        elif kind == "fc1":
            out[name] = np.ascontiguousarray(flat[rank * fg:(rank + 1) * fg])
        elif kind == "final_fc":
            b, n = vocab_shard(V, world, rank)
            out[name] = np.ascontiguousarray(flat[b:b + n])
        else:
            out[name] = a
    return out
