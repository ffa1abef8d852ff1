"""Column-sharded GPT-2 forward (the 6.7B-shape configuration's structure at a small size).

One rank (no communicator): the model is the unsharded one and must reproduce dnn::Gpt2 bit for bit.
Two ranks (needs 2 GPUs; one process per GPU, the NCCL id passed through a file): the residual stream is sharded
and the LayerNorm row sums are combined from the ranks' pieces, i.e. taken in another order than on one GPU, so an
activation on a rounding boundary may take the neighbouring fp8 code and the logits agree with the unsharded model
the way two roundings of the same 8-bit pipeline do: the maximum and RMS differences are held against the model's
own distance to the UNQUANTISED fp32 pipeline.  What must be exact: every rank computes the same hidden states, and
the exchange through peer-mapped buffers + copy engines (gathers pipelined in four row chunks: producer pushes a
chunk, the consuming GEMM runs chunk by chunk behind the tickets) gives bit for bit what the NCCL fallback (whole-tensor
gathers) gives.  Both
cases also upload a second, smaller set of weights WITHOUT asking for a re-quantisation and compare the next forward:
the per-tensor maxima of the sharded weights must be taken afresh (a maximum left from the first set would lose three
bits of every code)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CFG = dict(vocab=1000, max_seq_len=128, layers=2, heads=4, hidden=256, ffn=512)
B, T = 4, 128  # 512 token rows: four row chunks of 128 for the pipelined gathers


def _rel(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max())


def _rms(a, b):
    return float(((a.double() - b.double()) ** 2).mean().sqrt() / (b.double() ** 2).mean().sqrt())


def _compare(rank, world, id_path, act_kind, causal):
    import os

    import torch

    import deepfuse_b200 as df8
    import oracle
    from oracle import gpt2_ref

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    os.environ["DF8_SHARD_CHUNK_MIN_ROWS"] = "128"  # the peer-mapped arm gathers in four row chunks, the NCCL arm whole
    df8.dnn_check(df8.dnn_lib().dnn_init(rank), "dnn_init")
    df8.dnn_check(df8.dnn_lib().dnn_set_fp8_policy(0, act_kind))
    params = gpt2_ref.make_params(CFG, seed=11)
    ids_h = oracle.fill_token_ids(B * T, seed=12, vocab=CFG["vocab"]).reshape(B, T)
    ids = torch.from_numpy(ids_h).to(dev)

    full = df8.Gpt2(**CFG, device=rank)
    full.load_params(params)
    full.set_options(gelu=True, causal=causal)
    ref = df8.device_view(torch, full.forward_logits(ids), (B * T, CFG["vocab"])).clone()
    ref_hidden = df8.device_view(torch, full.forward_hidden(ids), (B * T, CFG["hidden"])).clone()

    results = []
    bad = []  # every check is recorded and the ranks run on: a rank that left early would strand its peer in a collective
    for transport in (("p2p", "1"), ("nccl", "0")) if world > 1 else (("single", "1"),):
        os.environ["DF8_COMM_P2P"] = transport[1]
        comm = df8.Comm(rank, world, None if id_path is None else id_path + "." + transport[0])
        try:
            model = df8.Gpt2ColumnSharded(comm, **CFG, device=rank)
            model.load_full_params(params)
            model.set_options(gelu=True, causal=causal)
            want = ref[:, model.vocab_begin:model.vocab_begin + model.vocab_rows]
            for _ in range(2):  # the second pass reuses the work space and the cached weight codes
                got = df8.device_view(torch, model.forward_logits_shard(ids), (B * T, model.vocab_rows)).clone()
                ptr, pitch = model.forward_logits_shard_pitched(ids)
                pitched = df8.device_view(torch, ptr, (B * T, pitch))[:, :model.vocab_rows].clone()
                torch.cuda.synchronize()
                if not torch.equal(got, pitched):
                    bad.append(f"{transport[0]}: dense and pitched logits differ in {(got != pitched).sum().item()} places")
                if world == 1 and not torch.equal(got, want):
                    bad.append("single rank: logits differ from the unsharded model")
            hidden = df8.device_view(torch, model.forward_hidden(ids), (B * T, CFG["hidden"])).clone()
            pushed = model.bytes_pushed()
            # a weight update that is NOT followed by an explicit re-quantisation: smaller weights, so a per-tensor
            # maximum left over from the first set would cost three bits of every code
            small = {k: (v * np.float32(0.125) if k.endswith("weight") and "embedding" not in k else v) for k, v in params.items()}
            model.load_full_params(small, prepare=False)
            full.load_params(small)
            ref_small = df8.device_view(torch, full.forward_hidden(ids), (B * T, CFG["hidden"])).clone()
            got_small = df8.device_view(torch, model.forward_hidden(ids), (B * T, CFG["hidden"])).clone()
            full.load_params(params)
            torch.cuda.synchronize()
            if world == 1:
                if not torch.equal(got_small, ref_small):
                    bad.append("re-upload: single rank differs from the unsharded model")
            else:
                f32s = torch.from_numpy(gpt2_ref.gpt2_forward(small, ids_h, CFG, act_kind=None, w_kind=None, causal=causal,
                                                              return_hidden=True)).to(dev)
                if _rel(got_small, ref_small) > 1.5 * _rel(ref_small, f32s) or _rms(got_small, ref_small) > 1.5 * _rms(ref_small, f32s):
                    bad.append(f"{transport[0]} re-upload: {_rel(got_small, ref_small)} against noise {_rel(ref_small, f32s)}")
            results.append((got, hidden, pushed, got_small))
            model.close()
        finally:
            comm.close()
    if world > 1:
        (g_p2p, h_p2p, pushed, s_p2p), (g_nccl, h_nccl, pushed_nccl, s_nccl) = results
        if not torch.equal(g_p2p, g_nccl):
            bad.append(f"logits: p2p and NCCL differ in {(g_p2p != g_nccl).sum().item()} places")
        if not torch.equal(h_p2p, h_nccl):
            bad.append(f"hidden: p2p and NCCL differ in {(h_p2p != h_nccl).sum().item()} places")
        if not torch.equal(s_p2p, s_nccl):
            bad.append(f"hidden after the re-upload: p2p and NCCL differ in {(s_p2p != s_nccl).sum().item()} places")
        if pushed <= 0 or pushed_nccl != 0:
            bad.append(f"bytes pushed: {pushed} over p2p, {pushed_nccl} over NCCL")
        # against the unsharded model, held to the distance of the 8-bit pipeline from the fp32 one
        f32 = torch.from_numpy(gpt2_ref.gpt2_forward(params, ids_h, CFG, act_kind=None, w_kind=None, causal=causal,
                                                     return_hidden=True)).to(dev)
        noise_max, noise_rms = _rel(ref_hidden, f32), _rms(ref_hidden, f32)
        if _rel(h_p2p, ref_hidden) > 1.5 * noise_max or _rms(h_p2p, ref_hidden) > 1.5 * noise_rms:
            bad.append(f"hidden {_rel(h_p2p, ref_hidden)} {noise_max} {_rms(h_p2p, ref_hidden)} {noise_rms}")
        if _rel(h_p2p, f32) > 1.25 * noise_max + 2e-3:
            bad.append(f"hidden vs fp32 {_rel(h_p2p, f32)} {noise_max}")
        if _rel(g_p2p, want) > 1e-1:
            bad.append(f"logits {_rel(g_p2p, want)}")
    if df8.status_word() != (0, 0):
        bad.append(f"device status word {df8.status_word()}")
    for b in bad:
        print(f"rank {rank}: {b}", flush=True)
    return not bad


@pytest.mark.parametrize("act_kind,causal", [(0, False), (1, True)])
def test_single_rank_equals_unsharded_model(cuda, act_kind, causal):
    assert _compare(0, 1, None, act_kind, causal)


def _worker(rank, world, tmp, results):
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    results[rank] = 1 if _compare(rank, world, os.path.join(tmp, "nccl_id.bin"), 0, False) else 0


def test_two_ranks_agree_with_unsharded_model(tmp_path):
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
        p.join(timeout=240)
    for p in procs:  # a rank that is still waiting for its peer must not outlive the test
        if p.is_alive():
            p.kill()
            p.join()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(results) == [1] * world


def _exchange_worker(rank, world, tmp, results):
    """The two exchange primitives on their own, many times over (ring slots and sequence numbers wrap)."""
    import ctypes as C
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch

    import deepfuse_b200 as df8

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    lib = df8.lib()
    comm = df8.Comm(rank, world, os.path.join(tmp, "nccl_id.bin"))
    ok = True
    try:
        n = 1 << 20
        p = C.c_void_p(0)
        df8.check(lib.df8_comm_symm_alloc(comm.h, world * n + 4096, C.byref(p)))
        enabled = C.c_int(0)
        df8.check(lib.df8_comm_p2p_enabled(comm.h, C.byref(enabled)))
        buf = df8.device_view(torch, p.value, (world * n + 4096,), dtype=torch.uint8)
        val = torch.zeros(1, device=dev)
        for it in range(200):
            size = n if it % 3 == 0 else 4096 * (1 + it % 7)
            off = 256 * (it % 5)
            mine = buf[off + rank * size: off + (rank + 1) * size]
            mine.copy_(torch.full((size,), (it * 7 + rank * 13) % 251, dtype=torch.uint8, device=dev))
            df8.check(lib.df8_comm_allgather_symm(comm.h, p.value, off, size, df8.stream_ptr()))
            got = buf[off: off + world * size].reshape(world, size)
            want = torch.tensor([(it * 7 + r * 13) % 251 for r in range(world)], dtype=torch.uint8, device=dev)
            ok = ok and bool((got == want[:, None]).all())
            val.fill_(float((it * (rank + 3)) % 17) + 0.5)
            df8.check(lib.df8_comm_allreduce_max_p2p(comm.h, df8.ptr(val), df8.stream_ptr()))
            ok = ok and val.item() == max(float((it * (r + 3)) % 17) + 0.5 for r in range(world))
        torch.cuda.synchronize()
        results[rank] = 1 if ok and enabled.value == 1 and df8.status_word() == (0, 0) else 0
    finally:
        comm.close()


def test_peer_exchange_primitives_two_ranks(tmp_path):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Array("i", [0] * world)
    procs = [ctx.Process(target=_exchange_worker, args=(r, world, str(tmp_path), results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.kill()
            p.join()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(results) == [1] * world
