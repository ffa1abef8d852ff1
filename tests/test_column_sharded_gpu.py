"""Column-sharded fully-connected layer over NCCL on 2 GPUs (skipped on a single-GPU box): every rank must end
up with exactly the codes, scale and amax that the unsharded two-pass GEMM produces on one GPU.  One process per
GPU; the 128-byte NCCL id travels through a file."""
import ctypes as C
import os
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, tmp, results):
    import torch

    import deepfuse_b200 as df8
    import oracle

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    lib = df8.lib()
    id_path = os.path.join(tmp, "nccl_id.bin")
    buf = C.create_string_buffer(128)
    if rank == 0:
        df8.check(lib.df8_comm_unique_id(buf), "df8_comm_unique_id")
        with open(id_path + ".tmp", "wb") as f:
            f.write(buf.raw)
        os.replace(id_path + ".tmp", id_path)
    else:
        for _ in range(600):
            if os.path.exists(id_path):
                break
            time.sleep(0.05)
        buf.raw = open(id_path, "rb").read()
    comm = C.c_void_p(0)
    df8.check(lib.df8_comm_init_rank(buf, world, rank, C.byref(comm)), "df8_comm_init_rank")
    try:
        ok = True
        for M, N, K, flags, out_kind in [(256, 512, 128, 0, 0), (1000, 3072, 768, 1, 0), (512, 2304, 768, 0, 1)]:
            x = oracle.fill_normal(M * K, seed=1).reshape(M, K)
            w = oracle.fill_normal(N * K, seed=2, std=0.05).reshape(N, K)
            b = oracle.fill_normal(N, seed=3, std=0.1)
            xc, sx = oracle.quantize(x, 0)
            wc, sw = oracle.quantize(w, 0)
            t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
            xcd, wcd, sxd, swd, bd = t(xc), t(wc), t(sx), t(sw), t(b)
            # single-GPU answer, computed on this rank
            ref_codes = torch.empty((M, N), dtype=torch.uint8, device=dev)
            ref_scale, ref_amax = torch.zeros(2, device=dev), torch.zeros(1, device=dev)
            df8.gemm_fp8_tn_q(xcd, 0, sxd, wcd, 0, swd, bd, M, N, K, flags, out_kind, ref_codes, ref_scale, ref_amax)
            # sharded
            n = N // world
            w_shard = wcd[rank * n:(rank + 1) * n].contiguous()
            b_shard = bd[rank * n:(rank + 1) * n].contiguous()
            slice_s = torch.empty(M * n, dtype=torch.uint8, device=dev)
            gath_s = torch.empty(M * N, dtype=torch.uint8, device=dev)
            out = torch.full((M, N), 0xAA, dtype=torch.uint8, device=dev)
            scale, amax = torch.zeros(2, device=dev), torch.zeros(1, device=dev)
            df8.check(lib.df8_fc_fp8_column_sharded(comm, df8.ptr(xcd), 0, df8.ptr(sxd), df8.ptr(w_shard), 0,
                                                    df8.ptr(swd), df8.ptr(b_shard), M, N, K, flags, out_kind,
                                                    df8.ptr(slice_s), df8.ptr(gath_s), df8.ptr(out), df8.ptr(scale),
                                                    df8.ptr(amax), df8.stream_ptr()), "df8_fc_fp8_column_sharded")
            torch.cuda.synchronize()
            ok = ok and torch.equal(out, ref_codes) and torch.equal(scale, ref_scale) and amax.item() == ref_amax.item()
        results[rank] = 1 if ok and df8.status_word() == (0, 0) else 0
    finally:
        df8.check(lib.df8_comm_destroy(comm), "df8_comm_destroy")


def test_column_sharded_fc_matches_single_gpu(tmp_path):
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
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(results) == [1] * world


def test_interleave_gathered_layout(df8, cuda):
    import torch

    world, M, n = 4, 37, 48
    g = torch.arange(world * M * n, dtype=torch.int64, device=cuda).remainder(251).to(torch.uint8).reshape(world, M, n)
    out = torch.zeros((M, world * n), dtype=torch.uint8, device=cuda)
    df8.check(df8.lib().df8_interleave_gathered_u8(df8.ptr(g), M, n, world, df8.ptr(out), df8.stream_ptr()))
    assert torch.equal(out, g.permute(1, 0, 2).reshape(M, world * n))


def test_split_gemm_passes_equal_the_fused_call(df8, oracle, cuda):
    import torch

    M, N, K = 300, 768, 256
    xc, sx = oracle.quantize(oracle.fill_normal(M * K, seed=5).reshape(M, K), 0)
    wc, sw = oracle.quantize(oracle.fill_normal(N * K, seed=6, std=0.05).reshape(N, K), 0)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    xcd, wcd, sxd, swd = t(xc), t(wc), t(sx), t(sw)
    c1 = torch.empty((M, N), dtype=torch.uint8, device=cuda)
    s1, a1 = torch.zeros(2, device=cuda), torch.zeros(1, device=cuda)
    df8.gemm_fp8_tn_q(xcd, 0, sxd, wcd, 0, swd, None, M, N, K, 0, 0, c1, s1, a1)
    c2 = torch.empty_like(c1)
    s2, a2 = torch.zeros(2, device=cuda), torch.zeros(1, device=cuda)
    lib = df8.lib()
    df8.check(lib.df8_gemm_fp8_tn_amax(df8.ptr(xcd), 0, df8.ptr(sxd), df8.ptr(wcd), 0, df8.ptr(swd), None, M, N, K, 0,
                                       df8.ptr(a2), df8.stream_ptr()))
    df8.check(lib.df8_gemm_fp8_tn_codes(df8.ptr(xcd), 0, df8.ptr(sxd), df8.ptr(wcd), 0, df8.ptr(swd), None, M, N, K, 0,
                                        0, df8.ptr(a2), df8.ptr(c2), df8.ptr(s2), df8.stream_ptr()))
    assert a1.item() == a2.item() and torch.equal(s1, s2) and torch.equal(c1, c2)
