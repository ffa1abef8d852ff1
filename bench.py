#!/usr/bin/env python
"""Benchmark of the fp8 fully-connected + attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line (rank 0).  A "step" is one pass of the hot path over one batch of seeded
synthetic input.  Workloads:

  gpt2s   (default) GPT-2 small fp8 forward, 12 layers, d_model 768, batch 8x1024 token ids per GPU -> fp32
          logits through dnn::Gpt2; tokens/s.  gpt2m: GPT-2 medium, e5m2 activations, batch 32 sharded
  gemm    the fp8 projections of one GPT-2 small layer + the vocabulary head at 8192 tokens; TFLOP/s
  quant   per-tensor amax + fp32->e4m3 quantise + dequantise round trip of one 2^30-element tensor
          (values ~N(0,1) with 0.1 % of positions replaced by 100*N(0,1) outliers), GB/s of
          algorithmic traffic (14 bytes per element)

`value` is measured with inputs resident in HBM; `e2e` is the same work through the C-ABI with
pinned HOST buffers, host<->device copies inside the timed region.  `--impl reference` times the
CPU oracle (a port of the upstream project's host-side math; upstream has no CPU implementation
of its own) on the host cores, on a bounded sample of the same workload.

Under torchrun (N > 1) every rank runs the same per-GPU work (weak scaling, no data-path
collective); timing is CUDA events, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def _peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()
        # nvidia-smi stalls kernel launches while it attaches to the driver: let it produce its first
        # sample before the timed region begins
        t0 = time.time()
        while not self.lines and time.time() - t0 < 5.0:
            time.sleep(0.02)

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------

class QuantWorkload:
    """amax + quantise(e4m3) + dequantise of one fp32 tensor, all through the C-ABI."""

    name = "quant"
    metric = "fp8 quantise+dequantise round-trip GB/s"
    unit = "GB/s"
    dtype = "f32->e4m3->f32"
    bytes_per_elem = 14  # 4 (amax read) + 4 (re-read) + 1 (codes) + 1 (codes read) + 4 (fp32 write)
    kernels_per_step = 3
    memsets_per_step = 1

    def __init__(self, log2n: int = 30, seed: int = 1):
        self.n = 1 << log2n
        self.log2n = log2n
        self.seed = seed

    def config(self, n_gpus):
        return {"workload": f"quantise/dequantise round trip, 2^{self.log2n} fp32 elements per GPU, e4m3, "
                            "N(0,1) + 0.1% outliers x100, seed 1",
                "elements_per_gpu": self.n, "l2_policy": "inputs (4 GiB) larger than L2",
                "parallelism": f"independent tensor per GPU x{n_gpus}"}

    def units_per_step(self):  # GB of algorithmic traffic per GPU per step
        return self.n * self.bytes_per_elem / 1e9

    def setup(self, torch, df8, dev, rank):
        self.torch, self.df8 = torch, df8
        g = torch.Generator(device=dev)
        g.manual_seed(self.seed + rank)
        self.x = torch.randn(self.n, device=dev, generator=g)
        k = self.n // 1000
        idx = torch.randint(0, self.n, (k,), device=dev, generator=g)
        self.x[idx] = 100.0 * torch.randn(k, device=dev, generator=g)
        self.amax = torch.zeros(1, device=dev)
        self.scale = torch.zeros(2, device=dev)
        self.codes = torch.empty(self.n, dtype=torch.uint8, device=dev)
        self.y = torch.empty(self.n, device=dev)

    def step(self):
        d = self.df8
        d.amax_f32(self.x, self.amax)
        d.quantize_f32(self.x, d.E4M3, self.amax, self.codes, self.scale)
        d.dequantize_f32(self.codes, d.E4M3, self.scale, self.y)

    # dominant kernel, timed on its own for the roofline entry
    def roofline(self, torch, peaks, iters=10):
        d = self.df8
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        d.amax_f32(self.x, self.amax)
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(iters):
            d.quantize_f32(self.x, d.E4M3, self.amax, self.codes, self.scale)
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1]) / iters
        achieved = self.n * 5 / 1e9 / (ms / 1e3)
        return {"kernel": "quantize_f32_kernel<e4m3>", "bound": "hbm", "achieved": round(achieved, 1),
                "peak": peaks["hbm_gbs"], "peak_source": peaks["source"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "ms_per_launch": round(ms, 4),
                "algorithmic_bytes_per_launch": self.n * 5,
                # ncu dram read+write bytes of one 2^27-element launch (619.17 MB,
                # profiles/quantize_f32_kernel_quant_2p27.md), scaled by the element count
                "traffic": round(619.17e6 * self.n / (1 << 27))}

    def e2e_setup(self, torch, dev):
        # a 2^28-element slice of the workload keeps the pinned allocations modest (1 GiB in)
        self.e2e_n = min(self.n, 1 << 28)
        self.hx = torch.empty(self.e2e_n, dtype=torch.float32, pin_memory=True)
        self.hx.copy_(self.x[: self.e2e_n])
        self.hy = torch.empty(self.e2e_n, dtype=torch.float32, pin_memory=True)
        self.hcodes = torch.empty(self.e2e_n, dtype=torch.uint8, pin_memory=True)

    def e2e_step(self):
        d, n = self.df8, self.e2e_n
        x, codes, y = self.x[:n], self.codes[:n], self.y[:n]
        x.copy_(self.hx, non_blocking=True)
        d.amax_f32(x, self.amax)
        d.quantize_f32(x, d.E4M3, self.amax, codes, self.scale)
        d.dequantize_f32(codes, d.E4M3, self.scale, y)
        self.hcodes.copy_(codes, non_blocking=True)
        self.hy.copy_(y, non_blocking=True)

    def e2e_units_per_step(self):
        return self.e2e_n * self.bytes_per_elem / 1e9

    def e2e_bytes(self):
        return self.e2e_n * 4, self.e2e_n * 5

    # CPU oracle on a bounded sample
    def cpu_sample(self, orc, log2n=25):
        n = 1 << log2n
        x = orc.fill_normal_outliers(n, seed=self.seed)
        t0 = time.perf_counter()
        a = orc.amax(x)
        codes, s = orc.quantize(x, orc.E4M3, amax_v=a)
        orc.dequantize(codes, orc.E4M3, s[1])
        dt = time.perf_counter() - t0
        return n * self.bytes_per_elem / 1e9, dt, f"2^{log2n} elements of the same distribution"



class GemmWorkload:
    """The fp8 projections of one GPT-2 layer at M tokens (QKV, out, FC1+GELU, FC2+residual) plus the
    vocabulary head, each one df8_gemm_fp8_tn call on pre-quantised e4m3 operands."""

    name = "gemm"
    metric = "fp8 GEMM TFLOP/s"
    unit = "TFLOP/s"
    dtype = "e4m3 x e4m3 -> f32"

    def __init__(self, M=8192, E=768, F=3072, V=50257, only=None):
        self.M, self.E, self.F, self.V = M, E, F, V
        shapes = [("qkv", 3 * E, E, 4), ("out", E, E, 2), ("fc1", F, E, 1 | 4), ("fc2", E, F, 2), ("head", V, E, 0)]
        # large square problem (tensor-pipe bound; not part of the default set): --only big
        # and the two projections whose output the next layer consumes as fp8 codes, through the two-pass
        # df8_gemm_fp8_tn_q (flag 8 here; counted as one product although the tensor work runs twice)
        extra = [("big", 8192, 8192, 0), ("big4k", 8192, 4096, 0), ("qkvq", 3 * E, E, 8), ("fc1q", F, E, 1 | 8)]
        self.shapes = [s for s in shapes if only is None or s[0] in only] + [s for s in extra if only and s[0] in only]
        self.kernels_per_step = sum(2 if f & 8 else 1 for _, _, _, f in self.shapes)

    def config(self, n_gpus):
        return {"workload": f"GPT-2 small projection set at M={self.M} tokens: "
                            + ", ".join(f"{n}[{self.M}x{N}x{K}]" for n, N, K, _ in self.shapes),
                "l2_policy": "L2 flushed by a 256 MiB write between steps", "parallelism": f"replicated x{n_gpus}"}

    def flops(self):
        return sum(2.0 * self.M * N * K for _, N, K, _ in self.shapes)

    def units_per_step(self):
        return self.flops() / 1e12

    def setup(self, torch, df8, dev, rank):
        self.torch, self.df8 = torch, df8
        g = torch.Generator(device=dev)
        g.manual_seed(5 + rank)
        self.ops = []
        one = torch.tensor([1.0, 1.0 / 64], device=dev)
        for name, N, K, flags in self.shapes:
            a = torch.randint(0, 0x78, (self.M, K), dtype=torch.uint8, device=dev, generator=g)
            w = torch.randint(0, 0x60, (N, K), dtype=torch.uint8, device=dev, generator=g)
            sign = torch.randint(0, 2, (N, K), dtype=torch.uint8, device=dev, generator=g) * 0x80
            w = w | sign
            bias = torch.zeros(N, device=dev)
            res = torch.randn(self.M, N, device=dev, generator=g) if flags & 2 else None
            out = (torch.empty(self.M, N, dtype=torch.uint8, device=dev) if flags & 8
                   else torch.empty(self.M, N, device=dev))
            amax = torch.zeros(1, device=dev)
            self.ops.append((a, w, bias, res, out, amax, N, K, flags))
        self.one = one
        self.out_scale = torch.zeros(2, device=dev)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def _call(self, op):
        d = self.df8
        a, w, bias, res, out, amax, N, K, flags = op
        if flags & 8:
            d.gemm_fp8_tn_q(a, d.E4M3, self.one, w, d.E4M3, self.one, bias, self.M, N, K, flags & 1, d.E4M3, out,
                            self.out_scale, amax)
        else:
            d.gemm_fp8_tn(a, d.E4M3, self.one, w, d.E4M3, self.one, bias, res, self.M, N, K, flags, out, amax)

    def step(self):
        self.flush.zero_()
        for op in self.ops:
            self._call(op)

    def roofline(self, torch, peaks, iters=20):
        d = self.df8
        per = {}
        best = None
        for (name, _, _, _), op in zip(self.shapes, self.ops):
            N, K = op[6], op[7]
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            for _ in range(3):
                self._call(op)
            torch.cuda.synchronize()
            ev[0].record()
            for _ in range(iters):
                self._call(op)
            ev[1].record()
            torch.cuda.synchronize()
            ms = ev[0].elapsed_time(ev[1]) / iters
            tf = 2.0 * self.M * N * K / 1e12 / (ms / 1e3)
            per[name] = {"ms": round(ms, 4), "tflops": round(tf, 1)}
            if best is None or 2.0 * self.M * N * K > best[0]:
                best = (2.0 * self.M * N * K, name, ms, tf)
        peak = 2.0 * peaks["bf16_tflops"]
        return {"kernel": f"gemm_fp8_tn_kernel ({best[1]})", "bound": "tensor", "achieved": round(best[3], 1),
                "peak": peak, "peak_source": peaks["source"] + " bf16 burst x2 (fp8 dense)", "unit": "TFLOP/s",
                "frac": round(best[3] / peak, 4), "ms_per_launch": round(best[2], 4),
                "algorithmic_flops_per_launch": best[0], "traffic": None, "per_shape": per}

    def e2e_setup(self, torch, dev):
        a = self.ops[0][0]
        self.h_a = torch.empty(a.shape, dtype=torch.uint8, pin_memory=True)
        self.h_a.copy_(a)
        self.h_out = torch.empty(self.M, dtype=torch.float32, pin_memory=True)

    def e2e_step(self):
        self.ops[0][0].copy_(self.h_a, non_blocking=True)
        self.step()
        self.h_out.copy_(self.ops[-1][4][:, 0], non_blocking=True)

    def e2e_units_per_step(self):
        return self.units_per_step()

    def e2e_bytes(self):
        return self.h_a.numel(), self.h_out.numel() * 4

    def cpu_sample(self, orc, rows=16):
        import numpy as np

        units, secs = 0.0, 0.0
        rng = np.random.default_rng(0)
        for name, N, K, flags in self.shapes:
            Nc = min(N, 4096)
            xc = rng.integers(0, 0x78, (rows, K), dtype=np.uint8)
            wc = rng.integers(0, 0x60, (Nc, K), dtype=np.uint8)
            t0 = time.perf_counter()
            orc.fc_forward_fp8(xc, orc.E4M3, 1.0, wc, orc.E4M3, 1.0)
            secs += time.perf_counter() - t0
            units += 2.0 * rows * Nc * K / 1e12
        return units, secs, f"{rows} token rows (and at most 4096 output columns) of each projection"


GPT2_CONFIGS = {
    # name: (layers, hidden, heads, ffn, vocab, context, batch per GPU, activation kind)
    "gpt2s": dict(layers=12, hidden=768, heads=12, ffn=3072, vocab=50257, ctx=1024, batch=8, act="e4m3"),
    "gpt2m": dict(layers=24, hidden=1024, heads=16, ffn=4096, vocab=50257, ctx=1024, batch=32, act="e5m2"),
}


def gpt2_flops_per_token(c, T):
    E, F, V, L = c["hidden"], c["ffn"], c["vocab"], c["layers"]
    return L * (2 * (3 * E * E + E * E + 2 * E * F) + 4 * T * E) + 2 * E * V


class Gpt2Workload:
    """GPT-2 fp8 forward (token ids -> fp32 logits) through dnn::Gpt2<float>::forward_logits."""

    unit = "tokens/s"

    def __init__(self, name="gpt2s", n_gpus=1, batch=None, layers=None):
        self.name = name
        self.c = dict(GPT2_CONFIGS[name])
        if layers:
            self.c["layers"] = layers
        self.n_gpus = n_gpus
        # gpt2s: weak scaling, 8 sequences per GPU; gpt2m: the fixed batch of 32 sharded across the GPUs
        self.strong = name == "gpt2m"
        self.B = batch or (max(1, self.c["batch"] // n_gpus) if self.strong else self.c["batch"])
        self.T = self.c["ctx"]
        self.metric = "GPT-2 fp8 forward tokens/s"
        self.dtype = f"{self.c['act']} activations x e4m3 weights -> f32 accumulate"
        # embedding; per layer: LN+quantise (one cooperative kernel when the activation fits the GPU's shared
        # memory, else two), QKV GEMM (max + codes), attention, quantise, out GEMM, LN+quantise, FC1 GEMM (max + codes),
        # FC2 GEMM; head: amax, quantise, GEMM
        rows, C = self.B * self.T, self.c["hidden"]
        ln = 1 if (C <= 1024 and rows >= 1024 and rows * C * 4 <= 148 * 200 * 1024) else 2
        # with DF8_GEMM_FUSED_Q=1 the two GEMM passes of QKV and FC1 are one cooperative launch where the single-CTA
        # kernel runs (K < 1024) with at least one 128 x 256 tile per SM
        one_launch = (C < 1024 and -(-rows // 128) * -(-3 * C // 256) >= 148
                      and os.environ.get("DF8_GEMM_FUSED_Q", "0")[:1] == "1")
        gq = 1 if one_launch else 2
        self.kernels_per_step = 1 + (4 + 2 * gq + 2 * ln) * self.c["layers"] + 3

    def config(self, n_gpus):
        c = self.c
        return {"workload": f"GPT-2 {'small' if self.name == 'gpt2s' else 'medium'} fp8 forward: {c['layers']} layers, "
                            f"d_model {c['hidden']}, {c['heads']} heads, FFN {c['ffn']}, vocab {c['vocab']}, "
                            f"batch {self.B}x{self.T} token ids per GPU, fp32 logits, random-init N(0,0.02) weights",
                "global_batch": self.B * n_gpus, "seq_len": self.T,
                "weights": ("e4m3 codes of the block weights in pinned host memory, streamed per layer through 2 "
                            "device slots on a side stream") if self.name == "gpt2m" else "resident e4m3 codes",
                "l2_policy": "working set per forward (1.65 GB of logits alone) larger than L2",
                "parallelism": f"batch-sharded x{n_gpus}, weights replicated, no data-path collective"}

    def units_per_step(self):
        return self.B * self.T

    def setup(self, torch, df8, dev, rank):
        import oracle as orc
        from oracle import gpt2_ref

        self.torch, self.df8 = torch, df8
        c = self.c
        cfg = dict(vocab=c["vocab"], max_seq_len=c["ctx"], layers=c["layers"], heads=c["heads"], hidden=c["hidden"],
                   ffn=c["ffn"])
        df8.dnn_check(df8.dnn_lib().dnn_init(dev.index), "dnn_init")
        df8.dnn_check(df8.dnn_lib().dnn_set_fp8_policy(0, 0 if c["act"] == "e4m3" else 1))
        self.model = df8.Gpt2(**cfg, device=dev.index)
        self.model.set_stream(torch.cuda.current_stream())
        self.model.load_params(gpt2_ref.make_params(cfg, seed=2 if self.name == "gpt2s" else 3))
        self.model.set_options(gelu=True, causal=False)
        if self.name == "gpt2m":  # e4m3 weights held in pinned host memory, streamed per layer
            self.model.enable_streaming(slots=2, release_fp32=True)
        ids = orc.fill_token_ids(self.B * self.T, seed=100 + rank, vocab=c["vocab"]).reshape(self.B, self.T)
        self.ids = torch.from_numpy(ids).to(dev)
        self.ids_host = torch.from_numpy(ids).pin_memory()
        self.last_logits = torch.empty((self.B, c["vocab"]), dtype=torch.float32, pin_memory=True)
        self.dev = dev

    def step(self):
        self.logits_ptr = self.model.forward_logits(self.ids, check_ids=False)

    def e2e_setup(self, torch, dev):
        pass

    def e2e_step(self):
        torch, c = self.torch, self.c
        ptr = self.model.forward_logits_host(self.ids_host)
        logits = self.df8.device_view(torch, ptr, (self.B, self.T, c["vocab"]))
        self.last_logits.copy_(logits[:, -1, :], non_blocking=True)  # the next-token logits of every sequence

    def e2e_units_per_step(self):
        return self.units_per_step()

    def e2e_bytes(self):
        return self.ids_host.numel() * 4, self.last_logits.numel() * 4

    def roofline(self, torch, peaks, iters=10):
        # dominant kernel: the vocabulary-head GEMM [B*T, V] x [V, E]
        d, c = self.df8, self.c
        M, N, K = self.B * self.T, c["vocab"], c["hidden"]
        g = torch.Generator(device=self.dev)
        g.manual_seed(1)
        a = torch.randint(0, 0x70, (M, K), dtype=torch.uint8, device=self.dev, generator=g)
        w = torch.randint(0, 0x70, (N, K), dtype=torch.uint8, device=self.dev, generator=g)
        one = torch.tensor([1.0, 1.0 / 64], device=self.dev)
        out = torch.empty((M, N), device=self.dev)
        for _ in range(2):
            d.gemm_fp8_tn(a, 0, one, w, 0, one, None, None, M, N, K, 0, out)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(iters):
            d.gemm_fp8_tn(a, 0, one, w, 0, one, None, None, M, N, K, 0, out)
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1]) / iters
        flops = 2.0 * M * N * K
        tf = flops / 1e12 / (ms / 1e3)
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        return {"kernel": "gemm_fp8_tn_kernel (vocabulary head)", "bound": "tensor", "achieved": round(tf, 1),
                "peak": peak, "peak_source": peaks["source"] + " bf16 sustained x2 (fp8 dense)", "unit": "TFLOP/s",
                "frac": round(tf / peak, 4), "ms_per_launch": round(ms, 4), "algorithmic_flops_per_launch": flops,
                # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this launch at batch 8 x 1024
                # (profiles/gemm_fp8_tn_kernel_head_8192x50257x768.md: 68.0 MB + 1.605 GB), scaled by the rows
                "traffic": round((68.0e6 + 1.605e9) * M / 8192) if c["hidden"] == 768 else None,
                "model_flops_per_token": gpt2_flops_per_token(c, self.T)}

    def cpu_sample(self, orc, tokens=128):
        from oracle import gpt2_ref

        c = self.c
        E = c["hidden"]
        cfg = dict(vocab=c["vocab"], max_seq_len=c["ctx"], layers=1, heads=c["heads"], hidden=E, ffn=c["ffn"])
        prm = gpt2_ref.make_params(cfg, seed=2)
        x = orc.fill_normal(tokens * E, seed=7).reshape(tokens, E)
        act = orc.E4M3 if c["act"] == "e4m3" else orc.E5M2
        t0 = time.perf_counter()
        y = gpt2_ref.block_forward(prm, "block0", x, 1, tokens, c["heads"], act, orc.E4M3, True)
        t_block = time.perf_counter() - t0
        t0 = time.perf_counter()
        gpt2_ref._fc(y, prm["final_fc.weight"], prm["final_fc.bias"], act, orc.E4M3)
        t_head = time.perf_counter() - t0
        # one block at `tokens` context -> L blocks at the full context, scaled by the per-token block flops
        blk = lambda T: 2 * (3 * E * E + E * E + 2 * E * c["ffn"]) + 4 * T * E
        secs = t_block * c["layers"] * blk(self.T) / blk(tokens) + t_head
        return tokens, secs, (f"one transformer block + the vocabulary head on 1x{tokens} tokens, extrapolated "
                              f"linearly in flops to {c['layers']} blocks at context {self.T}")


class AttnWorkload:
    """df8_attention_fp8 on a GPT-2 small sized QKV code buffer (B=8, T=1024, H=12, D=64), non-causal."""

    name = "attn"
    metric = "fp8 attention TFLOP/s"
    unit = "TFLOP/s"
    dtype = "e4m3 QKV -> f32"
    kernels_per_step = 1

    def __init__(self, B=8, T=1024, H=12, D=64):
        self.B, self.T, self.H, self.D = B, T, H, D

    def config(self, n_gpus):
        return {"workload": f"attention B={self.B} T={self.T} H={self.H} D={self.D}, e4m3 codes, no mask",
                "l2_policy": "L2 flushed by a 256 MiB write between steps", "parallelism": f"replicated x{n_gpus}"}

    def units_per_step(self):
        return 4.0 * self.B * self.H * self.T * self.T * self.D / 1e12

    def setup(self, torch, df8, dev, rank):
        self.torch, self.df8 = torch, df8
        g = torch.Generator(device=dev)
        g.manual_seed(3)
        E = self.H * self.D
        x = torch.randn(self.B * self.T, 3 * E, device=dev, generator=g)
        self.codes = torch.empty(x.shape, dtype=torch.uint8, device=dev)
        self.scale, amax = torch.zeros(2, device=dev), torch.zeros(1, device=dev)
        df8.amax_f32(x, amax)
        df8.quantize_f32(x, 0, amax, self.codes, self.scale)
        self.out = torch.empty(self.B * self.T, E, device=dev)
        self.amax = torch.zeros(1, device=dev)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step(self):
        self.flush.zero_()
        self.df8.attention_fp8(self.codes, 0, self.scale, self.B, self.T, self.H, self.D, 0, None, self.out, self.amax)

    def roofline(self, torch, peaks, iters=20):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(iters):
            self.df8.attention_fp8(self.codes, 0, self.scale, self.B, self.T, self.H, self.D, 0, None, self.out, self.amax)
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1]) / iters
        tf = self.units_per_step() / (ms / 1e3)
        peak = 2.0 * peaks["bf16_tflops"]
        wide = self.D == 64 and self.T % 256 == 0 and os.environ.get("DF8_ATTN_WIDE", "1")[:1] != "0"
        # one ncu capture of this launch each: the two-tile kernel read 19.0 MB and wrote nothing back inside the
        # capture (profiles/attention_fp8_wide_kernel_b8_t1024_h12_d64.md: the 25.2 MB of output stay in L2); the
        # one-tile kernel 19.2 MB read + 67.3 MB written (output plus write-back of the bench's L2 flush buffer)
        traffic = None
        if (self.B, self.T, self.H, self.D) == (8, 1024, 12, 64):
            traffic = round(19.0e6 + 9.7e3) if wide else round(19.15e6 + 67.33e6)
        return {"kernel": "attention_fp8_wide_kernel" if wide else f"attention_fp8_kernel<{self.D}>",
                "bound": "tensor", "achieved": round(tf, 1), "peak": peak,
                "peak_source": peaks["source"] + " bf16 burst x2 (fp8 dense)", "unit": "TFLOP/s",
                "frac": round(tf / peak, 4), "ms_per_launch": round(ms, 4),
                "algorithmic_flops_per_launch": self.units_per_step() * 1e12, "traffic": traffic}

    def e2e_setup(self, torch, dev):
        self.h_codes = torch.empty(self.codes.shape, dtype=torch.uint8, pin_memory=True)
        self.h_codes.copy_(self.codes)
        self.h_out = torch.empty(self.out.shape[0], dtype=torch.float32, pin_memory=True)

    def e2e_step(self):
        self.codes.copy_(self.h_codes, non_blocking=True)
        self.step()
        self.h_out.copy_(self.out[:, 0], non_blocking=True)

    def e2e_units_per_step(self):
        return self.units_per_step()

    def e2e_bytes(self):
        return self.h_codes.numel(), self.h_out.numel() * 4

    def cpu_sample(self, orc, T=256):
        import numpy as np

        E = self.H * self.D
        rng = np.random.default_rng(0)
        codes = rng.integers(0, 0x70, (T, 3 * E), dtype=np.uint8)
        t0 = time.perf_counter()
        orc.attention_fp8(codes, orc.E4M3, 0.01, 1, T, self.H, self.D)
        dt = time.perf_counter() - t0
        return 4.0 * self.H * T * T * self.D / 1e12, dt, f"one sequence of {T} tokens, {self.H} heads"

class Gpt2ShardedWorkload(Gpt2Workload):
    """BASELINE configs[4]: the 6.7B-shape GPT-2 forward (32 layers, d_model 4096, 32 heads, FFN 16384, context 2048,
    batch 16 x 2048 token ids, the same on every rank) with the fully-connected weights column-sharded over the
    GPUs and NCCL all-gathers between the layers (dnn::Gpt2ColumnSharded).  Total work is fixed: strong scaling.
    Weights are uniform with the standard deviation of N(0, 0.02), generated on the device."""

    CFG = dict(layers=32, hidden=4096, heads=32, ffn=16384, vocab=50257, ctx=2048, batch=16, act="e4m3")

    def __init__(self, n_gpus=1, batch=None, layers=None):
        self.name = "gpt67"
        self.c = dict(self.CFG)
        if layers:
            self.c["layers"] = layers
        self.n_gpus = n_gpus
        self.strong = True
        self.B = batch or self.c["batch"]
        self.T = self.c["ctx"]
        self.metric = "GPT-2 fp8 forward tokens/s"
        self.dtype = "e4m3 activations x e4m3 weights -> f32 accumulate"
        # embedding; per layer: 2 x (LayerNorm 2), QKV 2 passes, attention, quantise, gather + interleave, out GEMM,
        # gather + interleave, add, FC1 2 passes, gather + interleave, FC2, gather + interleave, add; head 3
        per_layer = 15 + (8 if n_gpus > 1 else 4)
        self.kernels_per_step = 1 + per_layer * self.c["layers"] + 3

    def config(self, n_gpus):
        c = self.c
        return {"workload": f"GPT-2 6.7B-shape fp8 forward: {c['layers']} layers, d_model {c['hidden']}, {c['heads']} "
                            f"heads, FFN {c['ffn']}, vocab {c['vocab']}, batch {self.B}x{self.T} token ids (the same "
                            f"on every rank), fp32 logits sharded by vocabulary rows, random-init weights",
                "global_batch": self.B, "seq_len": self.T, "weights": "resident e4m3 codes, 1/N of every matrix per GPU",
                "l2_policy": "working set per forward far larger than L2",
                "parallelism": f"fully-connected weights column-sharded x{n_gpus}, attention by heads, NCCL all-reduce(max) "
                               f"of per-tensor maxima and all-gather of fp8 codes / fp32 residual updates"}

    def units_per_step(self):
        return self.B * self.T / self.n_gpus  # every rank works on all tokens: count each token once

    def setup(self, torch, df8, dev, rank):
        import oracle as orc

        self.torch, self.df8, self.dev = torch, df8, dev
        c = self.c
        d = df8.dnn_lib()
        df8.dnn_check(d.dnn_init(dev.index), "dnn_init")
        df8.dnn_check(d.dnn_set_fp8_policy(0, 0))
        df8.dnn_check(d.dnn_set_host_init(0))
        self.comm = df8.Comm(rank, self.n_gpus)
        self.model = df8.Gpt2ColumnSharded(self.comm, vocab=c["vocab"], max_seq_len=c["ctx"], layers=c["layers"],
                                           heads=c["heads"], hidden=c["hidden"], ffn=c["ffn"], device=dev.index)
        df8.dnn_check(d.dnn_set_host_init(1))
        self.model.set_stream(torch.cuda.current_stream())
        self.model.initialize_on_device(4)
        self.model.set_options(gelu=True, causal=False)
        ids = orc.fill_token_ids(self.B * self.T, seed=4, vocab=c["vocab"]).reshape(self.B, self.T)
        self.ids = torch.from_numpy(ids).to(dev)
        self.ids_host = torch.from_numpy(ids).pin_memory()
        self.last_logits = torch.empty((self.B, self.model.vocab_rows), dtype=torch.float32, pin_memory=True)

    def step(self):
        self.logits_ptr = self.model.forward_logits_shard(self.ids, check_ids=False)

    def e2e_step(self):
        torch = self.torch
        ptr = self.model.forward_logits_shard_host(self.ids_host)
        logits = self.df8.device_view(torch, ptr, (self.B, self.T, self.model.vocab_rows))
        self.last_logits.copy_(logits[:, -1, :], non_blocking=True)

    def e2e_units_per_step(self):
        return self.units_per_step()

    def roofline(self, torch, peaks, iters=5):
        # dominant kernel: this rank's FC1 product [B*T, F/N] x [F/N, E], one fp8-codes pass
        d, c = self.df8, self.c
        M, N, K = self.B * self.T, c["ffn"] // self.n_gpus, c["hidden"]
        g = torch.Generator(device=self.dev)
        g.manual_seed(1)
        a = torch.randint(0, 0x70, (M, K), dtype=torch.uint8, device=self.dev, generator=g)
        w = torch.randint(0, 0x70, (N, K), dtype=torch.uint8, device=self.dev, generator=g)
        one = torch.tensor([1.0, 1.0 / 64], device=self.dev)
        out = torch.empty((M, N), dtype=torch.uint8, device=self.dev)
        amax, osc = torch.zeros(1, device=self.dev), torch.zeros(2, device=self.dev)
        for _ in range(2):
            d.gemm_fp8_tn_q(a, 0, one, w, 0, one, None, M, N, K, 1, 0, out, osc, amax)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(iters):
            d.gemm_fp8_tn_q(a, 0, one, w, 0, one, None, M, N, K, 1, 0, out, osc, amax)
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1]) / iters / 2  # two passes per call
        flops = 2.0 * M * N * K
        tf = flops / 1e12 / (ms / 1e3)
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        return {"kernel": "gemm_fp8_tn_pair_kernel (FC1 shard, average of its two passes)", "bound": "tensor",
                "achieved": round(tf, 1), "peak": peak, "peak_source": peaks["source"] + " bf16 sustained x2 (fp8 dense)",
                "unit": "TFLOP/s", "frac": round(tf / peak, 4), "ms_per_launch": round(ms, 4),
                "algorithmic_flops_per_launch": flops, "traffic": None,
                "model_flops_per_token": gpt2_flops_per_token(c, self.T)}

    def cpu_sample(self, orc, tokens=32):
        return super().cpu_sample(orc, tokens=tokens)


WORKLOADS = {"attn": AttnWorkload, "quant": QuantWorkload, "gemm": GemmWorkload, "gpt2s": Gpt2Workload, "gpt2m": Gpt2Workload,
             "gpt67": Gpt2ShardedWorkload}
DEFAULT_WORKLOAD = "gpt2s"


def make_workload(args):
    if args.workload == "quant" and args.log2n:
        return QuantWorkload(log2n=args.log2n)
    if args.workload == "gemm" and args.only:
        return GemmWorkload(only=args.only.split(","))
    if args.workload == "gpt67":
        return Gpt2ShardedWorkload(n_gpus=max(1, int(os.environ.get("WORLD_SIZE", args.gpus))), batch=args.batch,
                                   layers=args.layers)
    if args.workload in GPT2_CONFIGS:
        return Gpt2Workload(args.workload, n_gpus=max(1, int(os.environ.get("WORLD_SIZE", args.gpus))),
                            batch=args.batch, layers=args.layers)
    return WORKLOADS[args.workload]()


# ---------------------------------------------------------------------------------------------

def run_reference(args, rank, world):
    """CPU arm: the oracle port of the upstream host-side math on all host threads (rank 0 only)."""
    if rank != 0:
        return
    import oracle as orc

    orc.build()
    wl = make_workload(args)
    cores = orc.get_threads()
    for _ in range(min(max(args.warmup, 1), 1)):
        wl.cpu_sample(orc)  # one warm-up sample (page-in of the oracle library, thread pool start)
    units, secs, sample = 0.0, 0.0, ""
    for _ in range(args.steps):
        u, dt, sample = wl.cpu_sample(orc)
        units += u
        secs += dt
    value = units / secs
    line = {
        "impl": "reference", "metric": wl.metric, "value": round(value, 3), "unit": wl.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * secs / args.steps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": wl.config(args.gpus),
        "cpu_baseline": {"value": round(value, 3), "unit": wl.unit, "cores": cores, "kind": "port",
                         "sample": sample + " per step; upstream has no CPU implementation of this path, "
                                            "the oracle port of its host-side math is timed"},
        "e2e": {"value": round(value, 3), "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import deepfuse_b200 as df8

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    df8.lib()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    peaks = _peaks()
    wl = make_workload(args)
    wl.setup(torch, df8, dev, rank)

    for _ in range(args.warmup):
        wl.step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        wl.step()
    end.record()
    barrier()
    ms_total = start.elapsed_time(end)
    clocks = sampler.stop() if rank == 0 else None

    # end-to-end: host buffers, copies inside the timed region
    wl.e2e_setup(torch, dev)
    for _ in range(2):
        wl.e2e_step()
    barrier()
    e_steps = max(2, min(args.steps, 5))
    start.record()
    for _ in range(e_steps):
        wl.e2e_step()
    end.record()
    barrier()
    e2e_ms_total = start.elapsed_time(end)

    if world > 1:
        t = torch.tensor([ms_total, e2e_ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms_total = t.tolist()

    if rank == 0:
        value = wl.units_per_step() * world * args.steps / (ms_total / 1e3)
        e2e_value = wl.e2e_units_per_step() * world * e_steps / (e2e_ms_total / 1e3)
        h2d, d2h = wl.e2e_bytes()
        roofline = wl.roofline(torch, peaks)
        import oracle as orc

        orc.build()
        units, secs, sample = wl.cpu_sample(orc)
        line = {
            "metric": wl.metric, "value": round(value, 2), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_total / args.steps, 4), "higher_is_better": True,
            "scaling": "strong" if getattr(wl, "strong", False) else "weak", "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic", "config": wl.config(world), "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": wl.unit, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e_steps},
            "gpu_launches": wl.kernels_per_step * args.steps,
            "roofline": roofline,
            "cpu_baseline": {"value": round(units / secs, 3), "unit": wl.unit, "cores": orc.get_threads(),
                             "kind": "port", "sample": sample},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="gpt2 workloads: sequences per GPU (profiling)")
    ap.add_argument("--layers", type=int, default=None, help="gpt2 workloads: layer count override (profiling)")
    ap.add_argument("--only", default=None, help="gemm workload: comma list of projections (profiling)")
    ap.add_argument("--log2n", type=int, default=None, help="quant workload: tensor size override (profiling)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1 and args.impl == "ours":
        # convenience: relaunch under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29531"),
               str(Path(__file__).resolve()), *sys.argv[1:]]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
