#!/usr/bin/env python
"""Benchmark of the fp8 fully-connected + attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference] [--extras none]

Prints ONE JSON line (rank 0).  A "step" is one pass of the hot path over one batch of seeded synthetic input.

The default workload is the GPT-2 small fp8 forward (12 layers, d_model 768, vocabulary 50257, 8 x 1024 token ids per
GPU -> fp32 logits, e4m3 weights and activations) through dnn::Gpt2; tokens/s.  Its line carries:

  value            device-timed tokens/s (CUDA events, ids resident in HBM), exactly --steps steps
  sustained        the same forward looped for >= 3 s with the SM clock sampled (a power-capped figure beside the short one)
  e2e              Gpt2.serve_step with pinned HOST ids, and the FULL [B*T, vocab] fp32 logits copied back to pinned
                   host memory every step inside the timed region (1.65 GB per step: PCIe-bound); step i's copy runs
                   on a stream of its own under step i + 1's forward
  e2e_serial       the same with forward and copy back to back on one stream
  e2e_next_token   the same with only the last position's logits copied back (what a sampling loop needs)
  roofline         the longest single launch (vocabulary-head GEMM) timed with events INSIDE the forward
  gemm_tflops      fp8 GEMM TFLOP/s per projection shape of GPT-2 small and of the 6.7B shape  (the other half of
  quant_gbs        the metric) and quantise / dequantise GB/s for e4m3 and e5m2 at 2^20 ... 2^30 elements
  streamed_medium  GPT-2 medium, e5m2 activations, weights streamed per layer from pinned host memory, the fixed
                   batch of 32 sequences split over the GPUs (strong scaling)
  column_sharded   the 6.7B-shape forward with fully-connected weights column-sharded over the GPUs (strong scaling)
  cpu_baseline     the oracle port of the upstream host-side math on the box's cores (N = 1 only)

Other workloads (profiling): gemm, quant, attn, gpt2m, gpt67.  `--extras none` prints the main figures only.
`--impl reference` times the CPU oracle alone (upstream has no CPU implementation of this path).

Under torchrun (N > 1) every rank runs the same per-GPU work (weak scaling of the default workload, no data-path
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
    """Samples nvidia-smi SM clocks and throttle reasons while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

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
            return self
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()
        # nvidia-smi stalls kernel launches while it attaches to the driver: let it produce its first
        # sample before the timed region begins
        t0 = time.time()
        while not self.lines and time.time() - t0 < 5.0:
            time.sleep(0.02)
        return self

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
        sm, mx, pw, reasons = [], [], [], set()
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
            if len(parts) > 6:
                try:
                    pw.append(float(parts[6]))
                except ValueError:
                    pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "samples": len(sm), "reasons": sorted(reasons)}
        if pw:
            out["power_w_max"] = max(pw)
        return out


def _event_ms(torch, fn, iters, warm=3):
    """Average device time of fn() over `iters` back-to-back calls (CUDA events on the current stream)."""
    for _ in range(warm):
        fn()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    ev[0].record()
    for _ in range(iters):
        fn()
    ev[1].record()
    torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[1]) / iters


# ---------------------------------------------------------------------------------------------
# kernel-level workloads (also the secondary figures of the default line)
# ---------------------------------------------------------------------------------------------

class QuantWorkload:
    """amax + quantise + dequantise of one fp32 tensor, all through the C-ABI."""

    name = "quant"
    metric = "fp8 quantise+dequantise round-trip GB/s"
    unit = "GB/s"
    dtype = "f32->e4m3->f32"
    bytes_per_elem = 14  # 4 (amax read) + 4 (re-read) + 1 (codes) + 1 (codes read) + 4 (fp32 write)
    kernels_per_step = 3
    strong = False

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
        self.x = _device_normal_outliers(torch, dev, self.n, self.seed + rank)
        self.amax = torch.zeros(1, device=dev)
        self.scale = torch.zeros(2, device=dev)
        self.codes = torch.empty(self.n, dtype=torch.uint8, device=dev)
        self.y = torch.empty(self.n, device=dev)

    def step(self):
        d = self.df8
        d.amax_f32(self.x, self.amax)
        d.quantize_f32(self.x, d.E4M3, self.amax, self.codes, self.scale)
        d.dequantize_f32(self.codes, d.E4M3, self.scale, self.y)

    def roofline(self, torch, peaks):
        d = self.df8
        d.amax_f32(self.x, self.amax)
        ms = _event_ms(torch, lambda: d.quantize_f32(self.x, d.E4M3, self.amax, self.codes, self.scale), 10)
        achieved = self.n * 5 / 1e9 / (ms / 1e3)
        return {"kernel": "quantize_f32_kernel<e4m3>", "bound": "hbm", "achieved": round(achieved, 1),
                "peak": peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy bandwidth", "unit": "GB/s",
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

    def cpu_sample(self, orc, step=0, log2n=25):
        n = 1 << log2n
        x = orc.fill_normal_outliers(n, seed=self.seed)
        t0 = time.perf_counter()
        a = orc.amax(x)
        codes, s = orc.quantize(x, orc.E4M3, amax_v=a)
        orc.dequantize(codes, orc.E4M3, s[1])
        dt = time.perf_counter() - t0
        return n * self.bytes_per_elem / 1e9, dt, dt, f"2^{log2n} elements of the same distribution"


def _device_normal_outliers(torch, dev, n, seed):
    """N(0,1) with 0.1 % of the positions replaced by 100 x N(0,1), made on the device."""
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = torch.randn(n, device=dev, generator=g)
    k = max(1, n // 1000)
    idx = torch.randint(0, n, (k,), device=dev, generator=g)
    x[idx] = 100.0 * torch.randn(k, device=dev, generator=g)
    return x


def quant_sweep(torch, df8, dev, peaks):
    """amax + quantise + dequantise at 2^20 ... 2^30 elements, e4m3 and e5m2: GB/s of algorithmic traffic
    (round trip 14 B/element, amax + quantise 9 B/element) and the fraction of the copy bandwidth."""
    out = {"unit": "GB/s", "peak": peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy bandwidth",
           "bytes_per_element": {"round_trip": 14, "amax_quantise": 9, "dequantise": 5},
           "note": "tensors of 2^24 elements and fewer (<= 64 MB fp32) stay L2-resident between the passes and the "
                   "repeats; their figures are not HBM figures", "sizes": {}}
    n_max = 1 << 30
    x_all = _device_normal_outliers(torch, dev, n_max, 1)
    codes_all = torch.empty(n_max, dtype=torch.uint8, device=dev)
    y_all = torch.empty(n_max, device=dev)
    amax, scale = torch.zeros(1, device=dev), torch.zeros(2, device=dev)
    for log2n in range(20, 31):
        n = 1 << log2n
        x, codes, y = x_all[:n], codes_all[:n], y_all[:n]
        iters = max(5, min(200, (1 << 31) // n))
        row = {}
        for kind, kname in ((df8.E4M3, "e4m3"), (df8.E5M2, "e5m2")):
            def q():
                df8.amax_f32(x, amax)
                df8.quantize_f32(x, kind, amax, codes, scale)

            def rt():
                q()
                df8.dequantize_f32(codes, kind, scale, y)

            ms_q = _event_ms(torch, q, iters)
            ms_rt = _event_ms(torch, rt, iters)
            g_q, g_rt = n * 9 / 1e6 / ms_q, n * 14 / 1e6 / ms_rt
            row[kname] = {"round_trip": round(g_rt, 1), "amax_quantise": round(g_q, 1),
                          "round_trip_frac": round(g_rt / peaks["hbm_gbs"], 3)}
        out["sizes"][f"2^{log2n}"] = row
    del x_all, codes_all, y_all
    torch.cuda.empty_cache()
    return out


PROJECTIONS = {
    # name: (N, K, flags) with flags 1 GELU, 2 residual, 8 two-pass fp8-codes output (df8_gemm_fp8_tn_q), 16 pitched rows
    "gpt2_small": dict(M=8192, E=768, F=3072, V=50257),
    "6.7b_shape": dict(M=32768, E=4096, F=16384, V=50257),
}


def projection_set(c):
    E, F, V = c["E"], c["F"], c["V"]
    return [("qkv", 3 * E, E, 8), ("out", E, E, 2), ("fc1_gelu", F, E, 1 | 8), ("fc2", E, F, 2), ("head", V, E, 16)]


def gemm_sweep(torch, df8, dev, peaks, sets=("gpt2_small", "6.7b_shape")):
    """fp8 GEMM TFLOP/s of every projection of a transformer layer + the vocabulary head, as the forward calls them:
    QKV and FC1 through the two-pass fp8-codes form (the flops are counted once although the tensor work runs
    twice), out-projection and FC2 with the residual add, the head into row-pitched fp32 logits."""
    peak = 2.0 * peaks["bf16_tflops"]
    out = {"unit": "TFLOP/s", "peak": peak, "peak_source": peaks["source"] + " bf16 burst x2 (fp8 dense)",
           "note": "each shape timed alone, 10-20 launches back to back; qkv / fc1_gelu emit per-tensor-quantised "
                   "fp8 codes in two tensor-core passes and count 2MNK once", "sets": {}}
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    one = torch.tensor([1.0, 1.0 / 64], device=dev)
    for sname in sets:
        c = PROJECTIONS[sname]
        M = c["M"]
        rows = {}
        total_flops, total_ms = 0.0, 0.0
        for name, N, K, flags in projection_set(c):
            a = torch.randint(0, 0x78, (M, K), dtype=torch.uint8, device=dev, generator=g)
            w = torch.randint(0, 0x60, (N, K), dtype=torch.uint8, device=dev, generator=g)
            w |= torch.randint(0, 2, (N, K), dtype=torch.uint8, device=dev, generator=g) * 0x80
            bias = torch.zeros(N, device=dev)
            amax, osc = torch.zeros(1, device=dev), torch.zeros(2, device=dev)
            if flags & 8:
                o = torch.empty((M, N), dtype=torch.uint8, device=dev)
                fn = lambda: df8.gemm_fp8_tn_q(a, 0, one, w, 0, one, bias, M, N, K, flags & 1, 0, o, osc, amax)
            elif flags & 16:
                ldc = (N + 31) // 32 * 32
                o = torch.empty((M, ldc), device=dev)
                fn = lambda: df8.gemm_fp8_tn_ex(a, 0, one, 1, w, 0, one, bias, None, M, N, K, 0, o, ldc)
            else:
                o = torch.empty((M, N), device=dev)
                res = torch.randn(M, N, device=dev, generator=g)
                fn = lambda: df8.gemm_fp8_tn(a, 0, one, w, 0, one, bias, res, M, N, K, flags & 3, o)
            ms = _event_ms(torch, fn, 10 if sname != "gpt2_small" else 20)
            fl = 2.0 * M * N * K
            rows[name] = {"shape": [M, N, K], "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
                          "frac": round(fl / ms / 1e9 / peak, 3)}
            total_flops += fl
            total_ms += ms
            del a, w, o
        rows["all"] = {"ms": round(total_ms, 4), "tflops": round(total_flops / total_ms / 1e9, 1),
                       "frac": round(total_flops / total_ms / 1e9 / peak, 3)}
        out["sets"][sname] = rows
        torch.cuda.empty_cache()
    return out


class GemmWorkload:
    """The fp8 projections of one GPT-2 layer at M tokens plus the vocabulary head (profiling workload)."""

    name = "gemm"
    metric = "fp8 GEMM TFLOP/s"
    unit = "TFLOP/s"
    dtype = "e4m3 x e4m3 -> f32"
    strong = False

    def __init__(self, M=8192, E=768, F=3072, V=50257, only=None):
        self.M, self.E, self.F, self.V = M, E, F, V
        shapes = [("qkv", 3 * E, E, 4), ("out", E, E, 2), ("fc1", F, E, 1 | 4), ("fc2", E, F, 2), ("head", V, E, 0)]
        # --only: big / big4k (large square problems), qkvq / fc1q (two-pass fp8-codes output), headp (pitched logits)
        extra = [("big", 8192, 8192, 0), ("big4k", 8192, 4096, 0), ("qkvq", 3 * E, E, 8), ("fc1q", F, E, 1 | 8),
                 ("headp", V, E, 16)]
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
        for name, N, K, flags in self.shapes:
            a = torch.randint(0, 0x78, (self.M, K), dtype=torch.uint8, device=dev, generator=g)
            w = torch.randint(0, 0x60, (N, K), dtype=torch.uint8, device=dev, generator=g)
            w = w | (torch.randint(0, 2, (N, K), dtype=torch.uint8, device=dev, generator=g) * 0x80)
            bias = torch.zeros(N, device=dev)
            res = torch.randn(self.M, N, device=dev, generator=g) if flags & 2 else None
            ldc = (N + 31) // 32 * 32 if flags & 16 else N
            out = (torch.empty(self.M, N, dtype=torch.uint8, device=dev) if flags & 8
                   else torch.empty(self.M, ldc, device=dev))
            self.ops.append((a, w, bias, res, out, torch.zeros(1, device=dev), N, K, flags, ldc))
        self.one = torch.tensor([1.0, 1.0 / 64], device=dev)
        self.out_scale = torch.zeros(2, device=dev)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def _call(self, op):
        d = self.df8
        a, w, bias, res, out, amax, N, K, flags, ldc = op
        if flags & 8:
            d.gemm_fp8_tn_q(a, d.E4M3, self.one, w, d.E4M3, self.one, bias, self.M, N, K, flags & 1, d.E4M3, out,
                            self.out_scale, amax)
        else:
            d.gemm_fp8_tn_ex(a, d.E4M3, self.one, 1, w, d.E4M3, self.one, bias, res, self.M, N, K, flags & 7, out, ldc,
                             amax)

    def step(self):
        self.flush.zero_()
        for op in self.ops:
            self._call(op)

    def roofline(self, torch, peaks):
        per, best = {}, None
        for (name, _, _, _), op in zip(self.shapes, self.ops):
            N, K = op[6], op[7]
            ms = _event_ms(torch, lambda: self._call(op), 20)
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
        last = self.ops[-1][4]
        self.h_out.copy_(last[:, 0] if last.dtype == self.torch.float32 else last[:, 0].float(), non_blocking=True)

    def e2e_units_per_step(self):
        return self.units_per_step()

    def e2e_bytes(self):
        return self.h_a.numel(), self.h_out.numel() * 4

    def cpu_sample(self, orc, step=0, rows=16):
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
        return units, secs, secs, f"{rows} token rows (and at most 4096 output columns) of each projection"


class AttnWorkload:
    """df8_attention_fp8 on a GPT-2 small sized QKV code buffer (B=8, T=1024, H=12, D=64), non-causal."""

    name = "attn"
    metric = "fp8 attention TFLOP/s"
    unit = "TFLOP/s"
    dtype = "e4m3 QKV -> f32"
    kernels_per_step = 1
    strong = False

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

    def _call(self):
        self.df8.attention_fp8(self.codes, 0, self.scale, self.B, self.T, self.H, self.D, 0, None, self.out, self.amax)

    def step(self):
        self.flush.zero_()
        self._call()

    def roofline(self, torch, peaks):
        ms = _event_ms(torch, self._call, 20)
        tf = self.units_per_step() / (ms / 1e3)
        peak = 2.0 * peaks["bf16_tflops"]
        wide = self.D == 64 and self.T % 256 == 0 and os.environ.get("DF8_ATTN_WIDE", "1")[:1] != "0"
        return {"kernel": "attention_fp8_wide_kernel" if wide else f"attention_fp8_kernel<{self.D}>",
                "bound": "tensor", "achieved": round(tf, 1), "peak": peak,
                "peak_source": peaks["source"] + " bf16 burst x2 (fp8 dense)", "unit": "TFLOP/s",
                "frac": round(tf / peak, 4), "ms_per_launch": round(ms, 4),
                "algorithmic_flops_per_launch": self.units_per_step() * 1e12, "traffic": None}

    def e2e_setup(self, torch, dev):
        self.h_codes = torch.empty(self.codes.shape, dtype=torch.uint8, pin_memory=True)
        self.h_codes.copy_(self.codes)
        self.h_out = torch.empty(self.out.shape, dtype=torch.float32, pin_memory=True)

    def e2e_step(self):
        self.codes.copy_(self.h_codes, non_blocking=True)
        self.step()
        self.h_out.copy_(self.out, non_blocking=True)

    def e2e_units_per_step(self):
        return self.units_per_step()

    def e2e_bytes(self):
        return self.h_codes.numel(), self.h_out.numel() * 4

    def cpu_sample(self, orc, step=0, T=256):
        import numpy as np

        E = self.H * self.D
        rng = np.random.default_rng(0)
        codes = rng.integers(0, 0x70, (T, 3 * E), dtype=np.uint8)
        t0 = time.perf_counter()
        orc.attention_fp8(codes, orc.E4M3, 0.01, 1, T, self.H, self.D)
        dt = time.perf_counter() - t0
        return 4.0 * self.H * T * T * self.D / 1e12, dt, dt, f"one sequence of {T} tokens, {self.H} heads"


# ---------------------------------------------------------------------------------------------
# GPT-2 forward workloads
# ---------------------------------------------------------------------------------------------

GPT2_CONFIGS = {
    # name: layers, hidden, heads, ffn, vocab, context, batch, activation kind, weight seed
    "gpt2s": dict(layers=12, hidden=768, heads=12, ffn=3072, vocab=50257, ctx=1024, batch=8, act="e4m3", seed=2),
    "gpt2m": dict(layers=24, hidden=1024, heads=16, ffn=4096, vocab=50257, ctx=1024, batch=32, act="e5m2", seed=3),
}


def gpt2_flops_per_token(c, T):
    E, F, V, L = c["hidden"], c["ffn"], c["vocab"], c["layers"]
    return L * (2 * (3 * E * E + E * E + 2 * E * F) + 4 * T * E) + 2 * E * V


class Gpt2Workload:
    """GPT-2 fp8 forward (token ids -> fp32 logits) through dnn::Gpt2<float>.  The logits live in a row-pitched
    buffer [B*T, 50272] (Gpt2::forward_logits_pitched: rows of 50257 floats do not start on 16-byte boundaries);
    the end-to-end legs copy the dense [B*T, 50257] rows out of it."""

    unit = "tokens/s"

    def __init__(self, name="gpt2s", n_gpus=1, batch=None, layers=None, slots=2):
        self.name = name
        self.c = dict(GPT2_CONFIGS[name])
        if layers:
            self.c["layers"] = layers
        self.n_gpus = n_gpus
        self.slots = int(os.environ.get("DF8_BENCH_STREAM_SLOTS", slots))  # device slots of the layer streamer (gpt2m)
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
                "weights": ("e4m3 codes of the block weights in pinned host memory, streamed per layer through "
                            f"{self.slots} device slots on a side stream"
                            + (f", each rank uploading 1/{n_gpus} of a layer and an NVLink all-gather completing it"
                               if n_gpus > 1 else "")) if self.name == "gpt2m" else "resident e4m3 codes",
                "logits": "fp32 [B*T, 50257] in a row-pitched buffer (pitch 50272 floats)",
                "l2_policy": "working set per forward (1.65 GB of logits alone) larger than L2",
                "parallelism": f"batch-sharded x{n_gpus}, weights replicated, no data-path collective"}

    def units_per_step(self):
        return self.B * self.T

    def setup(self, torch, df8, dev, rank, comm=None):
        from deepfuse_b200 import synthetic

        self.torch, self.df8 = torch, df8
        c = self.c
        cfg = dict(vocab=c["vocab"], max_seq_len=c["ctx"], layers=c["layers"], heads=c["heads"], hidden=c["hidden"],
                   ffn=c["ffn"])
        d = df8.dnn_lib()
        df8.dnn_check(d.dnn_init(dev.index), "dnn_init")
        df8.dnn_check(d.dnn_set_fp8_policy(0, 0 if c["act"] == "e4m3" else 1))
        df8.dnn_check(d.dnn_set_host_init(0))  # weights are generated on the device below
        try:
            self.model = df8.Gpt2(**cfg, device=dev.index)
        finally:
            df8.dnn_check(d.dnn_set_host_init(1))
        self.model.set_stream(torch.cuda.current_stream())
        self.model.initialize_on_device(c["seed"], 0.02)
        self.model.set_options(gelu=True, causal=False)
        if self.name == "gpt2m":  # e4m3 weights held in pinned host memory, streamed per layer
            self.model.enable_streaming(slots=self.slots, release_fp32=True, comm=comm)
        ids = synthetic.fill_token_ids(self.B * self.T, seed=100 * c["seed"] + rank, vocab=c["vocab"]).reshape(self.B, self.T)
        self.ids = torch.from_numpy(ids).to(dev)
        self.ids_host = torch.from_numpy(ids).pin_memory()
        self.dev = dev
        self.full_logits = None
        self.last_logits = None

    def close(self):
        self.model.close()
        self.full_logits = self.last_logits = None

    def step(self):
        self.logits_ptr, self.pitch = self.model.forward_logits_pitched(self.ids, check_ids=False)

    # end to end: pinned host ids in, logits out to pinned host memory, both inside the timed region
    def e2e_setup(self, torch, dev, full=True):
        V = self.c["vocab"]
        if full and self.full_logits is None:
            self.full_logits = torch.empty((self.B * self.T, V), dtype=torch.float32, pin_memory=True)
        if self.last_logits is None:
            self.last_logits = torch.empty((self.B, V), dtype=torch.float32, pin_memory=True)

    def e2e_step(self):
        self.model.forward_logits_pitched(self.ids_host, check_ids=False)
        self.model.copy_logits_host(self.full_logits)

    # the same as a serving loop issues it: step i's logits travel to the host on a stream of their own while step
    # i + 1 computes; two pinned host buffers alternate, the last copy is waited for inside the timed region
    def e2e_setup_pipelined(self, torch):
        if getattr(self, "full_logits_b", None) is None:
            self.full_logits_b = torch.empty_like(self.full_logits).pin_memory()
        self._serve_i = 0

    def e2e_step_pipelined(self):
        dst = self.full_logits if self._serve_i % 2 == 0 else self.full_logits_b
        self._serve_i += 1
        self.model.serve_step(self.ids_host, dst)

    def e2e_flush_pipelined(self):
        self.model.serve_flush()

    def e2e_step_next_token(self):
        torch, V = self.torch, self.c["vocab"]
        ptr, pitch = self.model.forward_logits_pitched(self.ids_host, check_ids=False)
        logits = self.df8.device_view(torch, ptr, (self.B, self.T, pitch))
        self.last_logits.copy_(logits[:, -1, :V], non_blocking=True)

    def e2e_units_per_step(self):
        return self.units_per_step()

    def e2e_bytes(self):
        return self.ids_host.numel() * 4, self.full_logits.numel() * 4

    def roofline(self, torch, peaks, iters=20):
        """The vocabulary-head GEMM [B*T, E] x [V, E]^T, timed by two events around its launch inside the forward
        (Gpt2::set_stage_timing), i.e. on the model's own tensors with the cache state the blocks leave."""
        c = self.c
        M, N, K = self.B * self.T, c["vocab"], c["hidden"]
        self.model.set_stage_timing(True)
        ms_list = []
        for _ in range(iters + 2):
            self.step()
            ms_list.append(self.model.last_head_ms())
        self.model.set_stage_timing(False)
        ms_list = sorted(ms_list[2:])
        ms = sum(ms_list) / len(ms_list)
        flops = 2.0 * M * N * K
        tf = flops / 1e12 / (ms / 1e3)
        peak = 2.0 * peaks["bf16_tflops"]
        wbytes = M * N * 4
        write_roof_ms = wbytes / (peaks["hbm_gbs"] * 1e9) * 1e3
        return {"kernel": "gemm_fp8_tn_pair_kernel (vocabulary head, CTA pairs, TMA-store epilogue)", "bound": "tensor", "achieved": round(tf, 1),
                "peak": peak, "peak_source": peaks["source"] + " bf16 burst x2 (fp8 dense); the launch runs at full clock "
                                                                "inside a forward of a few ms",
                "unit": "TFLOP/s", "frac": round(tf / peak, 4),
                "frac_of_sustained_peak": round(tf / (2.0 * peaks["bf16_tflops_sustained"]), 4),
                "ms_per_launch": round(ms, 4), "ms_per_launch_min_max": [round(ms_list[0], 4), round(ms_list[-1], 4)],
                "timed": f"CUDA events around the launch inside {iters} forwards", "algorithmic_flops_per_launch": flops,
                # the roof that binds this shape: 1.65 GB of logits written once
                "hbm_write_roof": {"bytes": wbytes, "ms_at_peak": round(write_roof_ms, 4), "peak_gbs": peaks["hbm_gbs"],
                                   "achieved_gbs": round(wbytes / ms / 1e6, 1), "frac": round(write_roof_ms / ms, 4)},
                # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this launch at batch 8 x 1024
                # (profiles/gemm_fp8_tn_pair_kernel_head_8192x50257x768.md), scaled by the rows
                "traffic": round((61.2e6 + 1.588e9) * M / 8192) if c["hidden"] == 768 else None,
                "model_flops_per_token": gpt2_flops_per_token(c, self.T)}

    def cpu_sample(self, orc, step=0):
        """One 1024-token sequence through ONE of the identical transformer blocks at the full context, plus the
        vocabulary head; the block's time counts `layers` times (every block has the same shapes).  Returns
        (tokens, seconds of the full forward, seconds actually spent, description)."""
        from oracle import gpt2_ref

        c = self.c
        E, T = c["hidden"], self.T
        cfg = dict(vocab=c["vocab"], max_seq_len=c["ctx"], layers=1, heads=c["heads"], hidden=E, ffn=c["ffn"])
        if getattr(self, "_cpu_prm", None) is None:
            self._cpu_prm = gpt2_ref.make_params(cfg, seed=c["seed"])
        prm = self._cpu_prm
        x = orc.fill_normal(T * E, seed=7 + step).reshape(T, E)
        act = orc.E4M3 if c["act"] == "e4m3" else orc.E5M2
        t0 = time.perf_counter()
        y = gpt2_ref.block_forward(prm, "block0", x, 1, T, c["heads"], act, orc.E4M3, True)
        t_block = time.perf_counter() - t0
        rows = T // 4  # the head is a product per token row: a quarter of the rows, counted four times
        t0 = time.perf_counter()
        gpt2_ref._fc(y[:rows], prm["final_fc.weight"], prm["final_fc.bias"], act, orc.E4M3)
        t_head = time.perf_counter() - t0
        return (T, t_block * c["layers"] + t_head * (T / rows), t_block + t_head,
                f"one {T}-token sequence through one transformer block at the full context + the vocabulary head on "
                f"{rows} of its rows per step; the block counts {c['layers']} times (identical shapes) and the head "
                f"{T // rows} times (independent rows): extrapolated, not a full forward")


class Gpt2ShardedWorkload(Gpt2Workload):
    """The 6.7B-shape GPT-2 forward (32 layers, d_model 4096, 32 heads, FFN 16384, context 2048, batch 16 x 2048
    token ids, the same on every rank) with the fully-connected weights column-sharded over the GPUs
    (dnn::Gpt2ColumnSharded).  Total work is fixed: strong scaling.  Weights ~N(0, 0.02) generated on the device."""

    CFG = dict(layers=32, hidden=4096, heads=32, ffn=16384, vocab=50257, ctx=2048, batch=16, act="e4m3", seed=4)

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
        per_layer = 15 + (8 if n_gpus > 1 else 4)
        self.kernels_per_step = 1 + per_layer * self.c["layers"] + 3

    def config(self, n_gpus):
        c = self.c
        return {"workload": f"GPT-2 6.7B-shape fp8 forward: {c['layers']} layers, d_model {c['hidden']}, {c['heads']} "
                            f"heads, FFN {c['ffn']}, vocab {c['vocab']}, batch {self.B}x{self.T} token ids (the same "
                            f"on every rank), fp32 logits sharded by vocabulary rows, random-init weights",
                "global_batch": self.B, "seq_len": self.T, "weights": "resident e4m3 codes, 1/N of every matrix per GPU",
                "l2_policy": "working set per forward far larger than L2",
                "parallelism": f"fully-connected weights column-sharded x{n_gpus}, attention by heads, per-tensor maxima "
                               f"and fp8 codes exchanged between the GPUs"}

    def units_per_step(self):
        return self.B * self.T / self.n_gpus  # every rank works on all tokens: count each token once

    def setup(self, torch, df8, dev, rank, comm=None):
        from deepfuse_b200 import synthetic

        self.torch, self.df8, self.dev = torch, df8, dev
        c = self.c
        d = df8.dnn_lib()
        df8.dnn_check(d.dnn_init(dev.index), "dnn_init")
        df8.dnn_check(d.dnn_set_fp8_policy(0, 0))
        df8.dnn_check(d.dnn_set_host_init(0))
        self.comm = comm if comm is not None else df8.Comm(rank, self.n_gpus)
        self.owns_comm = comm is None
        try:
            self.model = df8.Gpt2ColumnSharded(self.comm, vocab=c["vocab"], max_seq_len=c["ctx"], layers=c["layers"],
                                               heads=c["heads"], hidden=c["hidden"], ffn=c["ffn"], device=dev.index)
        finally:
            df8.dnn_check(d.dnn_set_host_init(1))
        self.model.set_stream(torch.cuda.current_stream())
        self.model.initialize_on_device(c["seed"])
        self.model.set_options(gelu=True, causal=False)
        ids = synthetic.fill_token_ids(self.B * self.T, seed=c["seed"], vocab=c["vocab"]).reshape(self.B, self.T)
        self.ids = torch.from_numpy(ids).to(dev)
        self.ids_host = torch.from_numpy(ids).pin_memory()
        self.last_logits = torch.empty((self.B, self.model.vocab_rows), dtype=torch.float32, pin_memory=True)

    def close(self):
        self.model.close()
        if self.owns_comm:
            self.comm.close()

    def step(self):
        self.logits_ptr, self.pitch = self.model.forward_logits_shard_pitched(self.ids, check_ids=False)

    def e2e_setup(self, torch, dev, full=True):
        pass

    def e2e_step(self):
        torch = self.torch
        ptr, pitch = self.model.forward_logits_shard_pitched(self.ids_host, check_ids=False)
        logits = self.df8.device_view(torch, ptr, (self.B, self.T, pitch))
        self.last_logits.copy_(logits[:, -1, :self.model.vocab_rows], non_blocking=True)

    e2e_step_next_token = e2e_step

    def e2e_bytes(self):
        return self.ids_host.numel() * 4, self.last_logits.numel() * 4

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
        ms = _event_ms(torch, lambda: d.gemm_fp8_tn_q(a, 0, one, w, 0, one, None, M, N, K, 1, 0, out, osc, amax),
                       iters, warm=2) / 2  # two passes per call
        flops = 2.0 * M * N * K
        tf = flops / 1e12 / (ms / 1e3)
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        return {"kernel": "gemm_fp8_tn_pair_kernel (FC1 shard, average of its two passes)", "bound": "tensor",
                "achieved": round(tf, 1), "peak": peak,
                "peak_source": peaks["source"] + " bf16 sustained x2 (fp8 dense): the forward runs for hundreds of ms "
                                                 "under the power cap",
                "unit": "TFLOP/s", "frac": round(tf / peak, 4), "ms_per_launch": round(ms, 4),
                "algorithmic_flops_per_launch": flops, "traffic": None,
                "model_flops_per_token": gpt2_flops_per_token(c, self.T)}

    def cpu_sample(self, orc, step=0):
        raise RuntimeError("the 6.7B shape has no CPU sample of its own; see the default workload's cpu_baseline")


WORKLOADS = {"attn": AttnWorkload, "quant": QuantWorkload, "gemm": GemmWorkload, "gpt2s": Gpt2Workload, "gpt2m": Gpt2Workload,
             "gpt67": Gpt2ShardedWorkload}
DEFAULT_WORKLOAD = "gpt2s"


SIDE_REPORTS = {"ce": lambda *a: cross_entropy_report(*a), "decode": lambda *a: decode_report(*a),
                "decode_128": lambda *a: decode_report(*a, batch=128),
                "fc_backward": lambda *a: fc_backward_report(*a)}
WORKLOADS.update({k: None for k in SIDE_REPORTS})


def make_workload(args, world):
    if args.workload == "quant":
        return QuantWorkload(log2n=args.log2n or 30)
    if args.workload == "gemm":
        return GemmWorkload(only=args.only.split(",") if args.only else None)
    if args.workload == "gpt67":
        return Gpt2ShardedWorkload(n_gpus=world, batch=args.batch, layers=args.layers)
    if args.workload in GPT2_CONFIGS:
        return Gpt2Workload(args.workload, n_gpus=world, batch=args.batch, layers=args.layers)
    return WORKLOADS[args.workload]()


# ---------------------------------------------------------------------------------------------
# the CPU arm
# ---------------------------------------------------------------------------------------------

def run_reference(args, rank, world):
    """CPU arm: the oracle port of the upstream host-side math on all host threads (rank 0 only).  `ms_per_step` is
    the wall time a step really took; for the GPT-2 workloads a step times one of the identical blocks + the head
    and `value` counts the block `layers` times (see cpu_baseline.sample), which the line says in `extrapolated`."""
    if rank != 0:
        return
    import oracle as orc

    orc.build()
    wl = make_workload(args, max(1, args.gpus))
    cores = orc.get_threads()
    wl.cpu_sample(orc)  # one warm-up sample (page-in of the oracle library, thread pool start, weights)
    units, model_secs, spent, sample = 0.0, 0.0, 0.0, ""
    for i in range(args.steps):
        u, ms, sp, sample = wl.cpu_sample(orc, step=i)
        units += u
        model_secs += ms
        spent += sp
    value = units / model_secs
    extrapolated = abs(model_secs - spent) > 1e-9
    line = {
        "impl": "reference", "metric": wl.metric, "value": round(value, 3), "unit": wl.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * spent / args.steps, 3),
        "higher_is_better": True, "scaling": "strong" if wl.strong else "weak", "vs_baseline": None, "dtype": wl.dtype,
        "data": "synthetic", "config": wl.config(args.gpus), "extrapolated": extrapolated,
        "ms_per_step_means": "wall time of one step's CPU sample" + (
            "; `value` = sample tokens / (block time x layers + head time), i.e. the full forward's tokens/s with one "
            "of the identical blocks timed per step" if extrapolated else ""),
        "cpu_baseline": {"value": round(value, 3), "unit": wl.unit, "cores": cores, "kind": "port",
                         "sample": sample + "; upstream has no CPU implementation of this path, the oracle port of "
                                            "its host-side math is timed"},
        "e2e": {"value": round(value, 3), "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# the GPU arm
# ---------------------------------------------------------------------------------------------

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

    def max_over_ranks(*vals):
        if world == 1:
            return list(vals)
        t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def timed(step_fn, steps, sample_clocks=False):
        """K steps bracketed by barrier + synchronize; device time, max over ranks."""
        barrier()
        sampler = ClockSampler(local_rank).start() if (sample_clocks and rank == 0) else None
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(steps):
            step_fn()
        end.record()
        barrier()
        ms = max_over_ranks(start.elapsed_time(end))[0]
        return ms, (sampler.stop() if sampler else None)

    peaks = _peaks()
    extras = args.extras == "all"
    wl = make_workload(args, world)
    comm = None
    if world > 1 and isinstance(wl, Gpt2Workload):
        comm = df8.Comm(rank, world)
    if isinstance(wl, Gpt2Workload):
        wl.setup(torch, df8, dev, rank, comm=comm)
    else:
        wl.setup(torch, df8, dev, rank)

    for _ in range(args.warmup):
        wl.step()
    torch.cuda.nvtx.range_push("df8_timed_steps")  # lets a profiler pick exactly the timed launches
    ms_total, clocks = timed(wl.step, args.steps, sample_clocks=True)
    torch.cuda.nvtx.range_pop()
    status = df8.status_word()

    line = None
    if rank == 0:
        value = wl.units_per_step() * world * args.steps / (ms_total / 1e3)
        line = {
            "metric": wl.metric, "value": round(value, 2), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_total / args.steps, 4), "higher_is_better": True,
            "scaling": "strong" if wl.strong else "weak", "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic", "config": wl.config(world), "clocks": clocks,
            "gpu_launches": wl.kernels_per_step * args.steps,
            "device_wait_status": list(status),
        }

    # the same forward for at least 3 s: a figure under the power cap beside the short one
    if extras and isinstance(wl, Gpt2Workload):
        per_step = ms_total / args.steps
        n_long = max(args.steps, int(3200.0 / per_step) + 1)
        ms_long, clocks_long = timed(wl.step, n_long, sample_clocks=True)
        if rank == 0:
            line["sustained"] = {"value": round(wl.units_per_step() * world * n_long / (ms_long / 1e3), 2),
                                 "unit": wl.unit, "steps": n_long, "seconds": round(ms_long / 1e3, 2),
                                 "ms_per_step": round(ms_long / n_long, 4), "clocks": clocks_long}

    # end to end: host buffers, copies inside the timed region
    wl.e2e_setup(torch, dev)
    for _ in range(2):
        wl.e2e_step()
    e_steps = max(2, min(args.steps, 5))
    e2e_ms, _ = timed(wl.e2e_step, e_steps)
    if rank == 0:
        h2d, d2h = wl.e2e_bytes()
        line["e2e"] = {"value": round(wl.e2e_units_per_step() * world * e_steps / (e2e_ms / 1e3), 2), "unit": wl.unit,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e_steps,
                       "ms_per_step": round(e2e_ms / e_steps, 4),
                       "what": "pinned host ids in; the full fp32 logits [B*T, vocab] copied back to pinned host memory"
                       if isinstance(wl, Gpt2Workload) and not isinstance(wl, Gpt2ShardedWorkload) else
                       "host buffers in and out through the C-ABI"}
    if isinstance(wl, Gpt2Workload) and not isinstance(wl, Gpt2ShardedWorkload):
        # the serving call: step i's logits cross PCIe on a stream of their own while step i + 1 computes
        p_steps = max(e_steps, 6)
        issued = {"n": 0}

        def pipelined_step():
            wl.e2e_step_pipelined()
            issued["n"] += 1
            if issued["n"] == p_steps:
                wl.e2e_flush_pipelined()  # the last copy ends inside the timed region

        pl_ok = 1
        try:  # a second 1.65 GB pinned buffer per rank: if the host refuses it, the one-stream figure stays the e2e
            wl.e2e_setup_pipelined(torch)
            for _ in range(2):
                wl.e2e_step_pipelined()
            wl.e2e_flush_pipelined()
            torch.cuda.synchronize()
        except Exception:
            pl_ok = 0
        pl_ok = 0 if max_over_ranks(float(1 - pl_ok))[0] > 0 else 1  # every rank or none (the timed legs hold barriers)
        pl_ms = None
        if pl_ok:
            pl_ms, _ = timed(pipelined_step, p_steps)
        if rank == 0 and pl_ms is not None:
            line["e2e_serial"] = dict(line["e2e"], what="pinned host ids in; forward, then the full fp32 logits [B*T, vocab] "
                                                        "copied back to pinned host memory, on one stream")
            line["e2e"] = {"value": round(wl.e2e_units_per_step() * world * p_steps / (pl_ms / 1e3), 2), "unit": wl.unit,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": p_steps,
                           "ms_per_step": round(pl_ms / p_steps, 4),
                           "what": "Gpt2.serve_step: pinned host ids in, the full fp32 logits [B*T, vocab] copied back to "
                                   "pinned host memory every step; the copy of step i runs on a stream of its own under "
                                   "the forward of step i + 1, the last copy is waited for inside the timed region"}
        for _ in range(2):
            wl.e2e_step_next_token()
        nt_ms, _ = timed(wl.e2e_step_next_token, e_steps)
        if rank == 0:
            line["e2e_next_token"] = {"value": round(wl.units_per_step() * world * e_steps / (nt_ms / 1e3), 2),
                                      "unit": wl.unit, "h2d_bytes_per_step": wl.ids_host.numel() * 4,
                                      "d2h_bytes_per_step": wl.last_logits.numel() * 4, "steps": e_steps,
                                      "what": "pinned host ids in; only the last position's logits [B, vocab] copied back"}
        wl.full_logits = wl.full_logits_b = None  # 2 x 1.65 GB of pinned memory (released after the timed legs: unpinning stalls the device)

    roofline = wl.roofline(torch, peaks)  # every rank runs it (keeps the ranks in step); rank 0 reports
    if rank == 0:
        line["roofline"] = roofline

    if extras and isinstance(wl, Gpt2Workload) and args.workload == DEFAULT_WORKLOAD:
        wl.close()
        torch.cuda.empty_cache()
        sec = {}
        # the other half of the metric: per-shape GEMM TFLOP/s and quantiser GB/s (rank 0's GPU; the others wait)
        if rank == 0:
            for key, fn in (("gemm_tflops", lambda: gemm_sweep(torch, df8, dev, peaks)),
                            ("quant_gbs", lambda: quant_sweep(torch, df8, dev, peaks)),
                            ("decode", lambda: decode_report(torch, df8, dev, peaks)),
                            ("decode_128", lambda: decode_report(torch, df8, dev, peaks, batch=128)),
                            ("cross_entropy", lambda: cross_entropy_report(torch, df8, dev, peaks)),
                            ("fc_backward", lambda: fc_backward_report(torch, df8, dev, peaks))):
                try:
                    sec[key] = fn()
                except Exception as e:  # a secondary figure must not take the line down
                    sec[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.empty_cache()
        barrier()
        # the two configurations that have something to limit their scaling
        for key, make in (("streamed_medium", lambda: Gpt2Workload("gpt2m", n_gpus=world)),
                          ("column_sharded", lambda: Gpt2ShardedWorkload(n_gpus=world))):
            rec = secondary_forward(torch, df8, dev, rank, world, comm, make, timed, barrier, max_over_ranks)
            if rank == 0:
                sec[key] = rec
            torch.cuda.empty_cache()
        if rank == 0:
            line.update(sec)

    if rank == 0 and world == 1:
        import oracle as orc

        orc.build()
        units = model_secs = 0.0
        sample = ""
        base = wl if not isinstance(wl, Gpt2ShardedWorkload) else Gpt2Workload("gpt2s")
        for i in range(3):
            u, ms, _, sample = base.cpu_sample(orc, step=i)
            units += u
            model_secs += ms
        line["cpu_baseline"] = {"value": round(units / model_secs, 3), "unit": base.unit, "cores": orc.get_threads(),
                                "kind": "port", "sample": sample + " (3 steps)"}
    if rank == 0:
        line["device_wait_status"] = list(df8.status_word())
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


def decode_report(torch, df8, dev, peaks, batch=32, prompt=128, steps=64):
    """Autoregressive decode of GPT-2 small after a prefill: one new token per sequence and step through the KV cache
    (Gpt2::prefill / decode_step).  A step streams every weight code and the cached keys / values once: HBM-bound by
    its algorithmic bytes, launch-bound in practice at this model size (about ten kernels of a few microseconds per
    layer), which is what the record shows."""
    from deepfuse_b200 import synthetic

    c = dict(GPT2_CONFIGS["gpt2s"])
    cfg = dict(vocab=c["vocab"], max_seq_len=c["ctx"], layers=c["layers"], heads=c["heads"], hidden=c["hidden"], ffn=c["ffn"])
    d = df8.dnn_lib()
    df8.dnn_check(d.dnn_set_fp8_policy(0, 0))
    df8.dnn_check(d.dnn_set_host_init(0))
    try:
        model = df8.Gpt2(**cfg, device=dev.index)
    finally:
        df8.dnn_check(d.dnn_set_host_init(1))
    side = torch.cuda.Stream(device=dev)  # a stream of its own: the model replays a step from a CUDA graph there
    side.wait_stream(torch.cuda.current_stream())
    ctx = torch.cuda.stream(side)
    ctx.__enter__()
    try:
        model.set_stream(side)
        model.initialize_on_device(c["seed"], 0.02)
        model.set_options(gelu=True, causal=True)
        ids = torch.from_numpy(synthetic.fill_token_ids(batch * prompt, seed=7, vocab=c["vocab"]).reshape(batch, prompt)).to(dev)
        nxt = torch.from_numpy(synthetic.fill_token_ids(batch, seed=8, vocab=c["vocab"])).to(dev)
        max_len = prompt + 2 * steps + 8
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        model.prefill(ids, max_len=max_len)
        e1.record()
        torch.cuda.synchronize()
        prefill_ms = e0.elapsed_time(e1)
        for _ in range(steps // 4):
            model.decode_step(nxt, check_ids=False)
        torch.cuda.synchronize()
        n0 = prompt + steps // 4
        e0.record()
        for _ in range(steps):
            model.decode_step(nxt, check_ids=False)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        E, F, V, L = c["hidden"], c["ffn"], c["vocab"], c["layers"]
        weight_bytes = L * (3 * E * E + E * E + 2 * E * F) + V * E
        n_avg = n0 + (steps - 1) / 2.0
        kv_bytes = int(batch * L * 2 * n_avg * E)
        logits_bytes = batch * V * 4
        algo = weight_bytes + kv_bytes + logits_bytes
        gbs = algo / (ms * 1e6)
        graph = model.decode_graph_active()
        model.end_decode()
        return {"metric": "GPT-2 small fp8 decode tokens/s", "value": round(batch / (ms / 1e3), 1), "unit": "tokens/s",
                "ms_per_step": round(ms, 4), "steps": steps, "batch": batch, "prompt": prompt, "prefill_ms": round(prefill_ms, 3),
                "algorithmic_bytes_per_step": {"weight_codes": weight_bytes, "kv_cache_read": kv_bytes, "logits": logits_bytes},
                "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": "measured copy bandwidth"},
                "config": {"workload": f"GPT-2 small, {batch} sequences, prompt {prompt}, one token per sequence and step, "
                                       "KV cache of fp8 codes with one scale per position, causal"},
                "cuda_graph": graph, "device_wait_status": list(df8.status_word())}
    finally:
        ctx.__exit__(None, None, None)
        torch.cuda.current_stream().wait_stream(side)
        model.set_stream(torch.cuda.current_stream())  # the library's stream is process-wide
        model.close()


def cross_entropy_report(torch, df8, dev, peaks, rows=8192, classes=50257):
    """Softmax cross-entropy on the head's logits (df8_cross_entropy_f32 / _grad_f32): per-row loss from pitched
    fp32 logits and class indices, and the gradient.  HBM-bound: the logits cross HBM once per call (the second and
    third pass over a row find it in L2), the gradient is written once."""
    import ctypes as C

    from deepfuse_b200 import synthetic

    pitch = (classes + 31) // 32 * 32
    logits = torch.randn((rows, pitch), device=dev)
    idx = torch.from_numpy(synthetic.fill_token_ids(rows, seed=3, vocab=classes)).to(dev)
    row_loss = torch.empty(rows, device=dev)
    grad = torch.empty((rows, classes), device=dev)
    lib, st = df8.lib(), df8.stream_ptr()

    def timeit(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    ms_loss = timeit(lambda: df8.check(lib.df8_cross_entropy_f32(df8.ptr(logits), pitch, None, 0, df8.ptr(idx), rows, classes,
                                                                 df8.ptr(row_loss), st)))
    ms_grad = timeit(lambda: df8.check(lib.df8_cross_entropy_grad_f32(df8.ptr(logits), pitch, None, 0, df8.ptr(idx), rows,
                                                                      classes, df8.ptr(grad), classes, st)))
    bad = C.c_uint(0)
    df8.check(lib.df8_cross_entropy_bad_indices(C.byref(bad), 1))
    b_loss, b_grad = rows * classes * 4, 2 * rows * classes * 4
    return {"unit": "GB/s", "peak": peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy bandwidth",
            "shape": [rows, classes], "row_pitch": pitch, "targets": "class indices",
            "loss": {"ms": round(ms_loss, 4), "algorithmic_bytes": b_loss, "gbs": round(b_loss / ms_loss / 1e6, 1),
                     "frac": round(b_loss / ms_loss / 1e6 / peaks["hbm_gbs"], 4)},
            "gradient": {"ms": round(ms_grad, 4), "algorithmic_bytes": b_grad, "gbs": round(b_grad / ms_grad / 1e6, 1),
                         "frac": round(b_grad / ms_grad / 1e6 / peaks["hbm_gbs"], 4)},
            "mean_row_loss": round(float(row_loss.mean().item()), 4), "bad_indices": bad.value}


def fc_backward_report(torch, df8, dev, peaks, M=8192):
    """Backward of GPT-2 small's FC1 and FC2 at M tokens as the layer runs it (FullyConnectedLayer::backward): max|dY| and
    db in one pass, dY quantised to e5m2 in both layouts (one read), the weight codes transposed, dX = dY W, max|X|, X quantised transposed,
    dW = dY^T X, db = column sums.  TFLOP/s counts the two products (4 M N K)."""
    lib, st = df8.lib(), df8.stream_ptr()
    out = {"unit": "TFLOP/s", "peak": 2.0 * peaks["bf16_tflops"], "peak_source": peaks["source"] + " bf16 burst x2 (fp8 dense)",
           "tokens": M, "kinds": "dY e5m2, X e4m3, W e4m3 -> f32 accumulate", "layers": {}}
    for name, K, N in (("fc1", 768, 3072), ("fc2", 3072, 768)):  # in_features K, out_features N
        x = torch.randn((M, K), device=dev)
        dy = torch.randn((M, N), device=dev) * 1e-3
        w_codes = torch.randint(0, 120, (N, K), dtype=torch.uint8, device=dev)
        w_scale = torch.tensor([448.0, 1.0 / 448.0], device=dev)
        amax = torch.zeros(2, device=dev)
        dy_scale, x_scale = torch.zeros(2, device=dev), torch.zeros(2, device=dev)
        dy_t = torch.empty((N, M), dtype=torch.uint8, device=dev)
        dy_c = torch.empty((M, N), dtype=torch.uint8, device=dev)
        w_t = torch.empty((K, N), dtype=torch.uint8, device=dev)
        x_t = torch.empty((K, M), dtype=torch.uint8, device=dev)
        dx = torch.empty((M, K), device=dev)
        dw = torch.empty((N, K), device=dev)
        db = torch.empty(N, device=dev)
        partial = torch.empty(lib.df8_colsum_partial_floats(N), device=dev)

        def step():
            c = df8.check
            c(lib.df8_colsum_amax_f32(df8.ptr(dy), M, N, N, df8.ptr(partial), df8.ptr(db), df8.ptr(amax), st))
            c(lib.df8_quantize_both_layouts_f32(df8.ptr(dy), M, N, 1, df8.ptr(amax), df8.ptr(dy_t), M, df8.ptr(dy_c), N,
                                                df8.ptr(dy_scale), st))
            c(lib.df8_transpose_u8(df8.ptr(w_codes), N, K, K, df8.ptr(w_t), N, st))
            c(lib.df8_gemm_fp8_tn(df8.ptr(dy_c), 1, df8.ptr(dy_scale), df8.ptr(w_t), 0, df8.ptr(w_scale), None, None, M, K, N, 0,
                                  df8.ptr(dx), None, st))
            c(lib.df8_amax_f32(df8.ptr(x), x.numel(), df8.ptr(amax[1:]), st))
            c(lib.df8_quantize_transpose_f32(df8.ptr(x), M, K, 0, df8.ptr(amax[1:]), df8.ptr(x_t), M, df8.ptr(x_scale), st))
            c(lib.df8_gemm_fp8_tn(df8.ptr(dy_t), 1, df8.ptr(dy_scale), df8.ptr(x_t), 0, df8.ptr(x_scale), None, None, N, K, M, 0,
                                  df8.ptr(dw), None, st))

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        tf = 4.0 * M * N * K / ms / 1e9
        out["layers"][name] = {"shape_in_out": [K, N], "ms": round(ms, 4), "tflops": round(tf, 1), "frac": round(tf / out["peak"], 4),
                               "launches": 7}
    return out


def secondary_forward(torch, df8, dev, rank, world, comm, make, timed, barrier, max_over_ranks, steps=5, warmup=3):
    """tokens/s of another GPT-2 configuration at this GPU count, as a record of the default line."""
    wl = None
    try:
        wl = make()
        wl.setup(torch, df8, dev, rank, comm=comm)
        for _ in range(warmup):
            wl.step()
        ms, clocks = timed(wl.step, steps, sample_clocks=True)
        rec = {"metric": wl.metric, "value": round(wl.units_per_step() * world * steps / (ms / 1e3), 2),
               "unit": wl.unit, "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 3),
               "scaling": "strong", "config": wl.config(world), "dtype": wl.dtype, "clocks": clocks,
               "model_flops_per_token": gpt2_flops_per_token(wl.c, wl.T)}
        rec["model_tflops"] = round(rec["value"] * rec["model_flops_per_token"] / 1e12, 1)
        if hasattr(wl.model, "bytes_pushed"):
            b0 = wl.model.bytes_pushed()
            wl.step()
            torch.cuda.synchronize()
            pushed = wl.model.bytes_pushed() - b0
            rec["exchange"] = {"bytes_pushed_per_forward_per_rank": pushed,
                               "transport": "peer-mapped buffers + copy engines" if pushed > 0 else
                               ("none (single rank)" if world == 1 else "NCCL fallback"),
                               "nvlink_gbs_if_fully_exposed": round(pushed / (ms / steps) / 1e6, 1)}
        if getattr(wl.model, "_streaming", False):
            rec["streaming"] = streaming_report(torch, wl, steps + warmup, ms / steps, timed, max_over_ranks, barrier)
        rec["device_wait_status"] = list(df8.status_word())
        return rec
    except Exception as e:
        return {"error": f"{type(e).__name__}: {e}"[:400]}
    finally:
        try:
            if wl is not None and getattr(wl, "model", None) is not None:
                wl.close()
        except Exception:
            pass
        barrier()


def streaming_report(torch, wl, passes, ms_streamed, timed, max_over_ranks, barrier):
    """Host->device and NVLink bytes per rank and forward of the layer streamer, the rate of the uploads when they
    run alone, and how much of that upload time a forward hides under its compute:
    overlap = (upload alone - (streamed forward - forward with every layer resident)) / upload alone."""
    rep = {}
    try:
        h2d, gathered = wl.model.streaming_traffic()
        rep["h2d_bytes_per_forward_per_rank"] = h2d // max(1, passes)
        rep["gathered_bytes_per_forward_per_rank"] = gathered // max(1, passes)
        h0, g0 = wl.model.streaming_traffic()
        barrier()  # the ranks enter together: a sharded upload waits for its slowest peer
        up_ms = max_over_ranks(wl.model.time_uploads())[0]
        h1, g1 = wl.model.streaming_traffic()
        wl.model.resize_streaming_slots(wl.c["layers"])  # every layer resident after one pass
        wl.step()
        ms_res, _ = timed(wl.step, 3)
        ms_res /= 3
        rep.update({"upload_alone_ms": round(up_ms, 3), "forward_resident_ms": round(ms_res, 3),
                    "forward_streamed_ms": round(ms_streamed, 3),
                    "h2d_gbs_per_rank_alone": round((h1 - h0) / up_ms / 1e6, 1),
                    "nvlink_gbs_per_rank_alone": round((g1 - g0) / up_ms / 1e6, 1),
                    "overlap_fraction": round(max(0.0, min(1.0, (up_ms - (ms_streamed - ms_res)) / up_ms)), 3)})
    except Exception as e:
        rep["error"] = f"{type(e).__name__}: {e}"[:200]
    return rep


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extras", default="all", choices=["all", "none"],
                    help="none: main figures only (no sustained loop, no secondary records); for profiling")
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
    if args.workload in SIDE_REPORTS:  # one of the default line's secondary records on its own (profiling): rank 0's GPU
        if rank == 0 and args.impl == "ours":
            import torch

            import deepfuse_b200 as df8

            torch.cuda.set_device(local_rank)
            df8.lib()
            print(json.dumps({args.workload: SIDE_REPORTS[args.workload](torch, df8, torch.device("cuda", local_rank), _peaks())}),
                  flush=True)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
