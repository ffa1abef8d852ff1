"""Generates the committed golden fixtures of tests/golden/ from the CPU oracle, whose fp8
conversion is the CUDA toolkit's cuda_fp8.h host function.  Run from the repository root:

    python tests/golden/make_golden.py

The fixtures let `-m "not gpu"` tests notice any drift of the oracle itself (a toolkit change, an
edit to the generator), and give the GPU tests fixed vectors that do not depend on the oracle
being rebuilt on the GPU box.
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle as O  # noqa: E402

HERE = Path(__file__).resolve().parent


def main():
    O.build()
    # quantiser: 4096 seeded values with outliers + hand-picked edge values
    x = O.fill_normal_outliers(4096, seed=1)
    edge = np.array([0.0, -0.0, 1.0, -1.0, 448.0, 500.0, 2.0 ** -10, 17.0, 18.0, 19.0, 57344.0, 70000.0, 1e-10,
                     -3.5e4, 2.0 ** -17, 1.0e-3], dtype=np.float32)
    x = np.concatenate([x, edge]).astype(np.float32)
    out = {"x": x}
    for kind, name in ((O.E4M3, "e4m3"), (O.E5M2, "e5m2")):
        codes, s = O.quantize(x, kind)
        out[f"codes_{name}"] = codes
        out[f"scale_{name}"] = s
        out[f"deq_{name}"] = O.dequantize(codes, kind, s[1])
    np.savez_compressed(HERE / "quant_golden.npz", **out)

    # decode table of every code
    table = {name: [O.code_value(c, kind) for c in range(256)] for kind, name in ((O.E4M3, "e4m3"), (O.E5M2, "e5m2"))}
    np.savez_compressed(HERE / "fp8_code_values.npz", **{k: np.array(v, np.float32) for k, v in table.items()})

    # config-1 shaped FC (64x768 -> 3072) through the fp8 oracle, seed 0
    M, K, N = 64, 768, 3072
    xf = O.fill_normal(M * K, seed=0).reshape(M, K)
    wf = O.fill_normal(N * K, seed=100, std=0.02).reshape(N, K)
    xc, sx = O.quantize(xf, O.E4M3)
    wc, sw = O.quantize(wf, O.E4M3)
    y = O.fc_forward_fp8(xc, O.E4M3, sx[1], wc, O.E4M3, sw[1], np.zeros(N, np.float32))
    yb = O.fc_forward_f32(xf, wf, np.zeros(N, np.float32))
    np.savez_compressed(HERE / "fc_config1_golden.npz", y_fp8_rows8=y[:8].astype(np.float32), y_f32_row0=yb[0],
                        scale_x=sx, scale_w=sw, x_codes_row0=xc[0], w_codes_row0=wc[0])

    meta = {
        "normal_outliers_seed1_first4": [float(v) for v in O.fill_normal_outliers(4096, seed=1)[:4]],
        "token_ids_seed2_first4": [int(v) for v in O.fill_token_ids(1000, seed=2, vocab=50257)[:4]],
    }
    (HERE / "synthetic_meta.json").write_text(json.dumps(meta, indent=1) + "\n")


if __name__ == "__main__":
    main()
