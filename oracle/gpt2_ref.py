"""CPU oracle of the fp8 GPT-2 forward pipeline.  TEST INFRASTRUCTURE ONLY.

Composes the per-kernel oracle functions (oracle/df8_oracle.cpp) in the order the upstream project wires
its model: embedding + bias (dnn/tokens/token_embedding.cu:37-44), sinusoidal positions
(dnn/tokens/positional_encoding.cu:20-27,44-47), pre-LayerNorm blocks (dnn/layers/transformer_block.cu:59-86:
x1 = x + MHA(LN1(x)); y = x1 + FC2(act(FC1(LN2(x1))))), vocabulary head without a final LayerNorm
(dnn/models/gpt2.cu:66-83).  Where the 8-bit path quantises, this does too, at the same places: every
tensor that feeds a GEMM or the attention is quantised per tensor (scale = FP8_MAX / amax); weights are
quantised once.  `gelu=False` reproduces upstream's block, which applies no activation (:79-81).
"""
from __future__ import annotations

import numpy as np

import oracle as O


def make_params(cfg: dict, seed: int, std: float = 0.02) -> dict:
    """Seeded N(0, std) weights, zero biases, LayerNorm gamma 1 / beta 0, in the naming of
    dnn_gpt2_param_info (include/df8_dnn.h)."""
    V, E, F, L = cfg["vocab"], cfg["hidden"], cfg["ffn"], cfg["layers"]
    p = {}
    k = [seed * 1000]

    def normal(shape):
        k[0] += 1
        return O.fill_normal(int(np.prod(shape)), seed=k[0], std=std).reshape(shape)

    p["embedding.weight"] = normal((V, E))
    p["embedding.bias"] = np.zeros(E, np.float32)
    for i in range(L):
        b = f"block{i}"
        p[f"{b}.ln1.gamma"] = np.ones(E, np.float32)
        p[f"{b}.ln1.beta"] = np.zeros(E, np.float32)
        p[f"{b}.ln2.gamma"] = np.ones(E, np.float32)
        p[f"{b}.ln2.beta"] = np.zeros(E, np.float32)
        p[f"{b}.qkv.weight"] = normal((3 * E, E))
        p[f"{b}.qkv.bias"] = np.zeros(3 * E, np.float32)
        p[f"{b}.out.weight"] = normal((E, E))
        p[f"{b}.out.bias"] = np.zeros(E, np.float32)
        p[f"{b}.fc1.weight"] = normal((F, E))
        p[f"{b}.fc1.bias"] = np.zeros(F, np.float32)
        p[f"{b}.fc2.weight"] = normal((E, F))
        p[f"{b}.fc2.bias"] = np.zeros(E, np.float32)
    p["final_fc.weight"] = normal((V, E))
    p["final_fc.bias"] = np.zeros(V, np.float32)
    return p


def _fc(x_f32, w, b, act_kind, w_kind, residual=None, gelu=False):
    if act_kind is None:  # unquantised fp32 layer (upstream's FullyConnectedLayer math), for error budgets
        y = O.fc_forward_f32(x_f32, w, b)
        if gelu:
            y = O.gelu(y)
        return y + residual if residual is not None else y
    xc, xs = O.quantize(x_f32, act_kind)
    wc, ws = O.quantize(w, w_kind)
    flags = (O.GELU if gelu else 0) | (O.RESIDUAL if residual is not None else 0)
    return O.fc_forward_fp8(xc, act_kind, xs[1], wc, w_kind, ws[1], b, residual, flags)


def _attention(qkv, B, T, heads, act_kind, mask_mode, mask):
    E = qkv.shape[1] // 3
    D = E // heads
    if act_kind is not None:
        qc, qs = O.quantize(qkv, act_kind)
        return O.attention_fp8(qc, act_kind, qs[1], B, T, heads, D, mask_mode, mask)
    # fp32 attention with the upstream softmax (softmax_layer.cu:26-81), numpy matmuls in float64
    v = qkv.astype(np.float64).reshape(B, T, 3, heads, D)
    q, k, val = (v[:, :, n].transpose(0, 2, 1, 3) for n in range(3))
    scores = (q @ k.transpose(0, 1, 3, 2) / np.sqrt(D)).astype(np.float32)
    if mask_mode == O.MASK_CAUSAL:
        i, j = np.meshgrid(np.arange(T), np.arange(T), indexing="ij")
        mask = np.where(j <= i, 0.0, -1e9).astype(np.float32)[None, None]
    prob = O.softmax_masked(scores, mask if mask_mode != O.MASK_NONE else None).astype(np.float64)
    return (prob @ val).transpose(0, 2, 1, 3).reshape(B * T, E).astype(np.float32)


def block_forward(p: dict, prefix: str, x: np.ndarray, B: int, T: int, heads: int, act_kind: int, w_kind: int,
                  gelu: bool, mask_mode: int = O.MASK_NONE, mask=None) -> np.ndarray:
    """x [B*T, E] fp32 -> block output [B*T, E]."""
    E = x.shape[1]
    h = O.layernorm(x, p[f"{prefix}.ln1.gamma"], p[f"{prefix}.ln1.beta"], 1e-5)
    qkv = _fc(h, p[f"{prefix}.qkv.weight"], p[f"{prefix}.qkv.bias"], act_kind, w_kind)
    a = _attention(qkv, B, T, heads, act_kind, mask_mode, mask)
    x1 = _fc(a, p[f"{prefix}.out.weight"], p[f"{prefix}.out.bias"], act_kind, w_kind, residual=x)
    h2 = O.layernorm(x1, p[f"{prefix}.ln2.gamma"], p[f"{prefix}.ln2.beta"], 1e-5)
    f = _fc(h2, p[f"{prefix}.fc1.weight"], p[f"{prefix}.fc1.bias"], act_kind, w_kind, gelu=gelu)
    return _fc(f, p[f"{prefix}.fc2.weight"], p[f"{prefix}.fc2.bias"], act_kind, w_kind, residual=x1)


def block_trace(p: dict, prefix: str, x: np.ndarray, B: int, T: int, heads: int, act_kind: int, w_kind: int,
                gelu: bool, mask_mode: int = O.MASK_NONE, mask=None) -> dict:
    """block_forward with every intermediate kept, so that a test can feed the ORACLE's input into one GPU
    kernel at a time (a code that flips in one kernel then cannot compound through the chain).  Keys:
    ln1 / qkv / attn / x1 / ln2 / h / y are fp32 tensors; `<name>_q` = (codes, scale {q, dq}) of the tensors the
    8-bit path quantises (ln1, qkv, attn, ln2, h); w_<layer> = (codes, scale) of the four weight matrices."""
    t = {"x": x}
    qz = lambda a: O.quantize(a, act_kind)
    for name in ("qkv", "out", "fc1", "fc2"):
        t[f"w_{name}"] = O.quantize(p[f"{prefix}.{name}.weight"], w_kind)

    def fc(aq, name, residual=None, flags=0):
        wc, ws = t[f"w_{name}"]
        return O.fc_forward_fp8(aq[0], act_kind, aq[1][1], wc, w_kind, ws[1], p[f"{prefix}.{name}.bias"], residual,
                                flags | (O.RESIDUAL if residual is not None else 0))

    t["ln1"] = O.layernorm(x, p[f"{prefix}.ln1.gamma"], p[f"{prefix}.ln1.beta"], 1e-5)
    t["ln1_q"] = qz(t["ln1"])
    t["qkv"] = fc(t["ln1_q"], "qkv")
    t["qkv_q"] = qz(t["qkv"])
    E = x.shape[1]
    t["attn"] = O.attention_fp8(t["qkv_q"][0], act_kind, t["qkv_q"][1][1], B, T, heads, E // heads, mask_mode, mask)
    t["attn_q"] = qz(t["attn"])
    t["x1"] = fc(t["attn_q"], "out", residual=x)
    t["ln2"] = O.layernorm(t["x1"], p[f"{prefix}.ln2.gamma"], p[f"{prefix}.ln2.beta"], 1e-5)
    t["ln2_q"] = qz(t["ln2"])
    t["h"] = fc(t["ln2_q"], "fc1", flags=O.GELU if gelu else 0)
    t["h_q"] = qz(t["h"])
    t["y"] = fc(t["h_q"], "fc2", residual=t["x1"])
    return t


def mha_forward(p: dict, prefix: str, x: np.ndarray, B: int, T: int, heads: int, act_kind: int, w_kind: int,
                mask_mode: int = O.MASK_NONE, mask=None) -> np.ndarray:
    """MultiHeadAttentionLayer::forward on x [B*T, E]: QKV projection, attention, output projection."""
    qkv = _fc(x, p[f"{prefix}.qkv.weight"], p[f"{prefix}.qkv.bias"], act_kind, w_kind)
    a = _attention(qkv, B, T, heads, act_kind, mask_mode, mask)
    return _fc(a, p[f"{prefix}.out.weight"], p[f"{prefix}.out.bias"], act_kind, w_kind)


def gpt2_forward(p: dict, ids: np.ndarray, cfg: dict, act_kind: int = O.E4M3, w_kind: int = O.E4M3, gelu: bool = True,
                 causal: bool = False, return_hidden: bool = False) -> np.ndarray:
    """ids [B,T] int32 -> logits [B*T, V] (or hidden states [B*T, E]).  act_kind=None runs the same wiring
    in unquantised fp32 (the model the 8-bit path approximates)."""
    B, T = ids.shape
    E = cfg["hidden"]
    pe = O.pe_table(cfg["max_seq_len"], E)
    x = O.embed_pe(ids, p["embedding.weight"], p["embedding.bias"], pe).reshape(B * T, E)
    mode = O.MASK_CAUSAL if causal else O.MASK_NONE
    for i in range(cfg["layers"]):
        x = block_forward(p, f"block{i}", x, B, T, cfg["heads"], act_kind, w_kind, gelu, mode)
    if return_hidden:
        return x
    return _fc(x, p["final_fc.weight"], p["final_fc.bias"], act_kind, w_kind)


# ---- autoregressive decoding with a key / value cache ---------------------------------------------------------
#
# The step after a prefill, restated with the same per-kernel oracle functions.  Upstream has no cache (its
# Gpt2::forward recomputes the sequence, dnn/models/gpt2.cu:126-142); the semantics are those of its causal
# attention (multi_head_attention.cu:225-301 with the -1e9 mask of its tests, softmax_layer.cu:26-81) on the keys
# that exist.  Quantisation follows the 8-bit path: every tensor that feeds a product is quantised per tensor, so
# the keys / values of a prefill share one scale and every later step has its own; the cache keeps codes and one
# dequantisation factor per position.

def _attend_cached(q, k, v, heads):
    """q [B,E]; k, v [B,n,E] dequantised floats -> [B,E]: softmax(q.k/sqrt(D)) v per head, p = exp(s-max)/(sum+1e-6)."""
    B, E = q.shape
    D = E // heads
    out = np.zeros((B, E), np.float64)
    for b in range(B):
        for h in range(heads):
            sl = slice(h * D, (h + 1) * D)
            s = (k[b, :, sl].astype(np.float64) @ q[b, sl].astype(np.float64)).astype(np.float32) / np.float32(np.sqrt(D))
            p = np.exp(s - s.max()).astype(np.float32)
            p = p / (p.sum(dtype=np.float32) + np.float32(1e-6))
            out[b, sl] = p.astype(np.float64) @ v[b, :, sl].astype(np.float64)
    return out.astype(np.float32)


def decode_reference(p: dict, cfg: dict, ids: np.ndarray, next_ids: list, act_kind: int = O.E4M3, w_kind: int = O.E4M3,
                     gelu: bool = True):
    """Prefill on ids [B,T] (causal), then one decode step per entry of next_ids (each [B]).  Returns the list of
    logits [B,V]: after the prefill (last position) and after every step."""
    B, T = ids.shape
    E, H, L = cfg["hidden"], cfg["heads"], cfg["layers"]
    pe = O.pe_table(cfg["max_seq_len"], E)
    x = O.embed_pe(ids, p["embedding.weight"], p["embedding.bias"], pe).reshape(B * T, E)
    caches = []  # per layer: list of (codes [B, n, 3E], dq) pieces
    for i in range(L):
        t = block_trace(p, f"block{i}", x, B, T, H, act_kind, w_kind, gelu, O.MASK_CAUSAL)
        caches.append([(t["qkv_q"][0].reshape(B, T, 3 * E), float(t["qkv_q"][1][1]))])
        x = t["y"]
    outs = [_fc(x.reshape(B, T, E)[:, -1, :], p["final_fc.weight"], p["final_fc.bias"], act_kind, w_kind)]
    lut = np.array([O.code_value(c, act_kind) for c in range(256)], np.float32)
    pos = T
    for nxt in next_ids:
        idn = np.asarray(nxt, np.int32).reshape(B, 1)
        x = (p["embedding.weight"][idn[:, 0]] + p["embedding.bias"] + pe[pos]).astype(np.float32)
        for i in range(L):
            pre = f"block{i}"
            h1 = O.layernorm(x, p[f"{pre}.ln1.gamma"], p[f"{pre}.ln1.beta"], 1e-5)
            qkv = _fc(h1, p[f"{pre}.qkv.weight"], p[f"{pre}.qkv.bias"], act_kind, w_kind)
            qc, qs = O.quantize(qkv, act_kind)
            caches[i].append((qc.reshape(B, 1, 3 * E), float(qs[1])))
            k = np.concatenate([lut[c[:, :, E:2 * E]] * np.float32(dq) for c, dq in caches[i]], axis=1)
            v = np.concatenate([lut[c[:, :, 2 * E:]] * np.float32(dq) for c, dq in caches[i]], axis=1)
            a = _attend_cached(lut[qc[:, :E]] * qs[1], k, v, H)
            x1 = _fc(a, p[f"{pre}.out.weight"], p[f"{pre}.out.bias"], act_kind, w_kind, residual=x)
            h2 = O.layernorm(x1, p[f"{pre}.ln2.gamma"], p[f"{pre}.ln2.beta"], 1e-5)
            f = _fc(h2, p[f"{pre}.fc1.weight"], p[f"{pre}.fc1.bias"], act_kind, w_kind, gelu=gelu)
            x = _fc(f, p[f"{pre}.fc2.weight"], p[f"{pre}.fc2.bias"], act_kind, w_kind, residual=x1)
        outs.append(_fc(x, p["final_fc.weight"], p["final_fc.bias"], act_kind, w_kind))
        pos += 1
    return outs
