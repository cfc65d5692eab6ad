"""Plain, slow numpy statement of the Nufusun design, one function per mechanism.  Test infrastructure only: it shares
no code with the product path (powerserve_b200/), keeps no cache (every call recomputes the whole sequence) and works in
float64 unless told otherwise.

Notation: a sequence of n tokens has positions 0 .. n-1; W is stored [out, in] and applied as W @ x.

  embedding        x_t = E[token_t] * s_e
  unit-offset norm N(x; w) = x / sqrt(mean(x^2) + eps) * (1 + w)
  layer            h = N(x; w1);  x <- x + (mixer(h) + ff(h))          (ff absent: x <- x + mixer(h))
  biased attention a_hij = (q_hi . k_g(h)j) * c * tau_h + R[beta(i - j), h]      g(h) = floor(h / (H / G)), j <= i
                   b_hij = sum_g T[h, g] a_gij                                    (heads mixed before the soft-max)
                   p_hij = exp(b_hij) / (1 + sum_j' exp(b_hij'))                  (a sink of score 0 without a value)
                   o_hi  = sum_j p_hij v_g(h)j ;  out = W_o concat_h(o_hi) + b_o
  distance bucket  beta(n) = n                                                          for n < floor(B / 2)
                           = min(B - 1, B2 + floor(ln(n / B2) / ln(D / B2) * (B - B2)))  otherwise, B2 = floor(B / 2)
  expert           g = min(W_g z, L); u = clip(W_u z, -L, L); y = g * sigmoid(1.702 g) * (u + 1); out = W_d y
  routed ff        s = sigmoid(W_r h); the `top` largest s choose the experts; ff(h) = sum_e expert_e(s_e * h)
  output           logits = W_head N(x; w_final)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np


def bf16_round(a: np.ndarray) -> np.ndarray:
    """round-to-nearest-even of float32 values to bfloat16, returned as float32"""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def embed(table, tokens, scale, dt=np.float64):
    return table[np.asarray(tokens)].astype(dt) * dt(scale)


def unit_offset_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * (1.0 + w)


def distance_bucket(n: int, n_rows: int, d_max: float) -> int:
    half = n_rows // 2
    if n < half:
        return n
    r = np.float32(np.log(np.float32(n) / np.float32(half))) / np.float32(math.log(d_max / half)) * np.float32(n_rows - half)
    return min(n_rows - 1, half + int(math.floor(float(r))))


def biased_attention(h, w: Dict[str, np.ndarray], m: dict):
    """h [n, width] -> [n, width]; the whole sequence at once, causal"""
    n = h.shape[0]
    H, G, dq, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T + w["q.b"]).reshape(n, H, dq)
    k = (h @ w["k"].T + w["k.b"]).reshape(n, G, dq)
    v = (h @ w["v"].T + w["v.b"]).reshape(n, G, dv)
    rep = H // G
    rel, B = w["rel"], w["rel"].shape[0]
    a = np.zeros((H, n, n), h.dtype)
    for hh in range(H):
        a[hh] = (q[:, hh] @ k[:, hh // rep].T) * m["scale"] * w["temp"][hh]
    bucket = np.array([distance_bucket(d, B, m["bias_max"]) for d in range(n)])
    idx = np.arange(n)[:, None] - np.arange(n)[None, :]
    causal = idx >= 0
    bias = rel[bucket[np.where(causal, idx, 0)]]            # [n, n, H]
    a = a + np.transpose(bias, (2, 0, 1))
    b = np.einsum("hg,gij->hij", w["talk"], a)
    out = np.zeros((n, H, dv), h.dtype)
    for hh in range(H):
        for i in range(n):
            s = b[hh, i, : i + 1]
            mx = max(float(s.max()), 0.0)
            e = np.exp(s - mx)
            p = e / (math.exp(-mx) + e.sum())
            out[i, hh] = p @ v[: i + 1, hh // rep]
    return out.reshape(n, H * dv) @ w["o"].T + w["o.b"]


def expert(z, gate, up, down, limit):
    g = np.minimum(z @ gate.T, limit)
    u = np.clip(z @ up.T, -limit, limit)
    y = g * (1.0 / (1.0 + np.exp(-1.702 * g))) * (u + 1.0)
    return y @ down.T


def routed_ff(h, w: Dict[str, np.ndarray], mlp: dict):
    E, top, limit = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["limit"]
    s = 1.0 / (1.0 + np.exp(-(h @ w["router"].T)))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-s[t, e], e))[:top]
        for e in order:
            out[t] += expert(s[t, e] * h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)
    return out


def forward(cfg: dict, tensors: Dict[str, np.ndarray], tokens: List[int], dt=np.float64, taps: Optional[list] = None):
    """logits [n, vocab] of a whole sequence; `taps` (a list) receives the residual stream after every layer"""
    T = {k: v.astype(dt) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = embed(T["embed"], tokens, cfg["embedding"]["scale"], dt)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = unit_offset_norm(x, T[p + "norm1"], eps)
        assert layer["type"] == "attention"
        mw = {k[len(p) + 4:]: v for k, v in T.items() if k.startswith(p + "mix.")}
        y = biased_attention(h, mw, layer["mixer"])
        if layer.get("mlp") is not None:
            fw = {k[len(p) + 4:]: v for k, v in T.items() if k.startswith(p + "mlp.")}
            y = y + routed_ff(h, fw, layer["mlp"])
        x = x + y
        if taps is not None:
            taps.append(x.copy())
    return unit_offset_norm(x, T["final.norm"], eps) @ T["head"].T
