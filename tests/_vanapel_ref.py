"""Plain, slow numpy statement of the Vanapel design, one function per mechanism.  Test infrastructure only: it shares no
code with the product path (powerserve_b200/), keeps no cache (every call recomputes the whole sequence) and works in
float64.

Notation: n tokens at positions 0 .. n-1; matrices are stored [out, in] and applied as W @ x; d = i - j is the distance
from query i back to key j.

  group norm       G(x; w)  = concat_g( x_g / sqrt(mean(x_g^2) + eps) ) * w        x cut into `groups` equal parts
  layer            x <- x + G(mixer(G(x; w1)); w1b)
                   x <- x + G(ff(G(x; w2)); w2b)                                    (ff absent: the second line is skipped)
  unit rms         U(v) = v / sqrt(mean(v^2) + eps)                                 per head, no weight
  windowed attn    s_hij = U(q_hi) . U(k_g(h)j) * c - r1_h ln(1 + r2_h d)           0 <= d < window,  g(h) = floor(h / (H / G))
                   p_hij = exp(s_hij) / (exp(sink_h) + sum_j' exp(s_hij'))          the sink has no key, no value, no bias
                   v blended: layers marked v_mix use (1 - lam) v + lam v_first, v_first from the first marked layer
  rotation         pair (i, i + D/2), i < D/2, of the first D dims:  (u, v) -> (u cos a - v sin a, v cos a + u sin a) * m,
                   a = position * f_i,  f_i = base^(-2i / D);  YaRN: f_i <- f_i / factor * t_i + f_i (1 - t_i),
                   t_i = clip((i - lo) / max(hi - lo, 0.001), 0, 1),  lo = max(floor(c(fast)), 0),  hi = min(ceil(c(slow)), D - 1),
                   c(r) = D ln(original / (2 pi r)) / (2 ln base),  m = 0.1 ln(factor) + 1
  latent attn      cq = U(W_dq h) * w_dq;  q = W_uq cq, per head [plain dn | rotated dr]
                   W_dkv h = [latent rk | key part dr];  c = U(latent) * w_dkv;  key part rotated, shared by all heads
                   s_hij = (q_plain_hi . (W_uk c_j)_h + rot(q_rot_hi) . rot(kpart_j)) * scale,  j <= i;  values (W_uv c_j)_h; sink as above
  gated ff         g = min(W_g h, L); u = clip(W_u h, -L, L); out = W_d (g sigmoid(1.702 g) (u + 1))
  output           logits = W_head G(x; w_final)
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


def group_norm(x, w, eps, groups):
    n, width = x.shape
    parts = x.reshape(n, groups, width // groups)
    parts = parts / np.sqrt((parts * parts).mean(-1, keepdims=True) + eps)
    return parts.reshape(n, width) * w


def unit_rms(v, eps):
    return v / np.sqrt((v * v).mean(-1, keepdims=True) + eps)


def distance_penalty(r1: float, r2: float, n: int):
    """[n, n] matrix of r1 ln(1 + r2 d) for d >= 0 (0 elsewhere)"""
    d = np.arange(n)[:, None] - np.arange(n)[None, :]
    return r1 * np.log1p(r2 * np.maximum(d, 0).astype(np.float64))


def visible(n: int, window: Optional[int]):
    d = np.arange(n)[:, None] - np.arange(n)[None, :]
    ok = d >= 0
    if window:
        ok &= d < window
    return ok


def sink_softmax(s, ok, sink: float):
    """rows of s over the visible keys, with one more term exp(sink) in the denominator"""
    s = np.where(ok, s, -np.inf)
    top = np.maximum(s.max(-1, keepdims=True), sink)
    e = np.exp(s - top)
    return e / (e.sum(-1, keepdims=True) + np.exp(sink - top))


def windowed_attention(h, w: Dict[str, np.ndarray], m: dict, eps: float, shared: dict):
    """h [n, width] -> [n, width].  `shared` carries the first v_mix layer's values to the later ones."""
    n = h.shape[0]
    H, G, dq, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ w["q"].T).reshape(n, H, dq), eps)
    k = unit_rms((h @ w["k"].T).reshape(n, G, dq), eps)
    v = (h @ w["v"].T).reshape(n, G, dv)
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = float(np.asarray(w["vmix"]).reshape(()))
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    ok = visible(n, (m.get("mask") or {}).get("size"))
    out = np.zeros((n, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"] - distance_penalty(float(w["r1"][hh]), float(w["r2"][hh]), n)
        out[:, hh] = sink_softmax(s, ok, float(w["sink"][hh])) @ v[:, g]
    return out.reshape(n, H * dv) @ w["o"].T


def rotation_frequencies(rot: dict):
    """(f [D/2], magnitude m)"""
    D, base = rot["dims"], rot["base"]
    i = np.arange(D // 2, dtype=np.float64)
    f = base ** (-2.0 * i / D)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def c(r):
        return D * math.log(sc["original"] / (2.0 * math.pi * r)) / (2.0 * math.log(base))

    lo, hi = max(math.floor(c(sc["fast"])), 0), min(math.ceil(c(sc["slow"])), D - 1)
    t = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * t + f * (1.0 - t), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot: dict):
    """x [n, heads, d]: the first rot['dims'] dims of every head are turned, the rest pass"""
    D = rot["dims"]
    f, mag = rotation_frequencies(rot)
    a = np.asarray(positions, np.float64)[:, None] * f[None, :]
    cs, sn = (np.cos(a) * mag)[:, None, :], (np.sin(a) * mag)[:, None, :]
    u, v = x[..., : D // 2], x[..., D // 2: D]
    return np.concatenate([u * cs - v * sn, v * cs + u * sn, x[..., D:]], -1)


def latent_attention(h, w: Dict[str, np.ndarray], m: dict, eps: float):
    n = h.shape[0]
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = unit_rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(n, H, dn + dr)
    t = h @ w["dkv"].T
    c = unit_rms(t[:, :rk], eps) * w["dkv.norm"]
    pos = np.arange(n)
    q_rot = rotate(q[..., dn:], pos, m["rot"])
    k_rot = rotate(t[:, rk:].reshape(n, 1, dr), pos, m["rot"])[:, 0]
    k = (c @ w["uk"].T).reshape(n, H, dn)
    v = (c @ w["uv"].T).reshape(n, H, dv)
    ok = visible(n, (m.get("mask") or {}).get("size"))
    out = np.zeros((n, H, dv))
    for hh in range(H):
        s = (q[:, hh, :dn] @ k[:, hh].T + q_rot[:, hh] @ k_rot.T) * m["scale"]
        out[:, hh] = sink_softmax(s, ok, float(w["sink"][hh])) @ v[:, hh]
    return out.reshape(n, H * dv) @ w["o"].T


def gated_ff(h, w: Dict[str, np.ndarray], mlp: dict):
    L = mlp["limit"]
    g = np.minimum(h @ w["gate"].T, L)
    u = np.clip(h @ w["up"].T, -L, L)
    return (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)) @ w["down"].T


def forward(cfg: dict, tensors: Dict[str, np.ndarray], tokens: List[int], taps: Optional[list] = None):
    """logits [n, vocab] of a whole sequence; `taps` (a list) receives the residual stream after every layer"""
    T = {k: np.asarray(v, np.float64) for k, v in tensors.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    x = T["embed"][np.asarray(tokens)]
    shared: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mw = {k[len(p) + 4:]: v for k, v in T.items() if k.startswith(p + "mix.")}
        h = group_norm(x, T[p + "norm1"], eps, groups)
        if layer["type"] == "attention":
            y = windowed_attention(h, mw, layer["mixer"], eps, shared)
        else:
            assert layer["type"] == "latent_attention"
            y = latent_attention(h, mw, layer["mixer"], eps)
        x = x + group_norm(y, T[p + "norm1b"], eps, groups)
        if layer.get("mlp") is not None:
            fw = {k[len(p) + 4:]: v for k, v in T.items() if k.startswith(p + "mlp.")}
            x = x + group_norm(gated_ff(group_norm(x, T[p + "norm2"], eps, groups), fw, layer["mlp"]), T[p + "norm2b"], eps, groups)
        if taps is not None:
            taps.append(x.copy())
    return group_norm(x, T["final.norm"], eps, groups) @ T["head"].T
