"""Plain float64 statement of the Sopepel design, one function per mechanism, token loops and no cache: the slow oracle the
runtime is compared with.  It shares no code with calm_b200 (numpy only; tensors come in as float64 arrays).

Notation: x [T, width] is one sequence's residual stream; a sublayer reads x itself and its output y comes back through
an RMS norm, x <- x + norm(y).  p is the position of a token (0 for the first)."""
from __future__ import annotations

import math
from typing import Dict, List

import numpy as np

# mechanisms a test can leave out to show that the comparison would notice
KNOBS = {"weight_on_input": True, "shared_gate": True, "bigram": True, "norm_per_head": True, "gate_per_head": True}
# router margins of the last forward(): per routed layer, per token, the gap between the last chosen score and the best one left out
MARGINS: List[np.ndarray] = []


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def embed(t: Dict[str, np.ndarray], bg: dict, toks: List[int]) -> np.ndarray:
    """token row + a row of the bigram table picked by a hash of (previous token, token); the first token takes the last row"""
    B = int(bg["buckets"])
    out = []
    for i, tok in enumerate(toks):
        row = B if i == 0 else (toks[i - 1] * int(bg["mul_prev"]) + tok * int(bg["mul_cur"])) % B
        out.append(t["embed"][tok] + (t["bigram"][row] if KNOBS["bigram"] else 0.0))
    return np.stack(out)


def rotate(v: np.ndarray, rot: dict | None) -> np.ndarray:
    """v [T, heads, dim]: the first rot.dims channels of a head turn by the position, channel i paired with channel i + dims/2"""
    if not rot or int(rot.get("dims", 0)) < 2:
        return v
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    out = v.copy()
    for p in range(v.shape[0]):
        for i in range(half):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, w = v[p, :, i], v[p, :, i + half]
            out[p, :, i], out[p, :, i + half] = u * c - w * s, w * c + u * s
    return out


def sees(i: int, j: int, size: int) -> bool:
    """query position i sees key position j: causal, and (with a block size) inside the same block counted from position 0"""
    return j <= i and (size <= 0 or i // size == j // size)


def left_attention(t, m: str, mx: dict, h: np.ndarray, eps: float) -> np.ndarray:
    H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    G = int(mx.get("kv_heads", H))
    T = h.shape[0]
    q = (h @ t[m + "q"].T + t[m + "q.b"]).reshape(T, H, D)
    k = (h @ t[m + "k"].T + t[m + "k.b"]).reshape(T, G, D)
    v = (h @ t[m + "v"].T + t[m + "v.b"]).reshape(T, G, Dv)
    if KNOBS["norm_per_head"]:
        q, k = rms_norm(q, t[m + "q.norm"], eps), rms_norm(k, t[m + "k.norm"], eps)
    else:  # (a wrong reading: one norm over all heads)
        q = rms_norm(q.reshape(T, -1), np.tile(t[m + "q.norm"], H), eps).reshape(T, H, D)
        k = rms_norm(k.reshape(T, -1), np.tile(t[m + "k.norm"], G), eps).reshape(T, G, D)
    q, k = rotate(q, mx.get("rot")), rotate(k, mx.get("rot"))
    size = int((mx.get("mask") or {}).get("size", 0))
    gate = sigmoid(h @ t[m + "g"].T) if KNOBS["gate_per_head"] else np.ones((T, H))  # [T, H]
    out = np.zeros((T, H, Dv))
    for i in range(T):
        js = [j for j in range(i + 1) if sees(i, j, size)]
        for hh in range(H):
            g = hh // (H // G)
            sc = np.array([q[i, hh] @ k[j, g] for j in js]) * float(mx["scale"])
            w = np.exp(sc - sc.max())
            w /= w.sum()
            out[i, hh] = gate[i, hh] * sum(wj * v[j, g] for wj, j in zip(w, js))
    return out.reshape(T, H * Dv) @ t[m + "o"].T + t[m + "o.b"]


def right_linear(t, m: str, mx: dict, h: np.ndarray, eps: float) -> np.ndarray:
    """gated linear attention: per head S <- diag(alpha) S + k v^T, o = S^T q, with one decay per key channel"""
    H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    T = h.shape[0]
    q = (h @ t[m + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ t[m + "k"].T).reshape(T, H, D)
    v = (h @ t[m + "v"].T).reshape(T, H, Dv)
    z = (h @ t[m + "a1"].T) @ t[m + "a2"].T + t[m + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / float(mx["tau"]))).reshape(T, H, D)
    S = np.zeros((H, D, Dv))
    o = np.zeros((T, H, Dv))
    for i in range(T):
        S = alpha[i][:, :, None] * S + k[i][:, :, None] * v[i][:, None, :]
        o[i] = np.einsum("hdv,hd->hv", S, q[i])
    o = rms_norm(o, t[m + "norm"], eps).reshape(T, H * Dv)
    return (o * silu(h @ t[m + "g"].T)) @ t[m + "o"].T


def mixer(t, p: str, mx: dict, h: np.ndarray, eps: float) -> np.ndarray:
    return float(mx.get("left_scale", 1.0)) * left_attention(t, p + "mix.left.", mx["left"], h, eps) + \
        float(mx.get("right_scale", 1.0)) * right_linear(t, p + "mix.right.", mx["right"], h, eps)


def dense_unit(t, f: str, h: np.ndarray) -> np.ndarray:
    return (gelu_tanh(h @ t[f + "gate"].T) * (h @ t[f + "up"].T)) @ t[f + "down"].T


def small_unit(t, f: str, h: np.ndarray) -> np.ndarray:
    """an expert (and the shared unit): down(relu(up h)^2), no biases"""
    return np.maximum(h @ t[f + "up"].T, 0.0) ** 2 @ t[f + "down"].T


def route(z: np.ndarray, top: int):
    """per token: the `top` experts with the largest sigmoid scores (lowest index wins a tie), weights = those scores"""
    s = sigmoid(z)
    full = np.argsort(-s, axis=-1, kind="stable")
    order = full[:, :top]
    if top < s.shape[-1]:
        MARGINS.append(np.take_along_axis(s, full[:, top - 1:top], -1)[:, 0] - np.take_along_axis(s, full[:, top:top + 1], -1)[:, 0])
    return order, np.take_along_axis(s, order, -1)


def experts(t, f: str, ml: dict, h: np.ndarray) -> np.ndarray:
    E, top = int(ml["router"]["experts"]), int(ml["router"]["top"])
    sel, wt = route(h @ t[f + "router"].T, top)
    out = np.zeros_like(h)
    for n in range(h.shape[0]):
        for e, w in zip(sel[n], wt[n]):
            if KNOBS["weight_on_input"]:
                out[n] += small_unit(t, f + f"e{e}.", (w * h[n])[None])[0]  # the weight multiplies the expert's input
            else:
                out[n] += w * small_unit(t, f + f"e{e}.", h[n][None])[0]
    if ml.get("shared"):
        out += (sigmoid(h @ t[f + "shared.sg"].T) if KNOBS["shared_gate"] else 1.0) * small_unit(t, f + "shared.", h)
    assert E == t[f + "router"].shape[0]
    return out


def forward(cfg: dict, t: Dict[str, np.ndarray], toks: List[int], layers_out: list | None = None) -> np.ndarray:
    """logits [T, vocab] of one sequence"""
    eps = float(cfg["norm"]["eps"])
    x = embed(t, cfg["embedding"]["bigram"], toks)
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + rms_norm(mixer(t, p, lc["mixer"], x, eps), t[p + "norm1"], eps)
        ml = lc.get("mlp")
        if ml:
            y = dense_unit(t, p + "mlp.", x) if ml["kind"] == "dense" else experts(t, p + "mlp.", ml, x)
            x = x + rms_norm(y, t[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, t["final.norm"], eps) @ t["embed"].T * float(cfg.get("logit_scale", 1.0))
