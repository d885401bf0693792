"""Plain statement of the Zazilix family in float64 numpy: one function per mechanism, token loops, no cache, no batching.

It shares nothing with the runtime: the tests build small configurations with random weights, run them through the library
and compare with what these functions give.  Weights arrive as a dict name -> float64 array (the checkpoint's names).

Notation: h is a [T, width] matrix of one sequence's normed inputs, rows are positions 0 .. T-1."""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def logsigmoid(z):
    return -softplus(-z)


# ---------------------------------------------------------------- mixers

# What a test may switch off to show that a mechanism reaches the logits (the design itself has all of them on).
KNOBS = {"sink": True, "penalty": True, "value_norm": True}


def mlstm(h, w, p, mx, eps):
    """Matrix memory with exponential input gate and a running maximum that starts at zero."""
    H, D, Dv, cap = mx["heads"], mx["dim"], mx["vdim"], float(mx["gate_cap"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(T, H, D) / math.sqrt(D)
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, Dv)
    gi = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    gf = logsigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = np.zeros((T, H, Dv))
    for a in range(H):
        S, n, m = np.zeros((D, Dv)), np.zeros(D), 0.0
        for t in range(T):
            m_new = max(gf[t, a] + m, gi[t, a])
            keep, take = math.exp(gf[t, a] + m - m_new), math.exp(gi[t, a] - m_new)
            S = keep * S + take * np.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            m = m_new
            out[t, a] = (S.T @ q[t, a]) / (max(abs(n @ q[t, a]), math.exp(-m)) + 1e-6)
    out = rms(out, eps).reshape(T, H * Dv) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def slopes(H):
    return np.array([2.0 ** (-8.0 * (a + 1) / H) for a in range(H)])


def chunk_attention(h, w, p, mx, eps):
    """Grouped-query attention inside chunks of positions, a distance penalty per head, one added to the softmax denominator."""
    H, G, D, Dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
    size = int((mx.get("mask") or {}).get("size", 0))
    T = h.shape[0]
    q = rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    k = rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    q, k = q.reshape(T, H, D), k.reshape(T, G, D)
    v = (h @ w[p + "v"].T).reshape(T, G, Dv)
    v = rms(v, eps) if KNOBS["value_norm"] else v
    sl = slopes(H) if KNOBS["penalty"] else np.zeros(H)
    out = np.zeros((T, H, Dv))
    for t in range(T):
        first = (t // size) * size if size > 0 else 0
        js = np.arange(first, t + 1)
        for a in range(H):
            g = a // (H // G)
            s = (k[js, g] @ q[t, a]) * mx["scale"] - sl[a] * (t - js)
            top = max(s.max(), 0.0)
            e = np.exp(s - top)
            out[t, a] = (e / ((math.exp(-top) if KNOBS["sink"] else 0.0) + e.sum())) @ v[js, g]
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def hgrn2(h, w, p, mx, eps):
    """Linear attention whose forget gate (bounded below) also says what is written: the key is one minus the gate."""
    H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = silu(h @ w[p + "q"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, Dv)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * sigmoid(h @ w[p + "f"].T + w[p + "f.b"])).reshape(T, H, D)
    out = np.zeros((T, H, Dv))
    for a in range(H):
        S = np.zeros((D, Dv))
        for t in range(T):
            S = f[t, a][:, None] * S + np.outer(1.0 - f[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    out = rms(out, eps) * w[p + "norm"]
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def pair(h, w, p, mx, eps):
    return mx["left_scale"] * chunk_attention(h, w, p + "left.", mx["left"], eps) + mx["right_scale"] * hgrn2(h, w, p + "right.", mx["right"], eps)


def mamba2(h, w, p, mx, eps):
    """Selective state space with a scalar decay per head; inputs pass a short causal convolution first."""
    H, Dv, Ns, G, taps, parts = mx["heads"], mx["vdim"], mx["state"], mx["groups"], mx["conv"], mx["norm_groups"]
    inner, T = H * Dv, h.shape[0]
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * Ns], u[:, 2 * inner + 2 * G * Ns:]
    padded = np.concatenate([np.zeros((taps - 1, xbc.shape[1])), xbc], 0)
    cw = w[p + "conv"]  # [channels, taps], last tap = current token
    conv = sum(padded[j:j + T] * cw[:, j] for j in range(taps)) + w[p + "conv.b"]
    conv = silu(conv)
    x = conv[:, :inner].reshape(T, H, Dv)
    Bm = conv[:, inner:inner + G * Ns].reshape(T, G, Ns)
    Cm = conv[:, inner + G * Ns:].reshape(T, G, Ns)
    dt = softplus(dt + w[p + "dt_bias"])
    A = np.exp(w[p + "A_log"])
    y = np.zeros((T, H, Dv))
    for a in range(H):
        g = a // (H // G)
        S = np.zeros((Ns, Dv))
        for t in range(T):
            S = math.exp(-A[a] * dt[t, a]) * S + dt[t, a] * np.outer(Bm[t, g], x[t, a])
            y[t, a] = S.T @ Cm[t, g] + w[p + "D"][a] * x[t, a]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


MIXERS = {"mlstm": mlstm, "parallel": pair, "mamba2": mamba2}


# ---------------------------------------------------------------- feed-forward

def gated_unit(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


MARGINS = []


def route(h, w, p, ml):
    """-> (chosen [T, top], weights [T, top]); indices >= experts are identity experts."""
    r = ml["router"]
    z = h @ w[p + "router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    pick = s + w[p + "correction"] if (p + "correction") in w else s
    chosen = np.argsort(-pick, axis=-1, kind="stable")[:, :r["top"]]
    if r["top"] < pick.shape[-1]:  # how close each token's closest call was: tests in reduced precision leave coin tosses aside
        ranked = -np.sort(-pick, axis=-1)
        MARGINS.append(ranked[:, r["top"] - 1] - ranked[:, r["top"]])
    return chosen, np.take_along_axis(s, chosen, -1) * r.get("scale", 1.0)


def experts(h, w, p, ml):
    r = ml["router"]
    E = r["experts"]
    chosen, wt = route(h, w, p, ml)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(chosen[t], wt[t]):
            out[t] += c * (h[t] if e >= E else gated_unit(h[t:t + 1], w, p + f"e{e}.")[0])
    if ml.get("shared"):
        out += gated_unit(h, w, p + "shared.")
    return out


# ---------------------------------------------------------------- the model

def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence; layers_out (a list) receives the stream sum after every layer."""
    eps, S = cfg["norm"]["eps"], int(cfg.get("streams", 1))
    T = len(tokens)
    x = w["embed"][tokens] * (cfg.get("embedding") or {}).get("scale", 1.0) + w["pos"][:T]
    xs = [x.copy() for _ in range(S)]

    def sub(xs, hc, g, fn):
        u = sum(w[hc + "in"][s] * xs[s] for s in range(S))
        y = fn(rms(u, eps) * w[g])
        return [sum(w[hc + "mix"][s, t] * xs[s] for s in range(S)) + w[hc + "out"][t] * y for t in range(S)]

    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        xs = sub(xs, p + "hc1.", p + "norm1", lambda hh: MIXERS[lc["type"]](hh, w, p + "mix.", lc["mixer"], eps))
        if lc.get("mlp"):
            xs = sub(xs, p + "hc2.", p + "norm2", lambda hh: experts(hh, w, p + "mlp.", lc["mlp"]))
        if layers_out is not None:
            layers_out.append(sum(xs))
    return (rms(sum(xs), eps) * w["final.norm"]) @ w["head"].T
