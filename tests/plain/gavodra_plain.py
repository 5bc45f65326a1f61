"""A plain, slow restatement of the Gavodra decoder, one function per mechanism, in float64 on the
CPU.  It shares no code with the package: tests compare the engine's logits with it.

A model is a dict {tensor name: float64 array} plus the dict read from config.json.  Every
function takes whole sequences (all tokens of one request) and loops where the engine has kernels.
"""

from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance-bias table for a key n positions back: one row a distance below half
    the table, then rows spaced evenly in log(distance) up to `far`, the last row for all beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(table, far: float, n_positions: int):
    """bias[i - j, head] for distances 0 .. n_positions - 1."""
    rows = table.shape[0]
    return np.stack([table[distance_bucket(n, rows, far)] for n in range(n_positions)], axis=0)


def clipped_glu(h, w_gate, w_up, w_down, limit):
    """W_down (g sigmoid(1.702 g) (u + 1)) with g = min(W_gate h, limit) and u = W_up h clipped to
    [-limit, limit]."""
    g = np.minimum(h @ w_gate.T, limit)
    u = np.clip(h @ w_up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def route(h, w_router, correction, top: int, scale: float):
    """Chosen experts [tokens, top] and their weights: sigmoid scores; the correction enters the
    choice only; the weights are the chosen scores times `scale`, not renormalised."""
    s = sigmoid(h @ w_router.T)
    choice = s + correction
    idx = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=-1) * scale


def routed_ff(h, W, p, mlp):
    """Mixture of experts with a gated shared expert."""
    r = mlp["router"]
    idx, wts = route(h, W[p + "router"], W[p + "correction"], int(r["top"]), float(r.get("scale", 1.0)))
    limit = float(mlp["expert"]["limit"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(idx[t], wts[t]):
            q = f"{p}e{int(e)}."
            out[t] += wt * clipped_glu(h[t:t + 1], W[q + "gate"], W[q + "up"], W[q + "down"], limit)[0]
    sh = mlp.get("shared")
    if sh:
        q = p + "shared."
        y = clipped_glu(h, W[q + "gate"], W[q + "up"], W[q + "down"], float(sh["limit"]))
        out += sigmoid(h @ W[q + "sg"].T) * y
    return out


def feed_forward(h, W, p, mlp):
    if mlp["kind"] == "dense":
        return clipped_glu(h, W[p + "gate"], W[p + "up"], W[p + "down"], float(mlp["limit"]))
    return routed_ff(h, W, p, mlp)


def attention(h, W, p, m, eps, v_first, is_first):
    """One request's tokens [n, width] through a layer's attention.  Returns the output and the
    values this layer computed before any mixing (what the first mixing layer hands to the others)."""
    n = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[p + "q"].T).reshape(n, H, d)
    k = (h @ W[p + "k"].T).reshape(n, G, d)
    v = (h @ W[p + "v"].T).reshape(n, G, dv)
    own_v = v
    q = rms_norm(q, W[p + "q.norm"], eps)
    k = rms_norm(k, W[p + "k.norm"], eps)
    if m.get("v_mix") and not is_first:
        lam = float(W[p + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    bias = distance_bias(W[p + "rel"], float(m["bias_max"]), n)        # [distance, head]
    gate = sigmoid(h @ W[p + "g"].T)                                   # [n, H]
    out = np.zeros((n, H, dv))
    back = np.arange(n)[:, None] - np.arange(n)[None, :]               # query position - key position
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"]) + bias[np.maximum(back, 0), hd]
        s = np.where(back >= 0, s, -np.inf)                            # causal: a token sees itself and earlier ones
        w = np.exp(s - s.max(axis=-1, keepdims=True))
        w /= w.sum(axis=-1, keepdims=True)
        out[:, hd] = (w @ v[:, g]) * gate[:, hd:hd + 1]
    return out.reshape(n, H * dv) @ W[p + "o"].T, own_v


def forward(W, cfg, tokens, return_layers=False):
    """Logits [n, vocab] of one request's tokens (and the residual stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    m_res = float(cfg.get("residual_mult", 1.0))
    x = W["embed"][np.asarray(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    v_first, seen_mix, layers = None, False, []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mixes = bool(layer["mixer"].get("v_mix"))
        a, own_v = attention(x, W, p + "mix.", layer["mixer"], eps, v_first, is_first=not seen_mix)
        if mixes and not seen_mix:
            v_first, seen_mix = own_v, True
        x = x + m_res * rms_norm(a, W[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            f = feed_forward(x, W, p + "mlp.", layer["mlp"])
            x = x + m_res * rms_norm(f, W[p + "norm2"], eps)
        layers.append(x.copy())
    y = rms_norm(x, W["final.norm"], eps)
    logits = (y @ W["embed"].T) * float(cfg.get("logit_scale", 1.0))
    cap = cfg.get("logit_softcap")
    if cap is not None:
        logits = float(cap) * np.tanh(logits / float(cap))
    return (logits, np.stack(layers)) if return_layers else logits
