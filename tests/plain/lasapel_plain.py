"""A plain, slow restatement of the Lasapel decoder, one function per mechanism, in float64 on the
CPU.  It shares no code with the package: tests compare the engine's logits with it.

A model is a dict {tensor name: float64 array} plus the dict read from config.json.  Every
function takes whole sequences (all tokens of one request) and loops where the engine has kernels.
"""

from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def zero_centred_norm(x, w, eps):
    """RMS norm whose weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def relu_squared(z):
    return np.square(np.maximum(z, 0.0))


def rotary_table(rot: dict, n_positions: int):
    """cos, sin [positions, dims / 2] of the rotate-half rotation, with the YaRN rule where the
    config gives `scaling`."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = np.arange(half, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def dim_of(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    ang = np.arange(n_positions, dtype=np.float64)[:, None] * f[None, :]
    return np.cos(ang) * mult, np.sin(ang) * mult


def rotate(x, cos, sin, dims):
    """x [T, ..., d]: the first `dims` entries of the last axis are rotated, entry i paired with
    entry i + dims/2; the rest pass unchanged.  cos, sin [T, dims/2]."""
    half = dims // 2
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = cos.reshape(shape), sin.reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def latent_kv(W, p, mx, h, eps):
    """What a latent-attention layer caches: the normed latent c [T, kv_rank] and the rotated
    shared key part [T, rot_dim]."""
    r = int(mx["kv_rank"])
    z = h @ W[p + "dkv"].T
    c = plain_norm(z[:, :r], W[p + "dkv.norm"], eps)
    cos, sin = rotary_table(mx["rot"], h.shape[0])
    kr = rotate(z[:, r:], cos, sin, int(mx["rot"]["dims"]))
    return c, kr


def latent_attention(W, p, mx, h, eps, kv):
    """kv = (c, k_rot) of this layer or of the layer named by `kv_from`."""
    T = h.shape[0]
    H, d, dr, dv = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"])
    c, kr = kv
    cq = plain_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).reshape(T, H, d + dr)
    cos, sin = rotary_table(mx["rot"], T)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], cos, sin, int(mx["rot"]["dims"]))
    k_plain = (c @ W[p + "uk"].T).reshape(T, H, d)
    v = (c @ W[p + "uv"].T).reshape(T, H, dv)
    scale = float(mx["scale"])
    out = np.zeros((T, H, dv))
    sink = W[p + "sink"]
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ kr.T) * scale
        for t in range(T):
            row = s[t, :t + 1]
            m = max(row.max(), sink[hd])
            e = np.exp(row - m)
            out[t, hd] = (e @ v[:t + 1, hd]) / (e.sum() + math.exp(sink[hd] - m))
    return out.reshape(T, H * dv) @ W[p + "o"].T


def lightning(W, p, mx, h, eps):
    T = h.shape[0]
    H, d, dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    q = silu(h @ W[p + "q"].T).reshape(T, H, d)
    k = silu(h @ W[p + "k"].T).reshape(T, H, d)
    v = silu(h @ W[p + "v"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        S = np.zeros((d, dv))
        g = float(mx["decay"][hd])
        for t in range(T):
            S = g * S + np.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    o = plain_norm(out.reshape(T, H * dv), W[p + "norm"], eps) * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def dense_ff(W, p, h):
    return relu_squared(h @ W[p + "up"].T + W[p + "up.b"]) @ W[p + "down"].T + W[p + "down.b"]


def forward(cfg: dict, W: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][np.asarray(tokens, dtype=np.int64)]
    kept = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        h = zero_centred_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            if mx.get("kv_from") is None:
                kept[i] = latent_kv(W, p + "mix.", mx, h, eps)
                kv = kept[i]
            else:
                kv = kept[int(mx["kv_from"])]
            y = latent_attention(W, p + "mix.", mx, h, eps, kv)
        elif layer["type"] == "lightning":
            y = lightning(W, p + "mix.", mx, h, eps)
        else:
            raise ValueError(layer["type"])
        x = x + W[p + "ls1"] * zero_centred_norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = zero_centred_norm(x, W[p + "norm2"], eps)
            y = dense_ff(W, p + "mlp.", h)
            x = x + W[p + "ls2"] * zero_centred_norm(y, W[p + "norm2b"], eps)
        after.append(x.copy())
    logits = zero_centred_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, np.stack(after)) if return_layers else logits
