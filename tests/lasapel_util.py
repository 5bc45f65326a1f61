"""Small Lasapel configurations and weights for the tests.  The weights are drawn here (not by the
package's random-weights mode) with unit-variance products, so that attention is peaked and the
recurrent state matters: a key that is one position off, a lost state or a missing sink then moves
the logits far beyond rounding."""

from __future__ import annotations

import json
import os

import numpy as np
import torch


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, dims=None, scaling=None, kv_from=None, base=10000.0):
    rot = {"dims": dims or rot_dim, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


SHARED = latent(3, 16, 8, 24, 40, 32, 0.3, scaling=(4.0, 64, 8.0, 2.0))
CONFIGS = {
    # two kinds of mixer in both orders, a layer that reads another's latents, with and without feed-forward
    "X": {"architecture": "Lasapel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "layers": [
        layer("latent_attention", SHARED, 160),
        layer("lightning", {"heads": 2, "dim": 24, "vdim": 40, "decay": [0.9, 0.5]}, 72),
        layer("latent_attention", dict(SHARED, heads=5, dim=8, vdim=16, q_rank=24, kv_from=0)),
        layer("lightning", {"heads": 3, "dim": 16, "vdim": 16, "decay": [0.99, 0.7, 0.95]}),
    ]},
    # one head, no frequency scaling, a rotation over part of the rotated entries, decay 1, rows of the
    # latent cache that are no multiple of a 16-byte vector
    "Y": {"architecture": "Lasapel", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "layers": [
        layer("lightning", {"heads": 1, "dim": 8, "vdim": 48, "decay": [1.0]}, 40),
        layer("latent_attention", latent(1, 12, 4, 20, 10, 10, 0.5, dims=2, base=100.0)),
        layer("latent_attention", latent(4, 8, 12, 8, 16, 20, 0.25, dims=4, scaling=(2.0, 32, 4.0, 1.0)), 64),
    ]},
}
# latent rows that the tensor-core kernels take (multiples of 16 with a value width of 64 or 128): five heads
# (one padded tile of 16) and eighteen (two tiles), a layer that reads another's rows
WIDE = latent(5, 16, 32, 24, 48, 64, 0.2, dims=32, scaling=(16.0, 128, 16.0, 2.0))
CONFIGS["Z"] = {"architecture": "Lasapel", "vocab": 157, "width": 80, "norm": {"eps": 1e-6}, "layers": [
    layer("latent_attention", WIDE, 96),
    layer("latent_attention", latent(18, 8, 16, 8, 32, 128, 0.3, dims=8), 48),
    layer("lightning", {"heads": 2, "dim": 32, "vdim": 24, "decay": [0.97, 0.8]}),
    layer("latent_attention", dict(WIDE, heads=2, dim=40, vdim=16, q_rank=16, kv_from=0), 64),
]}
SEEDS = {"X": 3, "Y": 5, "Z": 8}


def tensor_shapes(cfg: dict) -> dict:
    """Names and shapes, listed here independently of the package."""
    W, out = cfg["width"], {}
    out["embed"] = out["head"] = (cfg["vocab"], W)
    out["final.norm"] = (W,)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        for n in ("norm1", "norm1b", "ls1") + (("norm2", "norm2b", "ls2") if l["mlp"] else ()):
            out[p + n] = (W,)
        if l["type"] == "lightning":
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({p + "mix.q": (hd, W), p + "mix.k": (hd, W), p + "mix.v": (hv, W), p + "mix.g": (hv, W),
                        p + "mix.o": (W, hv), p + "mix.norm": (hv,)})
        else:
            H = m["heads"]
            out.update({p + "mix.dq": (m["q_rank"], W), p + "mix.dq.norm": (m["q_rank"],),
                        p + "mix.uq": (H * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                        p + "mix.uk": (H * m["dim"], m["kv_rank"]), p + "mix.uv": (H * m["vdim"], m["kv_rank"]),
                        p + "mix.sink": (H,), p + "mix.o": (W, H * m["vdim"])})
            if "kv_from" not in m:
                out.update({p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], W), p + "mix.dkv.norm": (m["kv_rank"],)})
        if l["mlp"]:
            ff = l["mlp"]["ff"]
            out.update({p + "mlp.up": (ff, W), p + "mlp.up.b": (ff,), p + "mlp.down": (W, ff), p + "mlp.down.b": (W,)})
    return out


def draw_weights(cfg: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if len(shape) == 2:
            std = 1.0 if name == "embed" else 1.0 / np.sqrt(shape[1])
            x = rng.standard_normal(shape) * std
        elif last in ("ls1", "ls2"):
            x = 0.5 + 0.2 * rng.standard_normal(shape)
        elif name.endswith("dq.norm") or name.endswith("dkv.norm") or name.endswith("mix.norm"):
            x = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "sink":
            x = rng.standard_normal(shape) * 2.0
        else:                       # norms stored around zero, biases
            x = 0.2 * rng.standard_normal(shape)
        out[name] = torch.from_numpy(x.astype(np.float32)).to(torch.bfloat16)
    return out


def make_dir(root: str, which: str, cfg: dict | None = None, seed: int | None = None, edit=None) -> str:
    """Writes config.json and model.safetensors (with the `safetensors` package) once; `edit(weights)`
    may change tensors before they are stored."""
    from safetensors.torch import save_file
    out = os.path.join(root, f"lasapel_{which}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        os.makedirs(out, exist_ok=True)
        cfg = cfg or CONFIGS[which]
        w = draw_weights(cfg, SEEDS.get(which, 0) if seed is None else seed)
        if edit is not None:
            edit(w)
        save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(out, "model.safetensors"))
        with open(os.path.join(out, "config.json"), "w") as f:
            json.dump(cfg, f)
    return out


def plain_weights(model_dir: str) -> dict:
    from safetensors.torch import load_file
    return {k: v.to(torch.float64).numpy() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)
