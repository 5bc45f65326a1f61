"""Small Gavodra configurations and weights for the tests.  The weights are drawn here (not by the
package's random-weights mode) with unit-variance products and sizeable bias tables, so that attention is
peaked and a key that is one position off, a wrong table row, a missing gate or a value that was not
mixed moves the logits far beyond rounding."""

from __future__ import annotations

import json
import os

import numpy as np
import torch


def attn(heads, kv_heads, dim, vdim, scale, bias_max, v_mix=True):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max,
            "v_mix": v_mix}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, limit, scale, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(mixer, mlp=None):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def model(vocab, width, eps, layers, residual_mult=None, emb_scale=None, logit_scale=None, softcap=None):
    cfg = {"architecture": "Gavodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if residual_mult is not None:
        cfg["residual_mult"] = residual_mult
    if emb_scale is not None:
        cfg["embedding"] = {"scale": emb_scale}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


# rows of the distance-bias tables of each configuration's layers (the checkpoint's shapes say it, not the file)
BIAS_ROWS = {"A": [12, 12, 20, 12], "B": [9, 6, 9], "C": [16, 16, 10], "D": [7, 11], "E": [8, 14]}
CONFIGS = {
    # a layer that does not mix before the first that does, a layer without feed-forward, dense and routed
    # feed-forwards in both orders, with and without a shared expert, limits that differ
    "A": model(211, 96, 1e-5, [
        layer(attn(4, 2, 32, 16, 0.3, 40.0, v_mix=False), dense(72, 1.5)),
        layer(attn(4, 2, 32, 16, 0.2, 40.0), moe(5, 2, 24, 0.8, 1.7, shared=(40, 2.5))),
        layer(attn(6, 2, 16, 16, 0.35, 25.0)),
        layer(attn(2, 2, 48, 16, 0.15, 70.0), moe(4, 3, 40, 3.0, 0.6)),
    ], residual_mult=0.7, emb_scale=3.0, logit_scale=0.8, softcap=9.0),
    # as many key/value heads as query heads, one expert a token, tables with an odd number of rows and a
    # fractional reach, and none of the optional constants (all 1, no cap)
    "B": model(97, 64, 1e-6, [
        layer(attn(3, 3, 16, 48, 0.4, 30.5), moe(3, 1, 16, 1.0, 1.0, shared=(24, 1.0))),
        layer(attn(1, 1, 8, 24, 1.0, 7.0, v_mix=False), dense(40, 0.5)),
        layer(attn(3, 3, 24, 48, 0.25, 30.5)),
    ]),
    # head sizes that the tensor-core kernels take: 64 / 64 with three heads a group, 128 / 32 with one group
    "C": model(157, 128, 1e-5, [
        layer(attn(6, 2, 64, 64, 0.11, 90.0), dense(128, 2.0)),      # a feed-forward the product with the gated epilogue takes
        layer(attn(2, 1, 128, 32, 0.07, 300.0, v_mix=False), moe(6, 2, 32, 1.2, 2.0, shared=(48, 0.9))),
        layer(attn(4, 2, 128, 64, 0.06, 50.0)),
    ], residual_mult=0.5, emb_scale=2.0, logit_scale=0.6, softcap=20.0),
}
# sizes that are multiples of nothing in particular: rows of 100, 24, 20, 36 and 50 elements, seven experts
CONFIGS["D"] = model(131, 100, 1e-5, [
    layer(attn(5, 5, 24, 20, 0.2, 19.0), moe(7, 3, 36, 1.4, 0.9, shared=(50, 1.1))),
    layer(attn(10, 5, 12, 20, 0.3, 45.0), dense(50, 2.2)),
], residual_mult=0.8, emb_scale=1.5, softcap=12.0)
# experts whose products over prompts go to the grouped tcgen05 product (wide tiles of the sort, 256 columns)
CONFIGS["E"] = model(89, 256, 1e-5, [
    layer(attn(4, 2, 64, 64, 0.12, 60.0), moe(4, 2, 128, 1.3, 1.2)),
    layer(attn(2, 2, 128, 64, 0.08, 24.0), moe(3, 1, 256, 0.9, 2.0, shared=(128, 1.5))),
], residual_mult=0.6, emb_scale=2.0, logit_scale=0.7)
SEEDS = {"A": 3, "B": 5, "C": 8, "D": 13, "E": 21}


def tensor_shapes(cfg: dict, bias_rows) -> dict:
    """Names and shapes, listed here independently of the package."""
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "norm1": (W,), p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W),
                    p + "mix.q.norm": (d,), p + "mix.k.norm": (d,), p + "mix.rel": (bias_rows[i], H),
                    p + "mix.vmix": (), p + "mix.g": (H, W), p + "mix.o": (W, H * dv)})
        x = l["mlp"]
        if x is None:
            continue
        out[p + "norm2"] = (W,)

        def glu(q, ff):
            return {q + "gate": (ff, W), q + "up": (ff, W), q + "down": (W, ff)}
        if x["kind"] == "dense":
            out.update(glu(p + "mlp.", x["ff"]))
            continue
        for e in range(x["router"]["experts"]):
            out.update(glu(f"{p}mlp.e{e}.", x["expert"]["ff"]))
        out.update({p + "mlp.router": (x["router"]["experts"], W), p + "mlp.correction": (x["router"]["experts"],)})
        if "shared" in x:
            out.update(glu(p + "mlp.shared.", x["shared"]["ff"]))
            out[p + "mlp.shared.sg"] = (1, W)
    return out


def draw_weights(cfg: dict, seed: int, bias_rows) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, bias_rows).items():
        last = name.split(".")[-1]
        if last == "rel":
            x = rng.standard_normal(shape) * 1.5
        elif last == "vmix":
            x = np.asarray(rng.uniform(0.25, 0.75))
        elif last == "correction":
            x = rng.standard_normal(shape) * 0.3
        elif last in ("router", "sg"):
            x = rng.standard_normal(shape) * 2.0 / np.sqrt(shape[1])
        elif len(shape) == 2:
            std = (1.5 if name == "embed" else 1.0) / np.sqrt(shape[1])
            # queries and keys are normed, so their size is the norm weights'; gate, up and down see unit inputs
            x = rng.standard_normal(shape) * std
        elif last == "norm" and ("q.norm" in name or "k.norm" in name):
            x = 1.0 + 0.3 * rng.standard_normal(shape)
        else:
            x = 1.0 + 0.2 * rng.standard_normal(shape)
        out[name] = torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16)
    return out


def settle_routing(w: dict) -> None:
    """Corrections so far apart (more than a score's whole range) that the choice of experts no longer hangs
    on the scores: a choice that flips under bfloat16 rounding would move a token's logits as much as a fault
    does, and some tokens' scores always lie close.  The weights of the chosen experts still follow the
    scores.  The bfloat16 runs of whole models use such weights; the float32 runs, and the routing kernel's
    own test in both types, choose by the scores."""
    for name in [n for n in w if n.endswith(".correction")]:
        n = w[name].shape[0]
        order = np.random.default_rng(n + len(name)).permutation(n)
        w[name] = torch.from_numpy((order * 1.5).astype(np.float32)).to(torch.bfloat16)


def make_dir(root: str, which: str, cfg: dict | None = None, seed: int | None = None, bias_rows=None, edit=None) -> str:
    """Writes config.json and model.safetensors (with the `safetensors` package) once; `edit(weights)`
    may change tensors before they are stored."""
    from safetensors.torch import save_file
    out = os.path.join(root, f"gavodra_{which}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        os.makedirs(out, exist_ok=True)
        cfg = cfg or CONFIGS[which]
        rows = bias_rows or BIAS_ROWS.get(which) or [10] * len(cfg["layers"])
        w = draw_weights(cfg, SEEDS.get(which, 0) if seed is None else seed, rows)
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
