"""The Lasapel decoder as a description: layers of two kinds of mixer, latent attention (keys and
values as linear maps of a small cached latent, rotary positions with YaRN's frequency blend, a
learned sink in every head's softmax) and lightning attention (a decayed linear recurrence with a
float32 state per request), each in a block that norms a sublayer's result and scales it per
channel before it joins the float32 residual stream; dense feed-forwards with biases and a squared
ReLU.  This file holds no size: everything comes from LasapelConfig and the order of its layers.
"""

from __future__ import annotations

from ..config.lasapel_config import ARCHITECTURE, UNBOUNDED_POSITIONS, LasapelConfig
from ..config.registry import register_architecture
from ..parts.spec import (DenseFFSpec, EmbeddingSpec, LatentAttentionSpec, LayerCall, LayerSpec,
                          LightningAttentionSpec, LMHeadSpec, ModelSpec, RMSNormSpec, YarnRopeSpec)


def _mixer_spec(cfg: LasapelConfig, i: int):
    layer, p, W = cfg.layers[i], f"l{i}.mix.", cfg.width
    m = layer.mixer
    if layer.type == "lightning":
        return LightningAttentionSpec(
            hidden=W, n_heads=m.heads, dim=m.dim, v_dim=m.vdim, decay=tuple(m.decay), eps=cfg.eps,
            q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", gate_proj=p + "g", out_norm=p + "norm", o_proj=p + "o")
    own = m.kv_from is None
    r = m.rot
    return LatentAttentionSpec(
        hidden=W, n_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, v_dim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank,
        scale=m.scale, eps=cfg.eps, q_down=p + "dq", q_norm=p + "dq.norm", q_up=p + "uq",
        kv_down=p + "dkv" if own else None, kv_norm=p + "dkv.norm" if own else None,
        k_up=p + "uk", v_up=p + "uv", o_proj=p + "o", sink=p + "sink",
        position=YarnRopeSpec(r.dims, r.base, r.factor, r.original, r.fast, r.slow))


def describe_lasapel(cfg: LasapelConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda name: RMSNormSpec(W, cfg.eps, name, offset=1.0)      # weights stored around zero
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ff = None
        if layer.mlp is not None:
            ff = DenseFFSpec(W, layer.mlp.ff, p + "mlp.up", p + "mlp.down", p + "mlp.up.b", p + "mlp.down.b", "relu2")
        layers.append(LayerSpec(
            norm1=norm(p + "norm1"), mixer=_mixer_spec(cfg, i), post_norm1=norm(p + "norm1b"), scale1=p + "ls1",
            norm2=norm(p + "norm2") if ff else None, feed_forward=ff,
            post_norm2=norm(p + "norm2b") if ff else None, scale2=p + "ls2" if ff else None,
            arrangement="sandwich"))
        src = getattr(layer.mixer, "kv_from", None)
        # a layer without a key/value projection reads the cache slot of the layer it names
        order.append(LayerCall(i, i) if src is None else LayerCall(i, src, writes_cache=False))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden=W, embedding=EmbeddingSpec(cfg.vocab, W, "embed"), layers=tuple(layers),
        order=tuple(order), final_norm=norm("final.norm"), lm_head=LMHeadSpec(cfg.vocab, W, "head"),
        max_positions=UNBOUNDED_POSITIONS, eos_token_ids=tuple(cfg.eos_token_ids))


def lasapel_tensor_kinds(cfg: LasapelConfig) -> dict:
    """{name: (shape, kind)} of every checkpoint tensor, for the random-weights mode.  Kinds:
    "matrix" N(0, 0.02); "norm" N(1, 0.02); "offset" N(0, 0.1) for weights stored around zero and
    biases; "gain" N(0, 1) for sinks."""
    W = cfg.width
    out = {"embed": ((cfg.vocab, W), "matrix"), "head": ((cfg.vocab, W), "matrix"), "final.norm": ((W,), "offset")}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        out[p + "norm1"] = ((W,), "offset")
        out[p + "norm1b"] = ((W,), "offset")
        out[p + "ls1"] = ((W,), "norm")
        if layer.type == "lightning":
            out[p + "mix.q"] = ((m.heads * m.dim, W), "matrix")
            out[p + "mix.k"] = ((m.heads * m.dim, W), "matrix")
            out[p + "mix.v"] = ((m.heads * m.vdim, W), "matrix")
            out[p + "mix.g"] = ((m.heads * m.vdim, W), "matrix")
            out[p + "mix.o"] = ((W, m.heads * m.vdim), "matrix")
            out[p + "mix.norm"] = ((m.heads * m.vdim,), "norm")
        else:
            out[p + "mix.dq"] = ((m.q_rank, W), "matrix")
            out[p + "mix.dq.norm"] = ((m.q_rank,), "norm")
            out[p + "mix.uq"] = ((m.heads * (m.dim + m.rot_dim), m.q_rank), "matrix")
            if m.kv_from is None:
                out[p + "mix.dkv"] = ((m.kv_rank + m.rot_dim, W), "matrix")
                out[p + "mix.dkv.norm"] = ((m.kv_rank,), "norm")
            out[p + "mix.uk"] = ((m.heads * m.dim, m.kv_rank), "matrix")
            out[p + "mix.uv"] = ((m.heads * m.vdim, m.kv_rank), "matrix")
            out[p + "mix.sink"] = ((m.heads,), "gain")
            out[p + "mix.o"] = ((W, m.heads * m.vdim), "matrix")
        if layer.mlp is not None:
            out[p + "norm2"] = ((W,), "offset")
            out[p + "norm2b"] = ((W,), "offset")
            out[p + "ls2"] = ((W,), "norm")
            out[p + "mlp.up"] = ((layer.mlp.ff, W), "matrix")
            out[p + "mlp.up.b"] = ((layer.mlp.ff,), "offset")
            out[p + "mlp.down"] = ((W, layer.mlp.ff), "matrix")
            out[p + "mlp.down.b"] = ((W,), "offset")
    return out


register_architecture(ARCHITECTURE, LasapelConfig.from_dict, describe_lasapel, lasapel_tensor_kinds)
