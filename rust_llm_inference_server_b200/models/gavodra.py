"""The Gavodra decoder as a description: attention layers without rotation (queries and keys normed per
head, a learned bias by distance, values mixed with those of the first mixing layer, a gate on every
head's output) and gated feed-forwards with clipping, dense or routed to a few of many experts beside a
gated shared one.  Sublayers read the residual stream as it is; only their results are normed before
they join it, times a constant.  The logits come from the embedding table, scaled and capped smoothly.
This file holds no size: everything comes from GavodraConfig and the order of its layers.
"""

from __future__ import annotations

from ..config.gavodra_config import ARCHITECTURE, GavodraConfig
from ..config.registry import register_architecture
from ..parts.spec import (BiasedAttentionSpec, DistanceBiasSpec, EmbeddingSpec, LayerCall, LayerSpec, LMHeadSpec,
                          ModelSpec, RMSNormSpec, RoutedFFSpec, SwiGLUSpec)

# The design fixes the gate's slope and the shift of the linear branch of its feed-forwards.
GLU_SLOPE = 1.702
GLU_UP_SHIFT = 1.0


# rows of a distance-bias table that the random-weights mode writes when the configuration's optional
# mixer key "bias_rows" says nothing (a checkpoint's own tables may have any number of rows)
DEFAULT_BIAS_ROWS = 24


def _glu(W: int, p: str, ff: int, limit: float) -> SwiGLUSpec:
    return SwiGLUSpec(W, ff, p + "gate", p + "up", p + "down", slope=GLU_SLOPE, limit=limit, up_shift=GLU_UP_SHIFT)


def describe_gavodra(cfg: GavodraConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda name: RMSNormSpec(W, cfg.eps, name)
    first_mix = next((i for i, l in enumerate(cfg.layers) if l.mixer.v_mix), None)
    layers, order, unread = [], [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        q = p + "mix."
        mixes = m.v_mix and i != first_mix
        mixer = BiasedAttentionSpec(
            hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, dim=m.dim, v_dim=m.vdim, scale=m.scale, eps=cfg.eps,
            q_proj=q + "q", k_proj=q + "k", v_proj=q + "v", o_proj=q + "o", q_norm=q + "q.norm", k_norm=q + "k.norm",
            bias=DistanceBiasSpec(q + "rel", m.bias_rows, m.bias_max), head_gate=q + "g",
            value_mix=q + "vmix" if mixes else None, value_source=m.v_mix and i == first_mix)
        if not mixes:
            unread.append(q + "vmix")     # a mixing weight that a checkpoint may hold for a layer that mixes nothing
        ff = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            ff = _glu(W, p + "mlp.", layer.mlp.ff, layer.mlp.limit)
        elif layer.mlp is not None:
            x = layer.mlp
            ff = RoutedFFSpec(
                hidden=W, intermediate=x.expert.ff, n_experts=x.experts, top=x.top, router=p + "mlp.router",
                gate_proj=p + "mlp.e{e}.gate", up_proj=p + "mlp.e{e}.up", down_proj=p + "mlp.e{e}.down",
                correction=p + "mlp.correction", route_scale=x.scale, slope=GLU_SLOPE, limit=x.expert.limit,
                up_shift=GLU_UP_SHIFT,
                shared=_glu(W, p + "mlp.shared.", x.shared.ff, x.shared.limit) if x.shared is not None else None,
                shared_gate=p + "mlp.shared.sg" if x.shared is not None else None)
        layers.append(LayerSpec(norm1=norm(p + "norm1"), mixer=mixer, norm2=norm(p + "norm2") if ff else None,
                                feed_forward=ff, arrangement="outnorm", residual_mult=cfg.residual_mult))
        order.append(LayerCall(i, i))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden=W, embedding=EmbeddingSpec(cfg.vocab, W, "embed", scale=cfg.embedding_scale),
        layers=tuple(layers), order=tuple(order), final_norm=norm("final.norm"),
        lm_head=LMHeadSpec(cfg.vocab, W, "embed", logit_scale=cfg.logit_scale, soft_cap=cfg.logit_softcap),
        max_positions=cfg.max_positions, ignorable=tuple(unread), eos_token_ids=tuple(cfg.eos_token_ids))


def gavodra_tensor_kinds(cfg: GavodraConfig) -> dict:
    """{name: (shape, kind)} of every checkpoint tensor, for the random-weights mode.  Kinds: "matrix"
    N(0, 0.02); "norm" N(1, 0.02); "offset" N(0, 0.1) for bias tables, corrections and mixing weights."""
    W = cfg.width
    out = {"embed": ((cfg.vocab, W), "matrix"), "final.norm": ((W,), "norm")}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        out[p + "norm1"] = ((W,), "norm")
        out[p + "mix.q"] = ((m.heads * m.dim, W), "matrix")
        out[p + "mix.k"] = ((m.kv_heads * m.dim, W), "matrix")
        out[p + "mix.v"] = ((m.kv_heads * m.vdim, W), "matrix")
        out[p + "mix.q.norm"] = ((m.dim,), "norm")
        out[p + "mix.k.norm"] = ((m.dim,), "norm")
        out[p + "mix.rel"] = ((m.bias_rows or DEFAULT_BIAS_ROWS, m.heads), "offset")
        out[p + "mix.vmix"] = ((), "offset")
        out[p + "mix.g"] = ((m.heads, W), "matrix")
        out[p + "mix.o"] = ((W, m.heads * m.vdim), "matrix")
        x = layer.mlp
        if x is None:
            continue
        out[p + "norm2"] = ((W,), "norm")
        glu = lambda q, ff: {q + "gate": ((ff, W), "matrix"), q + "up": ((ff, W), "matrix"), q + "down": ((W, ff), "matrix")}
        if x.kind == "dense":
            out.update(glu(p + "mlp.", x.ff))
            continue
        for e in range(x.experts):
            out.update(glu(f"{p}mlp.e{e}.", x.expert.ff))
        out[p + "mlp.router"] = ((x.experts, W), "matrix")
        out[p + "mlp.correction"] = ((x.experts,), "offset")
        if x.shared is not None:
            out.update(glu(p + "mlp.shared.", x.shared.ff))
            out[p + "mlp.shared.sg"] = ((1, W), "matrix")
    return out


register_architecture(ARCHITECTURE, GavodraConfig.from_dict, describe_gavodra, gavodra_tensor_kinds)
