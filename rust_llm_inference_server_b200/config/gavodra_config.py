"""Typed configuration of the Gavodra decoder, read from its `config.json`.

The file lists the layers one by one; every size and every constant that can differ between two
models of the design comes from it:

    {"architecture": "Gavodra", "vocab": V, "width": W, "norm": {"eps": e}, "residual_mult": m,
     "embedding": {"scale": s}, "logit_scale": a, "logit_softcap": c,
     "layers": [{"type": "attention", "mixer": {...}, "mlp": {...} | null}, ...]}

attention mixer: heads, kv_heads, dim, vdim, scale, bias_max, v_mix (the rows of the distance-bias table are
the tensor's; an optional bias_rows says how many the random-weights mode writes).  mlp kind "dense": ff, limit;
kind "moe": expert {ff, limit}, router {experts, top, scale}, shared {ff, limit} or absent.  The
constants that multiply (residual_mult, embedding.scale, logit_scale, router.scale) default to 1 and
logit_softcap to none where the file leaves them out.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .lasapel_config import UNBOUNDED_POSITIONS, _float, _int    # the shared field readers
from .model_config import ConfigError

ARCHITECTURE = "Gavodra"


def _opt_float(d: dict, key: str, where: str, default):
    return default if d.get(key) is None else _float(d, key, where)


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: float
    v_mix: bool
    bias_rows: Optional[int] = None  # rows of the distance-bias table; None: the checkpoint's tensor decides

    @staticmethod
    def from_dict(d: dict, where: str) -> "AttentionMixerConfig":
        heads, kv = _int(d, "heads", where), _int(d, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
        v_mix = d.get("v_mix", False)
        if not isinstance(v_mix, bool):
            raise ConfigError(f"config.json: {where}.v_mix must be true or false, got {v_mix!r}")
        out = AttentionMixerConfig(heads, kv, _int(d, "dim", where), _int(d, "vdim", where), _float(d, "scale", where),
                                   _float(d, "bias_max", where), v_mix,
                                   _int(d, "bias_rows", where, 2) if d.get("bias_rows") is not None else None)
        if not out.bias_max > 1:
            raise ConfigError(f"config.json: {where}.bias_max must exceed 1, got {out.bias_max}")
        return out


@dataclass(frozen=True)
class GluConfig:
    ff: int
    limit: float

    @staticmethod
    def from_dict(d, where: str) -> "GluConfig":
        if not isinstance(d, dict):
            raise ConfigError(f"config.json: {where} must be an object with 'ff' and 'limit'")
        out = GluConfig(_int(d, "ff", where), _float(d, "limit", where))
        if not out.limit > 0:
            raise ConfigError(f"config.json: {where}.limit must be positive, got {out.limit}")
        return out


@dataclass(frozen=True)
class MoeConfig:
    expert: GluConfig
    experts: int
    top: int
    scale: float
    shared: Optional[GluConfig]
    kind: str = "moe"

    @staticmethod
    def from_dict(d: dict, where: str) -> "MoeConfig":
        r = d.get("router")
        if not isinstance(r, dict):
            raise ConfigError(f"config.json: {where}.router must be an object")
        experts, top = _int(r, "experts", where + ".router"), _int(r, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router: top {top} exceeds experts {experts}")
        shared = d.get("shared")
        return MoeConfig(GluConfig.from_dict(d.get("expert"), where + ".expert"), experts, top,
                         _opt_float(r, "scale", where + ".router", 1.0),
                         GluConfig.from_dict(shared, where + ".shared") if shared is not None else None)


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    limit: float
    kind: str = "dense"


@dataclass(frozen=True)
class GavodraLayer:
    type: str
    mixer: AttentionMixerConfig
    mlp: object                      # DenseConfig | MoeConfig | None


@dataclass(frozen=True)
class GavodraConfig:
    architecture = ARCHITECTURE

    vocab: int
    width: int
    eps: float
    residual_mult: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: Optional[float]
    layers: tuple
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    max_positions: int = UNBOUNDED_POSITIONS     # the design has no positional table and no limit of its own

    MIXERS = {"attention": AttentionMixerConfig}

    @classmethod
    def from_dict(cls, d: dict) -> "GavodraConfig":
        vocab, width = _int(d, "vocab", "config"), _int(d, "width", "config")
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _float(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        emb = d.get("embedding") or {}
        if not isinstance(emb, dict):
            raise ConfigError("config.json: 'embedding' must be an object")
        cap = _opt_float(d, "logit_softcap", "config", None)
        if cap is not None and not cap > 0:
            raise ConfigError(f"config.json: logit_softcap must be positive, got {cap}")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} must be an object with 'type' and 'mixer'")
            kind = entry.get("type")
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {sorted(cls.MIXERS)}")
            mixer = cls.MIXERS[kind].from_dict(entry["mixer"], where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None:
                w = where + ".mlp"
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"config.json: {w} must be null or an object of kind 'dense' or 'moe'")
                if mlp["kind"] == "dense":
                    g = GluConfig.from_dict(mlp, w)
                    mlp = DenseConfig(g.ff, g.limit)
                else:
                    mlp = MoeConfig.from_dict(mlp, w)
            layers.append(GavodraLayer(kind, mixer, mlp))
        mixing = [l.mixer for l in layers if l.mixer.v_mix]
        if any((m.kv_heads, m.vdim) != (mixing[0].kv_heads, mixing[0].vdim) for m in mixing):
            raise ConfigError("config.json: layers with v_mix must agree in kv_heads and vdim (they share values)")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else (eos,)))
        return cls(vocab, width, eps, _opt_float(d, "residual_mult", "config", 1.0),
                   _opt_float(emb, "scale", "embedding", 1.0), _opt_float(d, "logit_scale", "config", 1.0), cap,
                   tuple(layers), eos_ids, d.get("bos_token_id"))
