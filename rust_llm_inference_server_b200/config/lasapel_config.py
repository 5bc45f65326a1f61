"""Typed configuration of the Lasapel decoder, read from its `config.json`.

The file lists the layers one by one; every size and every constant that can differ between two
models of the design comes from it:

    {"architecture": "Lasapel", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "latent_attention" | "lightning", "mixer": {...}, "mlp": {...} | null}, ...]}

latent_attention mixer: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {dims, base, scaling
{factor, original, fast, slow} or absent}, optionally kv_from (the layer whose cached latents it
reads).  lightning mixer: heads, dim, vdim, decay (one factor a head).  mlp: kind "dense", ff.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .model_config import ConfigError

ARCHITECTURE = "Lasapel"
# The design has no positional table and no limit of its own; the engine's limits apply.
UNBOUNDED_POSITIONS = 1 << 30


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if not isinstance(v, int) or isinstance(v, bool) or v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _float(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    factor: Optional[float] = None   # None: no frequency scaling
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0

    @staticmethod
    def from_dict(d, where: str) -> "RotaryConfig":
        if not isinstance(d, dict):
            raise ConfigError(f"config.json: {where} must be an object")
        dims, base = _int(d, "dims", where, 2), _float(d, "base", where)
        if dims % 2 or not base > 1.0:
            raise ConfigError(f"config.json: {where}: dims must be even and base > 1")
        sc = d.get("scaling")
        if sc is None:
            return RotaryConfig(dims, base)
        w = where + ".scaling"
        if not isinstance(sc, dict):
            raise ConfigError(f"config.json: {w} must be an object or null")
        out = RotaryConfig(dims, base, _float(sc, "factor", w), _float(sc, "original", w), _float(sc, "fast", w),
                           _float(sc, "slow", w))
        if not (out.factor > 0 and out.original > 0 and out.fast > 0 and out.slow > 0):
            raise ConfigError(f"config.json: {w}: factor, original, fast and slow must be positive")
        return out


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    kv_from: Optional[int] = None

    @staticmethod
    def from_dict(d: dict, where: str) -> "LatentMixerConfig":
        rot = RotaryConfig.from_dict(d.get("rot"), where + ".rot")
        kv_from = d.get("kv_from")
        if kv_from is not None and (not isinstance(kv_from, int) or isinstance(kv_from, bool) or kv_from < 0):
            raise ConfigError(f"config.json: {where}.kv_from must be a layer index, got {kv_from!r}")
        out = LatentMixerConfig(_int(d, "heads", where), _int(d, "dim", where), _int(d, "rot_dim", where, 2),
                                _int(d, "vdim", where), _int(d, "q_rank", where), _int(d, "kv_rank", where),
                                _float(d, "scale", where), rot, kv_from)
        if rot.dims > out.rot_dim:
            raise ConfigError(f"config.json: {where}: rot.dims {rot.dims} exceeds rot_dim {out.rot_dim}")
        return out


@dataclass(frozen=True)
class LightningMixerConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple

    @staticmethod
    def from_dict(d: dict, where: str) -> "LightningMixerConfig":
        heads = _int(d, "heads", where)
        decay = d.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads or \
                any(isinstance(g, bool) or not isinstance(g, (int, float)) for g in decay):
            raise ConfigError(f"config.json: {where}.decay must list one number per head ({heads})")
        return LightningMixerConfig(heads, _int(d, "dim", where), _int(d, "vdim", where),
                                    tuple(float(g) for g in decay))


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    kind: str = "dense"


@dataclass(frozen=True)
class LasapelLayer:
    type: str                        # "latent_attention" | "lightning"
    mixer: object
    mlp: Optional[DenseMlpConfig]


@dataclass(frozen=True)
class LasapelConfig:
    architecture = ARCHITECTURE

    vocab: int
    width: int
    eps: float
    layers: tuple
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None

    MIXERS = {"latent_attention": LatentMixerConfig, "lightning": LightningMixerConfig}

    @classmethod
    def from_dict(cls, d: dict) -> "LasapelConfig":
        vocab, width = _int(d, "vocab", "config"), _int(d, "width", "config")
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _float(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
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
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp must be null or an object of kind 'dense'")
                mlp = DenseMlpConfig(_int(mlp, "ff", where + ".mlp"))
            layers.append(LasapelLayer(kind, mixer, mlp))
        for i, layer in enumerate(layers):
            src = getattr(layer.mixer, "kv_from", None)
            if src is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            if src >= i or layers[src].type != "latent_attention" or layers[src].mixer.kv_from is not None:
                raise ConfigError(f"config.json: {where} = {src} must name an earlier latent_attention layer "
                                  "that has a key/value projection of its own")
            a, b = layer.mixer, layers[src].mixer
            if (a.kv_rank, a.rot_dim, a.rot) != (b.kv_rank, b.rot_dim, b.rot):
                raise ConfigError(f"config.json: {where}: kv_rank, rot_dim and rot differ from layer {src}'s")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else (eos,)))
        return cls(vocab, width, eps, tuple(layers), eos_ids, d.get("bos_token_id"))
