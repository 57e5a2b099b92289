"""Typed configuration of the Lalepel design.

config.json of this design is nested: the model's ``width``, ``vocab`` and ``norm.eps``, and a list
``layers`` whose entries each give the ``type`` of their mixer, the mixer's sizes and constants
(``mixer``) and their feed-forward (``mlp``, or null for none).  Layers may differ from each other in
everything.  Every size and constant is read here; nothing about a particular model is fixed in code.

Mixer ``latent_attention``: ``heads``, ``dim`` (unrotated query/key size per head), ``rot_dim`` (rotated
size), ``vdim``, ``q_rank``, ``kv_rank``, ``scale`` (the score's factor, used as given), ``mask.size`` (the
sliding window; absent = every earlier token), ``rot`` = {``base``, ``dims``, ``scaling`` = {``factor``,
``original``, ``fast``, ``slow``} or absent}.

Mixer ``retention``: ``heads``, ``dim``, ``vdim``, ``decay`` (one number per head).

Feed-forward ``dense``: ``ff``.  ``moe``: ``router.experts``, ``router.top``, ``expert.ff``, and
``shared.ff`` when there is a shared expert.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, take


def _sub(raw: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = raw.get(key)
    if v is None:
        if optional:
            return None
        raise ConfigError(f"config.json: missing key: {where}{key}")
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key} must be an object, got {v!r}")
    return v


def _pos(raw, key, where) -> int:
    try:
        v = take(raw, key, int)
    except ConfigError as e:
        raise ConfigError(str(e).replace(key, where + key, 1)) from None
    if v <= 0:
        raise ConfigError(f"config.json: {where}{key} must be positive, got {v}")
    return v


def _num(raw, key, where) -> float:
    try:
        return take(raw, key, float)
    except ConfigError as e:
        raise ConfigError(str(e).replace(key, where + key, 1)) from None


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int                      # 0: every earlier token
    rot_base: float
    rot_dims: int                    # 0: no rotation
    rot_scaling: Optional[RotaryScaling]

    kind = "latent_attention"


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    kind = "retention"


@dataclass(frozen=True)
class DenseFfConfig:
    ff: int

    kind = "dense"


@dataclass(frozen=True)
class MoeFfConfig:
    experts: int
    top: int
    expert_ff: int
    shared_ff: int                   # 0: no shared expert

    kind = "moe"


@dataclass(frozen=True)
class LalepelLayer:
    mixer: Any                       # LatentAttentionConfig | RetentionConfig
    mlp: Any                         # DenseFfConfig | MoeFfConfig | None


def _latent(m: Dict[str, Any], where: str) -> LatentAttentionConfig:
    mask = _sub(m, "mask", where, optional=True)
    window = _pos(mask, "size", where + "mask.") if mask is not None else 0
    rot = _sub(m, "rot", where, optional=True)
    rot_dim = take(m, "rot_dim", int, 0)
    base, dims, scaling = 10000.0, 0, None
    if rot is not None:
        base = _num(rot, "base", where + "rot.")
        dims = _pos(rot, "dims", where + "rot.")
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most rot_dim {rot_dim}")
        if base <= 1.0:
            raise ConfigError(f"config.json: {where}rot.base must exceed 1, got {base}")
        sc = _sub(rot, "scaling", where + "rot.", optional=True)
        if sc is not None:
            scaling = RotaryScaling(*(_num(sc, k, where + "rot.scaling.") for k in ("factor", "original", "fast", "slow")))
            if scaling.factor <= 0 or scaling.original <= 0 or scaling.fast <= 0 or scaling.slow <= 0:
                raise ConfigError(f"config.json: {where}rot.scaling: every number must be positive")
    if rot_dim < 0:
        raise ConfigError(f"config.json: {where}rot_dim must not be negative")
    return LatentAttentionConfig(
        heads=_pos(m, "heads", where), dim=_pos(m, "dim", where), rot_dim=rot_dim, vdim=_pos(m, "vdim", where),
        q_rank=_pos(m, "q_rank", where), kv_rank=_pos(m, "kv_rank", where), scale=_num(m, "scale", where),
        window=window, rot_base=base, rot_dims=dims, rot_scaling=scaling)


def _retention(m: Dict[str, Any], where: str) -> RetentionConfig:
    heads = _pos(m, "heads", where)
    decay = take(m, "decay", list)
    if len(decay) != heads or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
        raise ConfigError(f"config.json: {where}decay must list one number per head ({heads})")
    return RetentionConfig(heads=heads, dim=_pos(m, "dim", where), vdim=_pos(m, "vdim", where),
                           decay=tuple(float(x) for x in decay))


def _mlp(raw: Optional[Dict[str, Any]], where: str):
    if raw is None:
        return None
    kind = raw.get("kind")
    if kind == "dense":
        return DenseFfConfig(ff=_pos(raw, "ff", where))
    if kind == "moe":
        router = _sub(raw, "router", where)
        expert = _sub(raw, "expert", where)
        shared = _sub(raw, "shared", where, optional=True)
        experts, top = _pos(router, "experts", where + "router."), _pos(router, "top", where + "router.")
        if top > experts:
            raise ConfigError(f"config.json: {where}router.top {top} exceeds the {experts} experts")
        return MoeFfConfig(experts=experts, top=top, expert_ff=_pos(expert, "ff", where + "expert."),
                           shared_ff=_pos(shared, "ff", where + "shared.") if shared is not None else 0)
    raise ConfigError(f"config.json: {where}kind must be 'dense' or 'moe', got {kind!r}")


@dataclass(frozen=True)
class LalepelConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[LalepelLayer, ...]

    architecture = "Lalepel"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "LalepelConfig":
        norm = _sub(raw, "norm", "")
        layers_raw = take(raw, "layers", list)
        if not layers_raw:
            raise ConfigError("config.json: layers must not be empty")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(lr, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = lr.get("type")
            mixer = _sub(lr, "mixer", where)
            if kind == "latent_attention":
                mx = _latent(mixer, where + "mixer.")
            elif kind == "retention":
                mx = _retention(mixer, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type must be 'latent_attention' or 'retention', got {kind!r}")
            mlp = lr.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            layers.append(LalepelLayer(mixer=mx, mlp=_mlp(mlp, where + "mlp.")))
        return cls(vocab=_pos(raw, "vocab", ""), width=_pos(raw, "width", ""), eps=_num(norm, "eps", "norm."),
                   layers=tuple(layers))
