"""Typed configuration of the Pozozen design.

config.json of this design is nested: the model's ``width``, ``vocab``, ``norm.eps``, ``residual_mult`` (a factor on
every sublayer's output), ``streams`` (copies of the residual stream; absent: one, and no stream tensors), ``loop`` =
{``start``, ``stop``, ``times``} (layers start .. stop - 1 run ``times`` times in a row; absent: every layer once) and a
list ``layers`` whose entries each give the ``type`` of their mixer, the mixer's sizes and constants (``mixer``) and
their feed-forward (``mlp``, or null for none).  Layers may differ from each other in everything.  Every size and
constant is read here; nothing about a particular model is fixed in code.

Mixer ``mlstm``: ``heads``, ``dim``, ``vdim``, ``gate_cap``.
Mixer ``parallel``: ``left`` = {``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (the sliding window;
absent = every earlier token)}, ``right`` = {``heads``, ``vdim``, ``state``, ``groups``, ``conv``, ``norm_groups``},
``left_scale``, ``right_scale``.
Feed-forward ``moe``: ``router.experts``, ``router.top``, ``router.identity`` (absent: 0), ``router.groups`` = {``count``,
``keep``} (absent: one group), ``expert.ff``, and ``shared.ff`` when there is a shared expert.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, take
from .lalepel import _num, _pos, _sub


@dataclass(frozen=True)
class MLstmConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    kind = "mlstm"


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                      # 0: every earlier token


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class ParallelConfig:
    left: WindowAttentionConfig
    right: StateSpaceConfig
    left_scale: float
    right_scale: float

    kind = "parallel"


@dataclass(frozen=True)
class RoutedFfConfig:
    experts: int
    identity: int
    top: int
    group_count: int
    group_keep: int
    expert_ff: int
    shared_ff: int                   # 0: no shared expert

    kind = "moe"


@dataclass(frozen=True)
class PozozenLayer:
    mixer: Any                       # MLstmConfig | ParallelConfig
    mlp: Optional[RoutedFfConfig]


def _mlstm(m: Dict[str, Any], where: str) -> MLstmConfig:
    cap = _num(m, "gate_cap", where)
    if not cap > 0:
        raise ConfigError(f"config.json: {where}gate_cap must be positive, got {cap}")
    return MLstmConfig(heads=_pos(m, "heads", where), dim=_pos(m, "dim", where), vdim=_pos(m, "vdim", where), gate_cap=cap)


def _parallel(m: Dict[str, Any], where: str) -> ParallelConfig:
    lw, rw = where + "left.", where + "right."
    l, r = _sub(m, "left", where), _sub(m, "right", where)
    mask = _sub(l, "mask", lw, optional=True)
    left = WindowAttentionConfig(heads=_pos(l, "heads", lw), kv_heads=_pos(l, "kv_heads", lw), dim=_pos(l, "dim", lw),
                                 vdim=_pos(l, "vdim", lw), scale=_num(l, "scale", lw),
                                 window=_pos(mask, "size", lw + "mask.") if mask is not None else 0)
    if left.heads % left.kv_heads:
        raise ConfigError(f"config.json: {lw}heads {left.heads} must be a multiple of kv_heads {left.kv_heads}")
    right = StateSpaceConfig(heads=_pos(r, "heads", rw), vdim=_pos(r, "vdim", rw), state=_pos(r, "state", rw),
                             groups=_pos(r, "groups", rw), conv=_pos(r, "conv", rw), norm_groups=_pos(r, "norm_groups", rw))
    if right.heads % right.groups:
        raise ConfigError(f"config.json: {rw}heads {right.heads} must be a multiple of groups {right.groups}")
    if (right.heads * right.vdim) % right.norm_groups:
        raise ConfigError(f"config.json: {rw}norm_groups {right.norm_groups} must divide heads * vdim")
    return ParallelConfig(left=left, right=right, left_scale=_num(m, "left_scale", where), right_scale=_num(m, "right_scale", where))


def _mlp(raw: Optional[Dict[str, Any]], where: str) -> Optional[RoutedFfConfig]:
    if raw is None:
        return None
    if raw.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}kind must be 'moe', got {raw.get('kind')!r}")
    router, expert = _sub(raw, "router", where), _sub(raw, "expert", where)
    shared = _sub(raw, "shared", where, optional=True)
    rw = where + "router."
    experts, top = _pos(router, "experts", rw), _pos(router, "top", rw)
    identity = take(router, "identity", int, 0)
    if identity < 0:
        raise ConfigError(f"config.json: {rw}identity must not be negative")
    if top > experts + identity:
        raise ConfigError(f"config.json: {rw}top {top} exceeds the {experts + identity} router outputs")
    groups = _sub(router, "groups", rw, optional=True)
    count = _pos(groups, "count", rw + "groups.") if groups is not None else 1
    keep = _pos(groups, "keep", rw + "groups.") if groups is not None else 1
    if (experts + identity) % count or keep > count:
        raise ConfigError(f"config.json: {rw}groups: {count} groups (keep {keep}) do not fit {experts + identity} router outputs")
    if keep * ((experts + identity) // count) < top:
        raise ConfigError(f"config.json: {rw}groups: the {keep} groups kept hold fewer than top {top} experts")
    return RoutedFfConfig(experts=experts, identity=identity, top=top, group_count=count, group_keep=keep,
                          expert_ff=_pos(expert, "ff", where + "expert."),
                          shared_ff=_pos(shared, "ff", where + "shared.") if shared is not None else 0)


@dataclass(frozen=True)
class PozozenConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    streams: int                     # 0: one residual stream, no stream tensors
    loop: Optional[Tuple[int, int, int]]   # (start, stop, times)
    layers: Tuple[PozozenLayer, ...]

    architecture = "Pozozen"

    def run_order(self) -> Tuple[int, ...]:
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        a, b, times = self.loop
        return tuple(range(a)) + tuple(range(a, b)) * times + tuple(range(b, n))

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PozozenConfig":
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
            if kind == "mlstm":
                mx = _mlstm(mixer, where + "mixer.")
            elif kind == "parallel":
                mx = _parallel(mixer, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type must be 'mlstm' or 'parallel', got {kind!r}")
            mlp = lr.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            layers.append(PozozenLayer(mixer=mx, mlp=_mlp(mlp, where + "mlp.")))
        loop = _sub(raw, "loop", "", optional=True)
        lp = None
        if loop is not None:
            a, b, times = take(loop, "start", int), take(loop, "stop", int), _pos(loop, "times", "loop.")
            if not (0 <= a <= b <= len(layers)):
                raise ConfigError(f"config.json: loop: start {a} and stop {b} must lie within the {len(layers)} layers, in order")
            lp = (a, b, times)
        streams = take(raw, "streams", int, 0)
        if streams < 0:
            raise ConfigError("config.json: streams must not be negative")
        return cls(vocab=_pos(raw, "vocab", ""), width=_pos(raw, "width", ""), eps=_num(norm, "eps", "norm."),
                   residual_mult=take(raw, "residual_mult", float, 1.0), streams=streams, loop=lp, layers=tuple(layers))
