"""A plain, slow, whole-sequence implementation of the Lalepel design: one function per
mechanism, float64 on the CPU, written from the design's equations and sharing no code with
the engine.  The tests compare the engine's parts and whole models with it.

The design: a decoder whose sublayers read the residual stream x itself and whose outputs
are normed before they are added,

    x <- x + rmsnorm_1(mixer(x)),   x <- x + rmsnorm_2(ff(x))      (ff may be absent),

with two mixers (latent attention with a sliding window and a sink; retention, a linear
recurrence with a fixed decay per head) and two feed-forwards (a gated dense one; routed
experts with a squared-ReLU activation, a router bias and a gated shared expert).

``weights`` is a dict name -> tensor (any float type; converted to float64 here), ``cfg`` the
dictionary of the model's config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def _w(weights, name) -> torch.Tensor:
    return weights[name].to(F64)


# ---------------------------------------------------------------------------
# norms and activations


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def relu2(z: torch.Tensor) -> torch.Tensor:
    r = torch.clamp(z, min=0.0)
    return r * r


# ---------------------------------------------------------------------------
# rotary positions with the long-context frequency ramp


def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]) -> Tuple[List[float], float]:
    """(frequency of every pair i < dims / 2, the factor on cosine and sine)."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turns_dim(t: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns_dim(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, freqs: List[float], mag: float) -> torch.Tensor:
    """x [T, ..., n]: the pairs (2i, 2i + 1), i < len(freqs), are turned by positions[t] * freqs[i];
    what lies behind 2 * len(freqs) passes unchanged."""
    out = x.clone()
    T = x.shape[0]
    shape = [T] + [1] * (x.dim() - 2)
    for i, fr in enumerate(freqs):
        a = positions.to(F64) * fr
        c, s = (torch.cos(a) * mag).view(shape), (torch.sin(a) * mag).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ---------------------------------------------------------------------------
# mixers


def latent_attention(h: torch.Tensor, weights, prefix: str, m: dict, eps: float,
                     positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h [T, width] of one sequence from position 0 on (or at ``positions``) -> [T, width]."""
    T = h.shape[0]
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    cq = rmsnorm(h @ _w(weights, prefix + ".dq").T, _w(weights, prefix + ".dq.norm"), eps)
    q = (cq @ _w(weights, prefix + ".uq").T).view(T, H, dn + dr)
    dkv = h @ _w(weights, prefix + ".dkv").T
    c = rmsnorm(dkv[:, :rk], _w(weights, prefix + ".dkv.norm"), eps)
    k_rot = dkv[:, rk:]
    rot = m.get("rot") or {}
    if rot:
        freqs, mag = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        q = torch.cat([q[..., :dn], rotate_pairs(q[..., dn:], pos, freqs, mag)], -1)
        k_rot = rotate_pairs(k_rot, pos, freqs, mag)
    k_nope = (c @ _w(weights, prefix + ".uk").T).view(T, H, dn)
    v = (c @ _w(weights, prefix + ".uv").T).view(T, H, dv)
    sink = _w(weights, prefix + ".sink")
    window = int((m.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        seen = torch.ones(t + 1, dtype=torch.bool)
        if window > 0:
            back = pos[t] - pos[: t + 1]
            seen = (back >= 0) & (back < window)
        for hh in range(H):
            s = (k_nope[: t + 1, hh] @ q[t, hh, :dn] + k_rot[: t + 1] @ q[t, hh, dn:]) * m["scale"]
            s = s[seen]
            big = max(float(s.max()), float(sink[hh]))
            e = torch.exp(s - big)
            den = e.sum() + math.exp(float(sink[hh]) - big)
            out[t, hh] = (e / den) @ v[: t + 1, hh][seen]
    return out.reshape(T, H * dv) @ _w(weights, prefix + ".o").T


def retention(h: torch.Tensor, weights, prefix: str, m: dict, eps: float,
              state: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """h [T, width] -> ([T, width], the state [heads, dim, vdim] behind the last token)."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ _w(weights, prefix + ".q").T).view(T, H, d)
    k = (h @ _w(weights, prefix + ".k").T).view(T, H, d) * d ** -0.5
    v = (h @ _w(weights, prefix + ".v").T).view(T, H, dv)
    g = silu(h @ _w(weights, prefix + ".g").T)
    S = torch.zeros(H, d, dv, dtype=F64) if state is None else state.to(F64).clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for hh in range(H):
            S[hh] = float(m["decay"][hh]) * S[hh] + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    o = rms_unit(o, eps).reshape(T, H * dv) * g
    return o @ _w(weights, prefix + ".o").T, S


# ---------------------------------------------------------------------------
# feed-forwards


def dense_ff(h: torch.Tensor, weights, prefix: str) -> torch.Tensor:
    a = silu(h @ _w(weights, prefix + ".gate").T) * (h @ _w(weights, prefix + ".up").T)
    return a @ _w(weights, prefix + ".down").T


def relu2_expert(h: torch.Tensor, weights, prefix: str) -> torch.Tensor:
    return relu2(h @ _w(weights, prefix + ".up").T) @ _w(weights, prefix + ".down").T


def route(h: torch.Tensor, weights, prefix: str, top: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(logits [T, E], the picked experts [T, top] by falling logit, their weights [T, top])."""
    z = h @ _w(weights, prefix + ".router").T + _w(weights, prefix + ".router.b")
    val, idx = torch.topk(z, top, dim=-1)
    return z, idx, torch.softmax(val, -1)


def moe_ff(h: torch.Tensor, weights, prefix: str, mlp: dict, picks: Optional[torch.Tensor] = None,
           aux: Optional[dict] = None) -> torch.Tensor:
    """``picks`` [T, top]: use these experts instead of the router's own choice (the weights
    are then the softmax over THEIR logits), for comparisons that must not hinge on a near-tie.
    ``aux``: gets the router's logits under the prefix."""
    T = h.shape[0]
    top = int(mlp["router"]["top"])
    z, idx, wts = route(h, weights, prefix, top)
    if aux is not None:
        aux[prefix] = z
    if picks is not None:
        idx = picks.to(torch.int64)
        wts = torch.softmax(torch.gather(z, 1, idx), -1)
    out = torch.zeros_like(h)
    for t in range(T):
        for s in range(top):
            e = int(idx[t, s])
            out[t] += wts[t, s] * relu2_expert(h[t:t + 1], weights, f"{prefix}.e{e}")[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ _w(weights, prefix + ".shared.sg").T)      # [T, 1]
        out = out + gate * relu2_expert(h, weights, prefix + ".shared")
    return out


# ---------------------------------------------------------------------------
# the model


def forward(cfg: dict, weights, tokens: List[int], picks: Optional[Dict[str, torch.Tensor]] = None,
            round_inputs=None, aux: Optional[dict] = None) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """Logits [T, vocab] of one sequence from position 0 on, and the residual stream behind every layer.
    ``round_inputs``: a function applied to what a sublayer reads (to mimic a 16-bit engine)."""
    eps = float(cfg["norm"]["eps"])
    rd = round_inputs or (lambda t: t)
    x = _w(weights, "embed")[torch.tensor(tokens, dtype=torch.int64)]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        if layer["type"] == "latent_attention":
            y = latent_attention(rd(x), weights, p + ".mix", layer["mixer"], eps)
        elif layer["type"] == "retention":
            y, _ = retention(rd(x), weights, p + ".mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rmsnorm(y, _w(weights, p + ".norm1"), eps)
        mlp = layer.get("mlp")
        if mlp:
            if mlp["kind"] == "dense":
                y = dense_ff(rd(x), weights, p + ".mlp")
            elif mlp["kind"] == "moe":
                y = moe_ff(rd(x), weights, p + ".mlp", mlp, None if picks is None else picks.get(p + ".mlp"), aux)
            else:
                raise ValueError(mlp["kind"])
            x = x + rmsnorm(y, _w(weights, p + ".norm2"), eps)
        streams.append(x.clone())
    logits = rmsnorm(x, _w(weights, "final.norm"), eps) @ _w(weights, "head").T
    return logits, streams
