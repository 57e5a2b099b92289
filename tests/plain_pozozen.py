"""A plain, slow, whole-sequence implementation of the Pozozen design: one function per mechanism,
float64 on the CPU, written from the design's equations and sharing no code with the engine.

The design: a decoder with ``streams`` copies of the residual stream.  A sublayer
(mixer, then feed-forward) reads a weighted sum of the streams through a layer norm with weight and bias, and
its output is written back into every stream while the streams are mixed among themselves:

    u = sum_s a[s] x_s;   y = sublayer(layernorm(u));   x_t <- sum_s M[s, t] x_s + mult * b[t] * y.

Mixers: ``mlstm`` (a matrix memory with exponential input gate, sigmoid forget gate and a running maximum that
keeps the exponentials in range) and ``parallel`` (windowed grouped-query softmax attention without positions
beside a selective state-space recurrence with a short causal convolution; their outputs are added with fixed
scales).  Feed-forward: routed gated experts with softmax scores, a selection-only correction, groups of
experts of which only the best stay eligible, identity experts that pass their input through, and a shared
expert.  A stretch of layers may run several times in a row with the same weights.

``weights`` is a dict name -> tensor (any float type; converted to float64 here), ``cfg`` the dictionary of
the model's config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def _w(weights, name) -> torch.Tensor:
    return weights[name].to(F64)


# ---------------------------------------------------------------------------
# norms and activations


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w + b


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -softplus(-z)


# ---------------------------------------------------------------------------
# mixers (h: [T, width], one sequence from its first token)


def mlstm(weights, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    T = h.shape[0]
    q = (h @ _w(weights, p + ".q").T).view(T, H, d) * d ** -0.5
    k = (h @ _w(weights, p + ".k").T).view(T, H, d)
    v = (h @ _w(weights, p + ".v").T).view(T, H, dv)
    gi = cap * torch.tanh((h @ _w(weights, p + ".i").T + _w(weights, p + ".i.b")) / cap)            # [T, H]
    gf = log_sigmoid(cap * torch.tanh((h @ _w(weights, p + ".f").T + _w(weights, p + ".f.b")) / cap))
    S = torch.zeros(H, d, dv, dtype=F64)
    n = torch.zeros(H, d, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(gf[t] + mx, gi[t])
        keep = torch.exp(gf[t] + mx - m_new)
        take = torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    o = rms_unit(out, eps).reshape(T, H * dv) * _w(weights, p + ".norm")
    o = o * torch.sigmoid(h @ _w(weights, p + ".g").T)
    return o @ _w(weights, p + ".o").T


def window_attention(weights, p: str, m: dict, h: torch.Tensor) -> torch.Tensor:
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ _w(weights, p + ".q").T + _w(weights, p + ".q.b")).view(T, H, d)
    k = (h @ _w(weights, p + ".k").T + _w(weights, p + ".k.b")).view(T, G, d)
    v = (h @ _w(weights, p + ".v").T + _w(weights, p + ".v.b")).view(T, G, dv)
    mask = m.get("mask")
    window = int(mask["size"]) if mask else 0
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        lo = max(0, t - window + 1) if window else 0
        for a in range(H):
            g = a // (H // G)
            s = (k[lo : t + 1, g] @ q[t, a]) * float(m["scale"])
            w = torch.softmax(s, 0)
            out[t, a] = w @ v[lo : t + 1, g]
    return out.reshape(T, H * dv) @ _w(weights, p + ".o").T


def state_space(weights, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    H, dv, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    parts = int(m["norm_groups"])
    inner, T = H * dv, h.shape[0]
    u = h @ _w(weights, p + ".in").T
    z, xbc, dt = u[:, :inner], u[:, inner : 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N :]
    cw, cb = _w(weights, p + ".conv"), _w(weights, p + ".conv.b")            # [channels, taps], [channels]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=F64), xbc], 0)
    conv = torch.zeros_like(xbc)
    for j in range(taps):                                                       # the last column is the current token's
        conv = conv + padded[j : j + T] * cw[:, j]
    xbc = silu(conv + cb)
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner : inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N :].view(T, G, N)
    dt = softplus(dt + _w(weights, p + ".dt_bias"))                            # [T, H]
    A = torch.exp(_w(weights, p + ".A_log"))
    D = _w(weights, p + ".D")
    S = torch.zeros(H, N, dv, dtype=F64)
    y = torch.zeros(T, H, dv, dtype=F64)
    grp = [a // (H // G) for a in range(H)]
    for t in range(T):
        Bt, Ct = B[t][grp], C[t][grp]                                           # [H, N]
        S = torch.exp(-A * dt[t])[:, None, None] * S + dt[t][:, None, None] * Bt[:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, Ct) + D[:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * _w(weights, p + ".norm")
    return y @ _w(weights, p + ".o").T


def parallel(weights, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    return (float(m["left_scale"]) * window_attention(weights, p + ".left", m["left"], h)
            + float(m["right_scale"]) * state_space(weights, p + ".right", m["right"], h, eps))


# ---------------------------------------------------------------------------
# feed-forward


def gated_expert(weights, p: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ _w(weights, p + ".gate").T) * (h @ _w(weights, p + ".up").T)) @ _w(weights, p + ".down").T


def route(weights, p: str, f: dict, h: torch.Tensor, picks: Optional[List[List[int]]] = None, aux: Optional[dict] = None):
    """(picked experts [T, top], weights [T, top]).  ``picks``: use these picks instead of choosing.  ``aux``: gets the
    choice scores, the groups' scores and the choice scores with the closed groups at minus infinity."""
    r = f["router"]
    E, I, top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.softmax(h @ _w(weights, p + ".router").T, -1)                    # [T, E + I]
    choice = s + _w(weights, p + ".correction")
    per = (E + I) // int(groups["count"])
    best = choice.view(-1, int(groups["count"]), per).max(-1).values            # a group's score: its best
    kept = torch.topk(best, int(groups["keep"]), -1).indices
    open_ = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True).repeat_interleave(per, 1)
    masked = torch.where(open_, choice, torch.full_like(choice, -math.inf))
    ids = torch.topk(masked, top, -1).indices
    if aux is not None:
        aux.update(choice=choice, groups=best, masked=masked, own=ids)
    if picks is not None:
        ids = torch.tensor(picks, dtype=torch.long)
    w = torch.gather(s, 1, ids)
    return ids, w / (w.sum(-1, keepdim=True) + 1e-20)


def moe_ff(weights, p: str, f: dict, h: torch.Tensor, picks=None, aux=None) -> torch.Tensor:
    E = int(f["router"]["experts"])
    ids, w = route(weights, p, f, h, picks, aux)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), w[t]):
            out[t] += g * (h[t] if e >= E else gated_expert(weights, f"{p}.e{e}", h[t : t + 1])[0])
    if f.get("shared"):
        out = out + gated_expert(weights, p + ".shared", h)
    return out


# ---------------------------------------------------------------------------
# the model


def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(weights: Dict[str, torch.Tensor], cfg: dict, tokens, picks: Optional[dict] = None,
            layers_out: Optional[list] = None, aux: Optional[dict] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token.  ``picks`` {index in the run order: experts of every
    row}; ``aux`` gets {index in the run order: the router's scores} (see ``route``); ``layers_out`` the sum of the
    streams behind every layer run."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    n_streams = int(cfg.get("streams", 0))
    x0 = _w(weights, "embed")[torch.as_tensor(tokens, dtype=torch.long)]
    xs = [x0.clone() for _ in range(max(n_streams, 1))]

    def sublayer(q: int, p: str, fn):
        nonlocal xs
        w, b = _w(weights, f"{p}.norm{q}"), _w(weights, f"{p}.norm{q}.b")
        if n_streams == 0:
            xs = [xs[0] + mult * fn(layer_norm(xs[0], w, b, eps))]
            return
        a, o, M = _w(weights, f"{p}.hc{q}.in"), _w(weights, f"{p}.hc{q}.out"), _w(weights, f"{p}.hc{q}.mix")
        y = fn(layer_norm(sum(a[s] * xs[s] for s in range(n_streams)), w, b, eps))
        xs = [sum(M[s, t] * xs[s] for s in range(n_streams)) + mult * o[t] * y for t in range(n_streams)]

    for call, i in enumerate(run_order(cfg)):
        layer, p = cfg["layers"][i], f"l{i}"
        m = layer["mixer"]
        if layer["type"] == "mlstm":
            sublayer(1, p, lambda h: mlstm(weights, p + ".mix", m, h, eps))
        elif layer["type"] == "parallel":
            sublayer(1, p, lambda h: parallel(weights, p + ".mix", m, h, eps))
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            pk = None if picks is None else picks.get(call)
            ax = None if aux is None else aux.setdefault(call, {})
            sublayer(2, p, lambda h: moe_ff(weights, p + ".mlp", layer["mlp"], h, pk, ax))
        if layers_out is not None:
            layers_out.append(sum(xs))
    x = sum(xs)
    x = layer_norm(x, _w(weights, "final.norm"), _w(weights, "final.norm.b"), eps)
    return x @ _w(weights, "head").T
