"""Tiny Pozozen configurations, random model folders with weights shaped so that faults show, and the helpers that
the host tests (plain twins of the kernels, CPU) and the gpu tests share to run schedules against the plain
implementation of ``plain_pozozen``.

Random weights of standard deviation 0.02 hide faults: attention is nearly uniform, every state decays in a few
tokens, the streams hardly mix and the router's correction never decides.  ``sharpen`` spreads the scores, gives the
recurrences slow and fast heads, forget gates near one, stream tables that mix, and corrections of the size of the
scores."""
import copy
import json
import os

import torch

import plain_pozozen as plain
from lalepel_cases import cuts, make_runner, schedules, tokens  # noqa: F401  (shared schedule helpers)


def mlstm(heads, dim, vdim, cap=15.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def parallel(heads, kv_heads, dim, vdim, window, s_heads, s_vdim, state, groups=1, conv=4, norm_groups=1,
             left_scale=0.7, right_scale=0.4, scale=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window:
        left["mask"] = {"size": window}
    right = {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def moe(experts, top, ff, identity=0, groups=None, shared=0):
    router = {"experts": experts, "top": top}
    if identity:
        router["identity"] = identity
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def with_mlp(layer, mlp):
    layer = copy.deepcopy(layer)
    layer["mlp"] = mlp
    return layer


def model(width, vocab, layers, streams=2, mult=0.5, loop=None, eps=1e-5):
    cfg = {"architecture": "Pozozen", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": mult,
           "layers": layers}
    if streams:
        cfg["streams"] = streams
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


CONFIGS = {
    # every mechanism, a loop of three passes over two layers, three streams, values unlike keys, two groups
    "mix": model(64, 97, [
        with_mlp(parallel(4, 2, 16, 32, 12, 4, 8, 16, groups=2, conv=3, norm_groups=2), moe(6, 3, 24, identity=2, groups=(4, 2), shared=32)),
        with_mlp(mlstm(2, 16, 24), moe(4, 2, 16, identity=4, groups=(2, 1))),
        with_mlp(parallel(2, 1, 32, 16, 0, 2, 16, 8, conv=2), None),
        with_mlp(mlstm(3, 8, 8, cap=6.0), moe(5, 5, 8, shared=16)),
    ], streams=3, loop=(1, 3, 3)),
    # nothing a multiple of 8 or 4, one stream with tables, one head, top 1, a window of one token
    "odd": model(50, 61, [
        with_mlp(mlstm(1, 10, 7), moe(3, 1, 7, identity=1)),
        with_mlp(parallel(3, 3, 10, 6, 1, 3, 5, 9, groups=3, conv=5, norm_groups=3, left_scale=1.0, right_scale=-0.5), moe(4, 2, 9, shared=5)),
        with_mlp(parallel(2, 1, 6, 10, 37, 1, 11, 7, conv=1), None),
    ], streams=1, mult=1.0, eps=1e-6),
    # no stream tables at all, no loop, layers without a feed-forward
    "plain": model(48, 50, [
        with_mlp(parallel(2, 2, 16, 16, 20, 2, 8, 8), None),
        with_mlp(mlstm(2, 12, 12), moe(4, 2, 16, identity=4, groups=(4, 3))),
    ], streams=0, mult=0.3),
    # one layer each: a mechanism alone
    "mlstm_only": model(48, 50, [with_mlp(mlstm(2, 24, 16), None)], streams=2),
    "attention_only": model(48, 50, [with_mlp(parallel(4, 2, 16, 16, 9, 1, 8, 8, right_scale=0.0), None)], streams=2),
    "ssm_only": model(48, 50, [with_mlp(parallel(1, 1, 16, 16, 4, 4, 12, 20, groups=2, conv=4, norm_groups=2, left_scale=0.0, right_scale=1.0), None)], streams=2),
    "moe_only": model(40, 50, [with_mlp(mlstm(1, 8, 8), moe(9, 3, 16, identity=3, groups=(4, 2), shared=24))], streams=2, loop=(0, 1, 2)),
    # larger heads: rows of the recurrences beyond one lane's first register, a state of 72, heads of 80
    "wide": model(128, 211, [
        with_mlp(parallel(2, 1, 80, 64, 100, 4, 40, 72, groups=2, norm_groups=4), moe(8, 2, 64, identity=8, groups=(8, 3), shared=64)),
        with_mlp(mlstm(2, 72, 40), moe(6, 2, 32, identity=2, groups=(2, 2))),
    ], streams=4, loop=(0, 2, 2)),
}
SEEDS = {n: 31 + i for i, n in enumerate(CONFIGS)}


def sharpen(name, w):
    """Weights (name -> float32 tensor) changed in place so that windows, far keys, states, streams and the router's
    correction matter."""
    g = torch.Generator().manual_seed(7)
    for n in list(w):
        t = w[n]
        if n.endswith((".left.q", ".left.k")):
            w[n] = t * 6.0
        elif n.endswith((".mix.q", ".mix.k")):
            w[n] = t * 5.0
        elif n.endswith((".mix.i", ".mix.f")):
            w[n] = t * 8.0
        elif n.endswith(".mix.f.b"):
            w[n] = torch.linspace(1.0, 6.0, t.numel())          # forget gates from 0.73 to 0.998
        elif n.endswith(".mix.i.b"):
            w[n] = torch.linspace(-1.0, 1.0, t.numel())
        elif n.endswith(".right.A_log"):
            w[n] = torch.linspace(-5.0, 0.5, t.numel())         # decays per unit step from 0.993 to 0.19
        elif n.endswith(".right.dt_bias"):
            w[n] = torch.linspace(-2.0, 1.0, t.numel())
        elif n.endswith(".right.in"):
            w[n] = t * 4.0
        elif n.endswith(".right.conv"):
            w[n] = t * 20.0
        elif n.endswith(".right.D"):
            w[n] = torch.linspace(0.5, 1.5, t.numel())
        elif n.endswith(".router"):
            w[n] = t * 8.0
        elif n.endswith(".correction"):
            w[n] = (torch.rand(t.shape, generator=g) - 0.6) * 0.3  # of the size of the scores, some negative
        elif n.endswith((".in", ".out")) and ".hc" in n:
            w[n] = 0.5 + torch.rand(t.shape, generator=g)
        elif n.endswith(".mix") and ".hc" in n:
            w[n] = torch.eye(t.shape[0]) * 0.8 + (torch.rand(t.shape, generator=g) - 0.5) * 0.5
        elif n.endswith(".b") and ".norm" in n:
            w[n] = t * 10.0
        elif n == "embed":
            w[n] = t * 30.0


def sharpen_mildly(name, w):
    """``sharpen`` with a softer router and softer scores, for drawn configurations: deeper models, in which weights as
    sharp as the fixed cases' let single positions amplify rounding a hundred times."""
    sharpen(name, w)
    for n in w:
        if n.endswith(".router"):
            w[n] = w[n] / 4.0
        elif n.endswith((".left.q", ".left.k", ".mix.q", ".mix.k")):
            w[n] = w[n] / 2.0
        elif n == "embed":
            w[n] = w[n] / 3.0


def make_dir(tmp_path, name, store_dtype=torch.bfloat16, raw=None, tweak=sharpen, seed=None):
    """A model folder of configuration ``name`` (or ``raw``): seeded random weights, then ``tweak``, stored in
    ``store_dtype``.  Returns (folder, config dict, weights as stored, float32)."""
    from locus_b200.weights.loader import write_random_model
    from locus_b200.weights.safetensors_io import ModelFiles, write_safetensors
    import locus_b200.models  # noqa: F401

    cfg = copy.deepcopy(raw if raw is not None else CONFIGS[name])
    d = os.path.join(str(tmp_path), f"pozozen_{name}_{str(store_dtype).split('.')[-1]}")
    write_random_model(cfg, SEEDS.get(name, 5) if seed is None else seed, d, torch.float32)
    mf = ModelFiles(d)
    w = {n: mf.tensor(n).clone().float() for n in mf.names()}
    mf.close()
    if tweak is not None:
        tweak(name, w)
    w = {n: t.to(store_dtype) for n, t in w.items()}
    write_safetensors(os.path.join(d, "model.safetensors"), [(n, tuple(t.shape), store_dtype) for n, t in w.items()],
                      lambda n: w[n], metadata={"format": "pt"})
    with open(os.path.join(d, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    return d, cfg, {n: t.float() for n, t in w.items()}


class Case:
    def __init__(self, name, tmp_path, store_dtype=torch.bfloat16, raw=None, requests=(), tweak=sharpen):
        self.name = name
        self.dir, self.cfg, self.weights = make_dir(tmp_path, name, store_dtype, raw=raw, tweak=tweak)
        self.tokens = {f"r{i}": tokens(n, self.cfg["vocab"], 1000 * (i + 1) + n) for i, n in enumerate(requests)}
        self.order = plain.run_order(self.cfg)
        self._ref = {}

    def ref(self, rid, picks=None):
        """(oracle logits [T, vocab] float64, the routers' scores by index in the run order)."""
        if picks is None and rid in self._ref:
            return self._ref[rid]
        aux = {}
        lg = plain.forward(self.weights, self.cfg, self.tokens[rid], picks=picks, aux=aux)
        if picks is None:
            self._ref[rid] = (lg, aux)
        return lg, aux

    def ref_following(self, rid, routed, near_tie):
        """The oracle's logits when it takes the engine's picks (``routed``: index in the run order -> {position:
        picks}) where they differ from its own.  A difference is allowed only at a near-tie of the oracle's own
        decision: the margin between the last expert it takes and the first it leaves (among the open groups), or
        between the last group it keeps and the first it closes, is below ``near_tie`` times the spread of the row's
        choice scores."""
        base, aux = self.ref(rid)
        T = len(self.tokens[rid])
        forced, differs = {}, 0
        for call, per_pos in (routed or {}).items():
            a = aux[call]
            rows = []
            for pos in range(T):
                mine = a["own"][pos].tolist()
                eng = per_pos.get(pos, mine)
                if sorted(eng) != sorted(mine):
                    differs += 1
                    ch = a["choice"][pos]
                    spread = float(ch.max() - ch.min())
                    m = torch.sort(a["masked"][pos], descending=True).values
                    margins = [float(m[len(mine) - 1] - m[len(mine)])] if len(mine) < len(m) else []
                    gs = torch.sort(a["groups"][pos], descending=True).values
                    keep = int((a["masked"][pos] > -float("inf")).sum()) // (len(ch) // len(gs))
                    if keep < len(gs):
                        margins.append(float(gs[keep - 1] - gs[keep]))
                    assert margins and min(margins) <= near_tie * spread, (
                        f"{self.name}/{rid} layer call {call} position {pos}: the engine picked {eng}, the oracle {mine}, "
                        f"and the oracle's decision is no near-tie (margins {margins}, spread {spread:.4f})")
                rows.append(eng)
            forced[call] = rows
        if differs == 0:
            return base
        # the picks of later layers were made by the engine on its own activations: follow them all
        return self.ref(rid, picks=forced)[0]


def run_steps(runner, cache, case, steps):
    """steps: lists of (request id, n tokens); every fed position's logits are wanted.  A request is released after
    its last token (its pages and its state slot are used again by whoever comes next).  Returns
    ({rid: [T, V] logits on the CPU}, {rid: {index in the run order: {position: picked experts}}})."""
    from locus_b200.engine.step import StepEntry

    fed, got, routed = {}, {}, {}
    seen = []
    for part in runner.model.all_parts():
        if hasattr(part, "observer"):
            part.observer = lambda prefix, ids, wts: seen.append((prefix, ids.detach().cpu().tolist()))
    # a looped layer's feed-forward reports once per pass: the n-th report of a prefix is its n-th call in the order
    calls_of = {}
    for call, i in enumerate(case.order):
        calls_of.setdefault(f"l{i}.mlp", []).append(call)
    for step in steps:
        entries = []
        for rid, n in step:
            a = fed.get(rid, 0)
            seq = cache.get(rid) or cache.open(rid)
            assert cache.ensure_capacity(seq, n), (rid, n)
            entries.append(StepEntry(seq, case.tokens[rid][a:a + n], list(range(n))))
        seen.clear()
        lg = runner.step(entries).detach().cpu().double()
        nth = {}
        by_call = {}
        for prefix, ids in seen:
            k = nth.get(prefix, 0)
            nth[prefix] = k + 1
            by_call[calls_of[prefix][k]] = ids
        row = 0
        for rid, n in step:
            a = fed.get(rid, 0)
            got.setdefault(rid, []).append(lg[row:row + n].clone())
            for call, ids in by_call.items():
                per = routed.setdefault(rid, {}).setdefault(call, {})
                for i in range(n):
                    per[a + i] = ids[row + i]
            row += n
            fed[rid] = a + n
        for rid, n in step:
            if fed[rid] == len(case.tokens[rid]):
                cache.release(cache.get(rid))
        cache.check_invariants()
    if hasattr(runner, "check_device_errors"):
        runner.check_device_errors()
    return {r: torch.cat(v) for r, v in got.items()}, routed


def compare(case, got, routed, tol_max, tol_mean, near_tie):
    for rid, out in got.items():
        ref = case.ref_following(rid, routed.get(rid), near_tie)
        assert out.shape == ref.shape, rid
        assert bool(torch.isfinite(out).all()), f"{case.name}/{rid}: logits that are not numbers (a page or slot read stale?)"
        d = (out - ref)
        d = d - d.mean(-1, keepdim=True)
        top = float((ref - ref.mean(-1, keepdim=True)).abs().max())
        err = d.abs().max(-1).values / top
        worst = int(err.argmax())
        assert float(err.max()) <= tol_max, f"{case.name}/{rid}: position {worst} is off by {float(err.max()):.2e} of the largest logit"
        assert float(d.abs().mean()) / top <= tol_mean, f"{case.name}/{rid}: mean error {float(d.abs().mean()) / top:.2e}"


def compare_together(case, got, routed, tol_max, tol_mean, near_tie, one_in=50, cap=10.0):
    """As ``compare``, for models in which single positions amplify rounding (a matrix memory's normaliser n . q that
    passes near zero, a router's choice that nearly flips): the mean error as everywhere, all but one row in ``one_in``
    within ``tol_max``, and no row beyond ``cap`` times that."""
    for rid, out in got.items():
        ref = case.ref_following(rid, routed.get(rid), near_tie)
        assert out.shape == ref.shape and bool(torch.isfinite(out).all()), rid
        d = out - ref
        d = d - d.mean(-1, keepdim=True)
        top = float((ref - ref.mean(-1, keepdim=True)).abs().max())
        err = d.abs().max(-1).values / top
        assert float(d.abs().mean()) / top <= tol_mean, f"{case.name}/{rid}: mean error {float(d.abs().mean()) / top:.2e}"
        assert float(err.max()) <= cap * tol_max, f"{case.name}/{rid}: position {int(err.argmax())} is off by {float(err.max()):.2e}"
        assert int((err > tol_max).sum()) <= max(1, len(err) // one_in), f"{case.name}/{rid}: {int((err > tol_max).sum())} rows beyond {tol_max}"


def random_config(seed):
    """A configuration drawn from the ranges a small model of this design may have: layer order, loop, streams, head
    counts and sizes, windows, groups, taps, experts, identity experts and constants all vary."""
    import random

    r = random.Random(seed)
    width = r.choice([64, 96, 128, 192, 256])

    def routed():
        if r.random() < 0.15:
            return None
        experts, identity = r.choice([4, 6, 8, 12, 16]), r.choice([0, 0, 2, 4])
        total = experts + identity
        count = r.choice([c for c in (1, 2, 3, 4, 6, 8) if total % c == 0])
        keep = r.randint(1, count)
        top = r.randint(1, min(6, keep * (total // count)))
        return moe(experts, top, r.choice([32, 64, 96]), identity=identity, groups=(count, keep) if count > 1 or r.random() < 0.5 else None,
                   shared=r.choice([0, 64, 128]))

    def layer():
        if r.random() < 0.5:
            return with_mlp(mlstm(r.choice([1, 2, 4]), r.choice([16, 32, 48, 64]), r.choice([16, 32, 48, 64]), cap=r.choice([10.0, 15.0, 30.0])), routed())
        heads = r.choice([1, 2, 4, 8])
        kv = r.choice([k for k in (1, 2, 4, 8) if heads % k == 0])
        dim = r.choice([16, 32, 48, 64, 96, 128])
        s_heads = r.choice([2, 4, 8])
        s_vdim = r.choice([16, 32, 64])
        return with_mlp(parallel(heads, kv, dim, r.choice([dim, dim, 32, 64]), r.choice([0, 8, 33, 64, 96, 128]), s_heads, s_vdim,
                                 r.choice([16, 32, 48, 64, 128]), groups=r.choice([g for g in (1, 2, 4) if s_heads % g == 0]),
                                 conv=r.choice([2, 3, 4]), norm_groups=r.choice([g for g in (1, 2, 4) if (s_heads * s_vdim) % g == 0]),
                                 left_scale=round(r.uniform(0.3, 1.0), 2), right_scale=round(r.uniform(0.3, 1.0), 2),
                                 scale=dim ** -0.5 * r.choice([1.0, 1.0, 0.5, 2.0])), routed())

    n = r.randint(3, 6)
    layers = [layer() for _ in range(n)]
    loop = None
    if r.random() < 0.7:
        a = r.randint(0, n - 1)
        loop = (a, r.randint(a + 1, n), r.randint(2, 3))
    return model(width, r.randint(100, 700), layers, streams=r.choice([0, 1, 2, 2, 3, 4]), mult=round(r.uniform(0.2, 1.0), 2),
                 loop=loop, eps=r.choice([1e-5, 1e-6]))
