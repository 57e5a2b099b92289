"""Tiny Lalepel configurations, random model folders with weights shaped so that faults show, and the
schedules that the host tests (plain twins of the kernels, CPU) and the gpu tests both run against the
plain implementation of ``plain_lalepel``.

Random weights of standard deviation 0.02 give scores near zero: attention is then nearly uniform, a sink
of 0.02 hardly counts, and a key more or less at a window's edge moves a logit by a hair.  ``sharpen``
scales the query and key projections so that scores spread over several units, sets sinks that compete
with the best scores, gives the router biases that matter, and mixes slow and fast decays."""
import copy
import json
import os

import torch

import plain_lalepel as plain


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window=None, rot_dims=None, scaling=None, scale=None, base=10000.0):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if rot_dims is None:
        rot_dims = rot_dim
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = scaling
    return {"type": "latent_attention", "mixer": m}


def retention(heads, dim, vdim, decay):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def with_mlp(layer, mlp):
    layer = copy.deepcopy(layer)
    layer["mlp"] = mlp
    return layer


DENSE = lambda ff: {"kind": "dense", "ff": ff}  # noqa: E731
MOE = lambda e, top, ff, shared=0: {"kind": "moe", "router": {"experts": e, "top": top}, "expert": {"ff": ff},  # noqa: E731
                                    **({"shared": {"ff": shared}} if shared else {})}
SCALING = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


def model(width, vocab, layers, eps=1e-5):
    return {"architecture": "Lalepel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # every mechanism, sizes that are multiples of 8, two latent layers of different shapes (two cache groups)
    "mix": model(64, 97, [
        with_mlp(latent(3, 16, 8, 24, 40, 32, window=12, scaling=SCALING), MOE(6, 2, 24, shared=32)),
        with_mlp(retention(2, 16, 8, [0.9, 0.97]), DENSE(96)),
        with_mlp(latent(2, 8, 16, 16, 24, 16, rot_dims=8, base=500.0), None),
        with_mlp(retention(1, 40, 12, [1.0]), MOE(4, 4, 16)),
    ]),
    # sizes that are no multiples of 8 or 4, one head, top 1, a window of one token and one of many
    "odd": model(52, 61, [
        with_mlp(retention(3, 12, 10, [0.5, 0.99, 0.999]), MOE(5, 1, 12, shared=20)),
        with_mlp(latent(1, 12, 6, 10, 20, 28, window=1, scaling={"factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0}), DENSE(36)),
        with_mlp(latent(5, 4, 2, 6, 12, 12, window=70), None),
    ], eps=1e-6),
    # nothing a multiple of 4: width 50, a latent of 10 + 4, rows of 5 and 3
    "odd2": model(50, 33, [
        with_mlp(latent(2, 6, 4, 5, 9, 10, window=5), MOE(3, 2, 7, shared=5)),
        with_mlp(retention(1, 5, 3, [0.8]), DENSE(9)),
    ]),
    # one layer each: a mechanism alone
    "latent_only": model(48, 50, [with_mlp(latent(4, 8, 16, 8, 16, 32, window=20, scaling=SCALING), None)]),
    "latent_full": model(48, 50, [with_mlp(latent(2, 16, 0, 8, 32, 40, rot_dims=0), None)]),
    "retention_only": model(48, 50, [with_mlp(retention(2, 24, 16, [0.95, 0.999]), None)]),
    "dense_only": model(40, 50, [with_mlp(retention(1, 8, 8, [0.9]), DENSE(72))]),
    "moe_only": model(40, 50, [with_mlp(retention(1, 8, 8, [0.9]), MOE(7, 3, 16, shared=24))]),
    # no routed layer: a window, a state and a layer that sees every key
    "no_router": model(64, 83, [
        with_mlp(latent(2, 16, 16, 16, 24, 32, window=24, scaling=SCALING), DENSE(64)),
        with_mlp(retention(2, 16, 16, [0.97, 0.9995]), DENSE(48)),
        with_mlp(latent(3, 8, 8, 8, 16, 16, base=300.0), None),
    ]),
    # larger heads: latent rows of 160 elements, state rows beyond one lane's first register
    "wide": model(128, 211, [
        with_mlp(latent(4, 32, 32, 32, 64, 128, window=100, scaling={"factor": 6.0, "original": 256, "fast": 24.0, "slow": 1.5}), DENSE(256)),
        with_mlp(retention(2, 72, 40, [0.98, 0.9995]), MOE(8, 2, 64, shared=64)),
    ]),
}
SEEDS = {n: 11 + i for i, n in enumerate(CONFIGS)}


def sharpen(name, w):
    """Weights (name -> float32 tensor) changed in place so that windows, sinks, far keys and router biases matter."""
    for n in list(w):
        if n.endswith(".mix.uq") or n.endswith(".mix.uk"):
            w[n] = w[n] * 9.0
        elif n.endswith(".mix.dkv"):
            w[n] = w[n] * 3.0
        elif n.endswith(".mix.sink"):
            w[n] = torch.linspace(-1.0, 2.5, w[n].numel())
        elif n.endswith(".router.b"):
            w[n] = w[n] * 20.0
        elif n.endswith(".router"):
            w[n] = w[n] * 6.0
        elif n.endswith(".mix.q") or n.endswith(".mix.k"):
            w[n] = w[n] * 4.0
        elif n == "embed":
            w[n] = w[n] * 30.0


def make_dir(tmp_path, name, store_dtype=torch.bfloat16, raw=None, tweak=sharpen, seed=None):
    """A model folder of configuration ``name`` (or ``raw``): seeded random weights, then ``tweak``, stored in
    ``store_dtype``.  Returns (folder, config dict, weights as stored, float32)."""
    from locus_b200.weights.loader import write_random_model
    from locus_b200.weights.safetensors_io import ModelFiles, write_safetensors
    import locus_b200.models  # noqa: F401

    cfg = copy.deepcopy(raw if raw is not None else CONFIGS[name])
    d = os.path.join(str(tmp_path), f"lalepel_{name}_{str(store_dtype).split('.')[-1]}")
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


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class Case:
    def __init__(self, name, tmp_path, store_dtype=torch.bfloat16, raw=None, requests=(), tweak=sharpen):
        self.name = name
        self.dir, self.cfg, self.weights = make_dir(tmp_path, name, store_dtype, raw=raw, tweak=tweak)
        self.tokens = {f"r{i}": tokens(n, self.cfg["vocab"], 1000 * (i + 1) + n) for i, n in enumerate(requests)}
        self._ref = {}

    def ref(self, rid, picks=None):
        """(oracle logits [T, vocab] float64, router logits by feed-forward prefix)."""
        key = rid if picks is None else None
        if key is not None and key in self._ref:
            return self._ref[key]
        aux = {}
        lg, _ = plain.forward(self.cfg, self.weights, self.tokens[rid], picks=picks, aux=aux)
        if key is not None:
            self._ref[key] = (lg, aux)
        return lg, aux

    def ref_following(self, rid, routed, near_tie):
        """The oracle's logits when it takes the engine's picks (``routed``: prefix -> {position: picks}) where they
        differ from its own.  A difference is allowed only at a near-tie: every expert the engine picked must have
        a logit within ``near_tie`` times the spread of the token's logits (largest minus smallest) of the oracle's
        weakest own pick."""
        base, aux = self.ref(rid)
        T = len(self.tokens[rid])
        forced, differs = {}, 0
        for prefix, per_pos in (routed or {}).items():
            z = aux[prefix]
            top = len(next(iter(per_pos.values()))) if per_pos else 0
            own = torch.topk(z, top, dim=-1).indices if top else None
            rows = []
            for pos in range(T):
                mine = own[pos].tolist()
                eng = per_pos.get(pos, mine)
                if sorted(eng) != sorted(mine):
                    differs += 1
                    weakest = min(float(z[pos, e]) for e in mine)
                    spread = float(z[pos].max() - z[pos].min())
                    for e in eng:
                        assert float(z[pos, e]) >= weakest - near_tie * spread, (
                            f"{self.name}/{rid} {prefix} position {pos}: the engine picked expert {e} with logit "
                            f"{float(z[pos, e]):.5f}; the oracle's weakest pick has {weakest:.5f}")
                rows.append(eng)
            forced[prefix] = torch.tensor(rows, dtype=torch.int64)
        if differs == 0:
            return base
        # the picks of later layers were made by the engine on its own activations: follow them all
        return self.ref(rid, picks=forced)[0]


def make_runner(case, dtype, device, *, page_tokens=16, n_pages=64, max_tokens=320, max_seq=1024, slots=4,
                use_graphs=False):
    from locus_b200.cache import CacheManager
    from locus_b200.engine.step import ModelRunner
    from locus_b200.models import load_model

    m = load_model(case.dir, dtype, device)
    cache = CacheManager(m.cache_needs(), page_tokens=page_tokens, n_pages=n_pages, n_state_slots=slots,
                         max_seq_tokens=max_seq, dtype=dtype, device=device, poison=True)
    return ModelRunner(m, cache, max_tokens=max_tokens, max_segments=slots, use_graphs=use_graphs), cache


def run_steps(runner, cache, case, steps):
    """steps: lists of (request id, n tokens); every fed position's logits are wanted.  A request is released after
    its last token (its pages and its state slot are used again by whoever comes next).  Returns
    ({rid: [T, V] logits on the CPU}, {rid: {feed-forward prefix: {position: picked experts}}})."""
    from locus_b200.engine.step import StepEntry

    fed, got, routed = {}, {}, {}
    seen = {}
    for part in runner.model.all_parts():
        if hasattr(part, "observer"):
            part.observer = lambda prefix, ids, wts: seen.__setitem__(prefix, ids.detach().cpu().tolist())
    for step in steps:
        entries = []
        for rid, n in step:
            a = fed.get(rid, 0)
            seq = cache.get(rid) or cache.open(rid)
            assert cache.ensure_capacity(seq, n), (rid, n)
            entries.append(StepEntry(seq, case.tokens[rid][a:a + n], list(range(n))))
        seen.clear()
        lg = runner.step(entries).detach().cpu().double()
        row = 0
        for rid, n in step:
            a = fed.get(rid, 0)
            got.setdefault(rid, []).append(lg[row:row + n].clone())
            for prefix, ids in seen.items():
                per = routed.setdefault(rid, {}).setdefault(prefix, {})
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


def cuts(n, sizes):
    """n tokens in portions of the given sizes, repeated as needed."""
    out, i = [], 0
    while n > 0:
        k = min(n, sizes[i % len(sizes)])
        out.append(k)
        n -= k
        i += 1
    return out


def schedules(case):
    """name -> steps over the case's requests r0.. (see ``run_steps``)."""
    toks = case.tokens
    rids = list(toks)
    whole = [[(r, len(toks[r]))] for r in rids]
    decode = []
    for r in rids:
        n = len(toks[r])
        tail = min(n - 1, 24) if n > 1 else 0
        decode += ([[(r, n - tail)]] if n - tail else []) + [[(r, 1)]] * tail
    chunked = []
    for i, r in enumerate(rids):
        n = len(toks[r])
        tail = min(n - 1, 5)
        chunked += [[(r, k)] for k in cuts(n - tail, [2, 7, 16, 3, 33, 2, 64][i % 3:] + [5])] + [[(r, 1)]] * tail
    # up to four live requests, portions beside single tokens, requests that end and are followed by others
    left = {r: len(toks[r]) for r in rids}
    waiting, live, mixed, turn = list(rids), [], [], 0
    sizes = [3, 1, 17, 2, 1, 30, 1, 8, 1, 1, 40, 5]
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        step = []
        for j, r in enumerate(list(live)):
            if (turn + j) % 5 == 4 and len(live) > 1:
                continue  # sits this step out
            k = min(left[r], sizes[(turn + 3 * j) % len(sizes)])
            step.append((r, k))
            left[r] -= k
            if left[r] == 0:
                live.remove(r)
        if step:
            mixed.append(step)
        turn += 1
    return {"whole": whole, "decode": decode, "chunked": chunked, "mixed": mixed}
