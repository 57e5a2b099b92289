"""The Pozozen design through the engine's host logic on the CPU (the kernels replaced by their plain torch twins):
configuration and plan, weights by name, the loop's passes with caches of their own, pages of a window and state
slots that are freed and used again, whole prompts, decoding token by token, portions down to two tokens, mixed
batches, and greedy generation through the scheduler -- all against the plain implementation, which shares no code
with any of it.  The kernels themselves are covered by the gpu tests."""
import copy

import pytest
import torch

import emulated_kernels as EK
import plain_pozozen as plain
from pozozen_cases import CONFIGS, Case, compare, compare_together, make_runner, run_steps, schedules
import locus_b200.models  # noqa: F401  (registers the architectures)
from locus_b200.config import ConfigError, find_arch
from locus_b200.config.pozozen import PozozenConfig

TOL = (2e-5, 4e-6)   # max and mean |error| of the logits relative to the largest |logit|; float32 twins
NEAR_TIE = 2e-5


@pytest.fixture(autouse=True)
def _emulate(monkeypatch):
    EK.install(monkeypatch)


def test_config_reads_every_size_and_refuses_what_is_wrong():
    cfg = PozozenConfig.from_dict(copy.deepcopy(CONFIGS["mix"]))
    assert find_arch("Pozozen").parse_config is not None
    p, m = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (p.left.heads, p.left.kv_heads, p.left.dim, p.left.vdim, p.left.window) == (4, 2, 16, 32, 12)
    assert (p.right.heads, p.right.vdim, p.right.state, p.right.groups, p.right.conv, p.right.norm_groups) == (4, 8, 16, 2, 3, 2)
    assert (p.left_scale, p.right_scale) == (0.7, 0.4) and cfg.layers[2].mixer.left.window == 0
    assert (m.heads, m.dim, m.vdim, m.gate_cap) == (2, 16, 24, 15.0) and cfg.layers[3].mixer.gate_cap == 6.0
    f = cfg.layers[0].mlp
    assert (f.experts, f.identity, f.top, f.group_count, f.group_keep, f.expert_ff, f.shared_ff) == (6, 2, 3, 4, 2, 24, 32)
    assert cfg.layers[2].mlp is None and cfg.layers[3].mlp.identity == 0 and cfg.layers[3].mlp.group_count == 1
    assert cfg.run_order() == (0, 1, 2, 1, 2, 1, 2, 3) and cfg.streams == 3 and cfg.residual_mult == 0.5
    plainer = PozozenConfig.from_dict(copy.deepcopy(CONFIGS["plain"]))
    assert plainer.streams == 0 and plainer.loop is None and plainer.run_order() == (0, 1)
    assert tuple(plain.run_order(CONFIGS["mix"])) == cfg.run_order()
    for path, value, word in ((("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "gate_cap"), 0.0, "gate_cap"),
                              (("layers", 0, "mlp", "router", "top"), 9, "top"), (("norm",), None, "norm"),
                              (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
                              (("layers", 0, "mlp", "router", "groups", "count"), 3, "groups"),
                              (("layers", 0, "mixer", "right", "norm_groups"), 5, "norm_groups"),
                              (("loop", "stop"), 9, "loop")):
        raw = copy.deepcopy(CONFIGS["mix"])
        node = raw
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            PozozenConfig.from_dict(raw)


def test_plan_gives_every_pass_of_the_loop_a_cache_of_its_own():
    from locus_b200.models.model import Model

    e = find_arch("Pozozen")
    m = Model(e.build_plan(e.parse_config(copy.deepcopy(CONFIGS["mix"]))), torch.float32, "cpu")
    needs = m.cache_needs()
    assert len(needs) == 8 and all(c is None for _, _, c in needs)
    assert [p is not None for p, _, _ in needs] == [True, False, True, False, True, False, True, False]
    assert all(s is not None for _, s, _ in needs)
    assert needs[0][0].window == 12 and needs[2][0].window == 0 and needs[0][0].head_dim == 32 and needs[2][0].head_dim == 32
    assert m.plan.residual_streams == 3


def test_plain_recurrences_against_their_closed_forms():
    """The oracle's state-space recurrence against y_t = sum_j (prod_(j < l <= t) a_l) dt_j (C_t . B_j) x_j + D x_t, and
    its matrix memory against the sums over all earlier tokens with the weights exp(sum of later f + i_j - m_t)."""
    g = torch.Generator().manual_seed(5)
    D = 24
    h = torch.randn(11, D, generator=g, dtype=torch.float64)
    m = {"heads": 2, "vdim": 3, "state": 4, "groups": 1, "conv": 1, "norm_groups": 1}
    W = {"s.in": torch.randn(2 * 6 + 8 + 2, D, generator=g, dtype=torch.float64) * 0.3, "s.conv": torch.ones(14, 1, dtype=torch.float64),
         "s.conv.b": torch.zeros(14, dtype=torch.float64), "s.dt_bias": torch.tensor([0.1, -0.4], dtype=torch.float64),
         "s.A_log": torch.tensor([-1.0, 0.3], dtype=torch.float64), "s.D": torch.tensor([0.5, 2.0], dtype=torch.float64),
         "s.norm": torch.ones(6, dtype=torch.float64), "s.o": torch.eye(6, dtype=torch.float64)}
    out = plain.state_space(W, "s", m, h, 1e-6)
    u = h @ W["s.in"].T
    z, xbc, dt = u[:, :6], plain.silu(u[:, 6:20]), plain.softplus(u[:, 20:] + W["s.dt_bias"])
    x, B, C = xbc[:, :6].view(11, 2, 3), xbc[:, 6:10], xbc[:, 10:14]
    a = torch.exp(-torch.exp(W["s.A_log"]) * dt)
    y = torch.zeros(11, 2, 3, dtype=torch.float64)
    for t in range(11):
        for j in range(t + 1):
            y[t] += (a[j + 1:t + 1].prod(0) * dt[j] * (C[t] @ B[j]))[:, None] * x[j]
        y[t] += W["s.D"][:, None] * x[t]
    want = plain.rms_unit((y.reshape(11, 6) * plain.silu(z)).view(11, 1, 6), 1e-6).reshape(11, 6)
    assert torch.allclose(out, want, rtol=1e-9, atol=1e-12)

    mm = {"heads": 1, "dim": 4, "vdim": 3, "gate_cap": 5.0}
    W = {f"m.{n}": torch.randn(r, D, generator=g, dtype=torch.float64) * 0.3 for n, r in (("q", 4), ("k", 4), ("v", 3), ("g", 3), ("i", 1), ("f", 1))}
    W.update({"m.i.b": torch.tensor([0.2], dtype=torch.float64), "m.f.b": torch.tensor([2.0], dtype=torch.float64),
              "m.norm": torch.ones(3, dtype=torch.float64), "m.o": torch.eye(3, dtype=torch.float64)})
    out = plain.mlstm(W, "m", mm, h, 1e-6)
    q, k, v = (h @ W["m.q"].T) * 0.5, h @ W["m.k"].T, h @ W["m.v"].T
    gi = 5.0 * torch.tanh((h @ W["m.i"].T + 0.2) / 5.0)[:, 0]
    gf = plain.log_sigmoid(5.0 * torch.tanh((h @ W["m.f"].T + 2.0) / 5.0))[:, 0]
    want = torch.zeros(11, 3, dtype=torch.float64)
    for t in range(11):
        logw = torch.stack([gf[j + 1:t + 1].sum() + gi[j] for j in range(t + 1)])
        mt = torch.maximum(logw.max(), gf[:t + 1].sum())           # the running maximum started at 0
        wgt = torch.exp(logw - mt)
        num = (wgt * (k[:t + 1] @ q[t]))[:, None] * v[:t + 1]
        den = torch.maximum((wgt * (k[:t + 1] @ q[t])).sum().abs(), torch.exp(-mt)) + 1e-6
        want[t] = num.sum(0) / den
    want = plain.rms_unit(want, 1e-6) * torch.sigmoid(h @ W["m.g"].T)
    assert torch.allclose(out, want, rtol=1e-9, atol=1e-12)
    # a window of w tokens sees exactly the token itself and the w - 1 before it
    am = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 50.0, "mask": {"size": 3}}
    W = {"a.q": torch.eye(2, D, dtype=torch.float64), "a.k": torch.eye(2, D, dtype=torch.float64), "a.v": torch.eye(2, D, dtype=torch.float64),
         "a.q.b": torch.zeros(2, dtype=torch.float64), "a.k.b": torch.zeros(2, dtype=torch.float64),
         "a.v.b": torch.zeros(2, dtype=torch.float64), "a.o": torch.eye(2, dtype=torch.float64)}
    hh = torch.zeros(6, D, dtype=torch.float64)
    hh[0, 0] = 9.0     # a key that every later query prefers while it is visible
    hh[1:, 0] = 1.0
    hh[1:, 1] = 0.1
    o = plain.window_attention(W, "a", am, hh)
    assert o[2, 0] > 8.9 and o[3, 0] < 1.01           # position 2 still sees position 0 (2 - 0 < 3), position 3 does not


LENGTHS = {"mix": (1, 2, 37, 70, 45, 19), "odd": (3, 90, 33, 16, 75), "plain": (44, 3, 21), "mlstm_only": (50,),
           "attention_only": (40,), "ssm_only": (50,), "moe_only": (30,)}


@pytest.mark.parametrize("name", list(LENGTHS))
def test_every_schedule_agrees_with_plain(name, tmp_path):
    case = Case(name, tmp_path, torch.float32, requests=LENGTHS[name])
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=30, max_tokens=128)
    for sched_name, steps in schedules(case).items():
        got, routed = run_steps(runner, cache, case, steps)
        compare(case, got, routed, *TOL, NEAR_TIE)
        assert cache.free_pages() == cache.total_pages() and cache.state_slots.free == cache.state_slots.total, sched_name


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_drawn_configurations(seed, tmp_path):
    from pozozen_cases import random_config, sharpen_mildly

    case = Case(f"drawn{seed}", tmp_path, torch.float32, raw=random_config(200 + seed), requests=(60, 1, 35), tweak=sharpen_mildly)
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=16, n_pages=12, max_tokens=64, max_seq=128)
    got, routed = run_steps(runner, cache, case, schedules(case)["mixed"])
    # deeper models than the fixed cases, and one position of one of them amplifies float32 rounding 100 times (with the
    # twins in float64 it agrees to 2e-5): the tolerances of the float32 kernels, the rows judged together
    compare_together(case, got, routed, 5e-5, 1e-5, NEAR_TIE)


def test_the_sharpened_weights_show_each_fault(tmp_path):
    """What the comparisons above rest on: with these weights a window one key too long or short, a lost state of
    either recurrence, lost inputs of the convolution, the correction, the groups, an identity expert taken for an
    ordinary one, the streams' mixing, a running maximum that starts elsewhere, and a far token each move the logits
    by far more than the tolerance."""
    case = Case("mix", tmp_path, torch.float32, requests=(60,))
    ref, _ = case.ref("r0")
    scale = float((ref - ref.mean(-1, keepdim=True)).abs().max())

    def moved(cfg=None, weights=None, toks=None, last=20):
        lg = plain.forward(weights or case.weights, cfg or case.cfg, toks or case.tokens["r0"])
        return float((lg[-last:] - ref[-last:]).abs().max()) / scale

    for delta in (-1, 1):
        cfg = copy.deepcopy(case.cfg)
        cfg["layers"][0]["mixer"]["left"]["mask"]["size"] += delta
        assert moved(cfg) > 100 * TOL[0]
    for key, value in ((("layers", 0, "mixer", "right", "conv"), None), (("layers", 0, "mlp", "router", "groups", "keep"), 4),
                       (("layers", 1, "mlp", "router", "groups", "keep"), 2), (("layers", 0, "mixer", "right", "groups"), 1),
                       (("layers", 0, "mixer", "right", "norm_groups"), 1), (("layers", 3, "mixer", "gate_cap"), 15.0),
                       (("loop", "times"), 2), (("streams",), 2)):
        cfg = copy.deepcopy(case.cfg)
        node = cfg
        for k in key[:-1]:
            node = node[k]
        w = dict(case.weights)
        if key[-1] == "conv":       # the convolution sees one token less: its first column is taken away
            node["conv"] = 2
            w["l0.mix.right.conv"] = w["l0.mix.right.conv"][:, 1:].contiguous()
        elif key[-1] == "groups" and key[-2] == "right":
            node["groups"] = 1      # both groups' heads read the first group's B and C
            n = cfg["layers"][0]["mixer"]["right"]["state"]
            inner = 4 * 8
            keep = list(range(2 * inner + n)) + list(range(2 * inner + 2 * n, 2 * inner + 3 * n)) + list(range(2 * inner + 4 * n, 2 * inner + 4 * n + 4))
            w["l0.mix.right.in"] = w["l0.mix.right.in"][keep].contiguous()
            ch = list(range(inner + n)) + list(range(inner + 2 * n, inner + 3 * n))
            w["l0.mix.right.conv"], w["l0.mix.right.conv.b"] = w["l0.mix.right.conv"][ch].contiguous(), w["l0.mix.right.conv.b"][ch].contiguous()
        elif key[-1] == "streams":
            node["streams"] = 2
            for n_ in list(w):
                if ".hc" in n_:
                    w[n_] = w[n_][:2, :2].contiguous() if n_.endswith(".mix") else w[n_][:2].contiguous()
        else:
            node[key[-1]] = value
        assert moved(cfg, w) > 100 * TOL[0], key
    for name in ("l0.mlp.correction", "l1.mlp.correction"):
        w = dict(case.weights)
        w[name] = torch.zeros_like(w[name])
        assert moved(weights=w) > 100 * TOL[0], name
    # identity experts taken for ordinary ones: the router's last outputs get experts of their own
    cfg = copy.deepcopy(case.cfg)
    cfg["layers"][1]["mlp"]["router"].update(experts=8, identity=0)
    w = dict(case.weights)
    for e in range(4, 8):
        for n_ in ("gate", "up", "down"):
            w[f"l1.mlp.e{e}.{n_}"] = w[f"l1.mlp.e{e - 4}.{n_}"]
    assert moved(cfg, w) > 100 * TOL[0]
    # lost states: a sequence that starts 25 tokens later has forgotten what came before
    lg = plain.forward(case.weights, case.cfg, case.tokens["r0"][25:])
    assert float((lg[-20:] - ref[-20:]).abs().max()) / scale > 100 * TOL[0]
    toks = list(case.tokens["r0"])
    toks[1] = (toks[1] + 1) % case.cfg["vocab"]     # a token 40 and more back: only the states and the full attention carry it
    assert moved(toks=toks) > 100 * TOL[0]


def test_far_tokens_reach_through_each_state_alone(tmp_path):
    """One-layer models: a token 45 positions back moves the last logits through the matrix memory alone and through
    the state-space recurrence alone (whose attention sees 4 tokens), and not through a window of 9 alone."""
    for name, reaches in (("mlstm_only", True), ("ssm_only", True), ("attention_only", False)):
        case = Case(name, tmp_path, torch.float32, requests=(50,))
        ref, _ = case.ref("r0")
        scale = float((ref - ref.mean(-1, keepdim=True)).abs().max())
        toks = list(case.tokens["r0"])
        toks[2] = (toks[2] + 1) % case.cfg["vocab"]
        lg = plain.forward(case.weights, case.cfg, toks)
        move = float((lg[-3:] - ref[-3:]).abs().max()) / scale
        assert (move > 100 * TOL[0]) == reaches, (name, move)


def test_window_pages_go_back_while_the_request_lives_and_slots_are_used_again(tmp_path):
    case = Case("attention_only", tmp_path, torch.float32, requests=(90, 90, 40, 40, 40))
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=14, max_tokens=72, slots=2)
    steps = [[("r0", 30)], [("r0", 30)], [("r0", 30)], [("r1", 24), ("r2", 8)], [("r1", 33), ("r2", 32)],
             [("r1", 33), ("r3", 2)], [("r3", 38), ("r4", 1)], [("r4", 39)]]
    got, routed = run_steps(runner, cache, case, steps)
    compare(case, got, routed, *TOL, NEAR_TIE)
    assert cache.free_pages() == cache.total_pages()
    # a request of 60 tokens holds, behind its last step, only the pages that its window of 9 still reaches
    from locus_b200.engine.step import StepEntry
    seq = cache.open("z")
    for a in (0, 20, 40):
        assert cache.ensure_capacity(seq, 20)
        runner.step([StepEntry(seq, case.tokens["r0"][a:a + 20], [19])])
    assert seq.pages_held(0) <= 3 < cache.pages_for(60)
    cache.release(seq)


def test_a_slot_used_again_starts_from_zero(tmp_path):
    """Two requests through the same state slot one after the other, and two side by side: the second one's states
    (matrix memory, running maximum, state-space matrix, the convolution's inputs) start at zero."""
    case = Case("plain", tmp_path, torch.float32, requests=(30, 30, 12))
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=16, max_tokens=64, slots=1)
    got, routed = run_steps(runner, cache, case, [[("r0", 30)], [("r1", 7)], [("r1", 23)], [("r2", 2)], [("r2", 10)]])
    compare(case, got, routed, *TOL, NEAR_TIE)


def test_greedy_generation_through_the_scheduler(tmp_path):
    from locus_b200.engine.engine import Engine
    from locus_b200.models import load_model

    case = Case("mix", tmp_path, torch.float32, requests=(9, 21, 3))
    m = load_model(case.dir, torch.float32, "cpu")
    eng = Engine.from_model(m, ctx=256, page_tokens=8, max_batch_tokens=16, chunk=8, max_running=2, use_graphs=False)
    prompts = [case.tokens[r] for r in ("r0", "r1", "r2")]
    outs = eng.generate(prompts, max_new_tokens=6)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = plain.forward(case.weights, case.cfg, seq)
            top2 = torch.topk(lg[-1], 2).values
            if float(top2[0] - top2[1]) > 1e-4 * float(lg[-1].abs().max()):
                assert int(torch.argmax(lg[-1])) == tok
            seq.append(tok)
    assert eng.cache.free_pages() == eng.cache.total_pages()
