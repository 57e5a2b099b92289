"""The Lalepel design through the engine's host logic on the CPU (the kernels replaced by their plain torch
twins): configuration and plan, weights by name, the cache's pages (a window's pages go back while a request
lives) and state slots (freed and used again), whole prompts, decoding token by token, portions down to two
tokens, mixed batches, and greedy generation through the scheduler -- all against the plain implementation,
which shares no code with any of it.  The kernels themselves are covered by the gpu tests."""
import copy
import math

import pytest
import torch

import emulated_kernels as EK
import plain_lalepel as plain
from lalepel_cases import CONFIGS, Case, compare, make_runner, run_steps, schedules, latent, with_mlp, model
import locus_b200.models  # noqa: F401  (registers the architectures)
from locus_b200.config import ConfigError, find_arch
from locus_b200.config.lalepel import LalepelConfig

TOL = (2e-5, 4e-6)   # max and mean |error| of the logits relative to the largest |logit|; float32 twins
NEAR_TIE = 2e-5


@pytest.fixture(autouse=True)
def _emulate(monkeypatch):
    EK.install(monkeypatch)


def test_config_reads_every_size_and_refuses_what_is_wrong():
    cfg = LalepelConfig.from_dict(copy.deepcopy(CONFIGS["mix"]))
    assert find_arch("Lalepel").parse_config is not None
    m0, m2 = cfg.layers[0].mixer, cfg.layers[2].mixer
    assert (m0.heads, m0.dim, m0.rot_dim, m0.vdim, m0.q_rank, m0.kv_rank, m0.window) == (3, 16, 8, 24, 40, 32, 12)
    assert m0.rot_scaling.factor == 4.0 and m2.rot_scaling is None and m2.window == 0 and m2.rot_dims == 8
    assert cfg.layers[1].mixer.decay == (0.9, 0.97) and cfg.layers[2].mlp is None
    assert cfg.layers[3].mlp.shared_ff == 0 and cfg.layers[0].mlp.shared_ff == 32
    for path, value, word in ((("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "decay"), [0.5], "decay"),
                              (("layers", 0, "mlp", "router", "top"), 7, "top"), (("norm",), None, "norm"),
                              (("layers", 0, "mixer", "rot", "dims"), 10, "rot.dims")):
        raw = copy.deepcopy(CONFIGS["mix"])
        node = raw
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            LalepelConfig.from_dict(raw)


def test_frequencies_of_the_ramp_against_the_plain_formula():
    from locus_b200.parts.position import Rotary

    for dims, base, sc in ((8, 10000.0, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}),
                           (32, 50000.0, {"factor": 16.0, "original": 1024, "fast": 24.0, "slow": 2.0}),
                           (6, 77.0, None)):
        r = Rotary("p", head_dim=dims, theta=base, rot_dim=dims, interleaved=True, scaling=sc)
        f, mag = plain.rotary_frequencies(dims, base, sc)
        assert torch.allclose(r.frequencies(), torch.tensor(f, dtype=torch.float64), rtol=1e-14, atol=0)
        assert math.isclose(r.magnitude(), mag, rel_tol=1e-15)
        if sc:
            assert f[0] == 1.0 and f[-1] < base ** (-2.0 * (dims // 2 - 1) / dims)  # the fast pair is left alone


def test_plain_retention_is_the_decayed_sum():
    """The oracle's recurrence against the closed form o_t = sum_j decay^(t-j) (q_t . k_j) v_j."""
    case_cfg = CONFIGS["retention_only"]["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(3)
    W = {f"m.{n}": torch.randn(r, 48, generator=g, dtype=torch.float64) * 0.2
         for n, r in (("q", 48), ("k", 48), ("v", 32), ("g", 32))}
    W["m.o"] = torch.eye(32, dtype=torch.float64)[:, :32].repeat(2, 1)[:48]
    h = torch.randn(9, 48, generator=g, dtype=torch.float64)
    out, S = plain.retention(h, W, "m", case_cfg, 1e-6)
    q = (h @ W["m.q"].T).view(9, 2, 24)
    k = (h @ W["m.k"].T).view(9, 2, 24) * 24 ** -0.5
    v = (h @ W["m.v"].T).view(9, 2, 16)
    o = torch.zeros(9, 2, 16, dtype=torch.float64)
    for t in range(9):
        for j in range(t + 1):
            for hh in range(2):
                o[t, hh] += case_cfg["decay"][hh] ** (t - j) * (q[t, hh] @ k[j, hh]) * v[j, hh]
    gate = h @ W["m.g"].T
    want = (plain.rms_unit(o, 1e-6).reshape(9, 32) * (gate / (1 + torch.exp(-gate)))) @ W["m.o"].T
    assert torch.allclose(out, want, rtol=1e-10, atol=1e-12)
    # a state handed on gives the same as one pass
    a, Sa = plain.retention(h[:4], W, "m", case_cfg, 1e-6)
    b, Sb = plain.retention(h[4:], W, "m", case_cfg, 1e-6, state=Sa)
    assert torch.allclose(torch.cat([a, b]), out, rtol=1e-10, atol=1e-12) and torch.allclose(Sb, S)


@pytest.mark.parametrize("name,lengths", [("mix", (1, 2, 37, 70, 45, 19)), ("odd", (3, 90, 33, 16, 75)),
                                          ("latent_only", (50,)), ("latent_full", (40,)), ("retention_only", (50,)),
                                          ("dense_only", (20,)), ("moe_only", (30,)), ("odd2", (44, 3, 21))])
def test_every_schedule_agrees_with_plain(name, lengths, tmp_path):
    case = Case(name, tmp_path, torch.float32, requests=lengths)
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=30, max_tokens=128)
    for sched_name, steps in schedules(case).items():
        got, routed = run_steps(runner, cache, case, steps)
        compare(case, got, routed, *TOL, NEAR_TIE)
        assert cache.free_pages() == cache.total_pages() and cache.state_slots.free == cache.state_slots.total, sched_name


def test_the_sharpened_weights_show_a_window_off_by_one_a_lost_sink_and_a_lost_state(tmp_path):
    """What the comparisons above rest on: with these weights a window one key too long or short, a sink left
    out, a state that is not carried, and a far key in a layer without a window each move the logits by far more
    than the tolerance."""
    case = Case("mix", tmp_path, torch.float32, requests=(60,))
    ref, _ = case.ref("r0")
    scale = float((ref - ref.mean(-1, keepdim=True)).abs().max())

    def moved(cfg=None, weights=None, toks=None):
        lg, _ = plain.forward(cfg or case.cfg, weights or case.weights, toks or case.tokens["r0"])
        return float((lg[-20:] - ref[-20:]).abs().max()) / scale

    for delta in (-1, 1):
        cfg = copy.deepcopy(case.cfg)
        cfg["layers"][0]["mixer"]["mask"]["size"] += delta
        assert moved(cfg) > 100 * TOL[0]
    w = dict(case.weights)
    w["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -30.0)
    assert moved(weights=w) > 100 * TOL[0]
    cfg = copy.deepcopy(case.cfg)
    cfg["layers"][1]["mixer"]["decay"] = [0.0, 0.0]
    assert moved(cfg) > 100 * TOL[0]
    toks = list(case.tokens["r0"])
    toks[1] = (toks[1] + 1) % case.cfg["vocab"]     # a key 40 and more tokens back (layer 2 has no window)
    assert moved(toks=toks) > 100 * TOL[0]


def test_window_pages_go_back_while_the_request_lives_and_slots_are_used_again(tmp_path):
    case = Case("latent_only", tmp_path, torch.float32, requests=(90, 90, 40, 40, 40))
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=14, max_tokens=72, slots=2)
    steps = [[("r0", 30)], [("r0", 30)], [("r0", 30)], [("r1", 24), ("r2", 8)], [("r1", 33), ("r2", 32)],
             [("r1", 33), ("r3", 2)], [("r3", 38), ("r4", 1)], [("r4", 39)]]
    got, routed = run_steps(runner, cache, case, steps)
    compare(case, got, routed, *TOL, NEAR_TIE)
    assert cache.free_pages() == cache.total_pages()
    # a request of 60 tokens holds, behind its last step, only the pages that its window of 20 still reaches
    from locus_b200.engine.step import StepEntry
    seq = cache.open("z")
    for a in (0, 20, 40):
        assert cache.ensure_capacity(seq, 20)
        runner.step([StepEntry(seq, case.tokens["r0"][a:a + 20], [19])])
    assert seq.pages_held(0) <= 4 < cache.pages_for(60)
    cache.release(seq)


def test_greedy_generation_through_the_scheduler(tmp_path):
    from locus_b200.engine.engine import Engine

    case = Case("mix", tmp_path, torch.float32, requests=(9, 21, 3))
    from locus_b200.models import load_model
    m = load_model(case.dir, torch.float32, "cpu")
    eng = Engine.from_model(m, ctx=256, page_tokens=8, max_batch_tokens=16, chunk=8, max_running=2, use_graphs=False)
    prompts = [case.tokens[r] for r in ("r0", "r1", "r2")]
    outs = eng.generate(prompts, max_new_tokens=6)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg, _ = plain.forward(case.cfg, case.weights, seq)
            top2 = torch.topk(lg[-1], 2).values
            if float(top2[0] - top2[1]) > 1e-4 * float(lg[-1].abs().max()):
                assert int(torch.argmax(lg[-1])) == tok
            seq.append(tok)
    assert eng.cache.free_pages() == eng.cache.total_pages()
