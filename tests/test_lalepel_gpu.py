"""The Lalepel design on the GPU against the plain implementation (float64), in float32 and in bfloat16:
each mechanism alone (one-layer models) and together, at sizes that are and are not multiples of 8; whole prompts,
decoding token by token, portions down to two tokens, mixed batches with pages and state slots that are used
again; keys just inside and just outside a window in prompts and while decoding; a far key in a layer without a
window; long decoding through CUDA graphs; other page sizes; the kernels alone against their plain twins; greedy
generation through the engine's entry point; trace replay as a program.  Pages are filled with NaN when they are
made and when they go back."""
import json
import os
import subprocess
import sys

import pytest
import torch

import emulated_kernels as EK
import plain_lalepel as plain
from lalepel_cases import Case, compare, make_runner, run_steps, schedules

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# max and mean |error| of the logits (their mean over the vocabulary taken off) relative to the largest |logit|
TOL = {torch.float32: (5e-5, 1e-5), torch.bfloat16: (3e-2, 5e-3)}
NEAR_TIE = {torch.float32: 2e-5, torch.bfloat16: 5e-2}   # of the spread of a token's router logits (measured: rounding the
# sublayers' inputs alone moves a logit by up to 1.5 % of the spread at width 128)
DTYPES = [torch.float32, torch.bfloat16]
LENGTHS = {"mix": (1, 2, 37, 70, 45, 19, 130), "odd": (3, 90, 33, 16, 75), "wide": (150, 40, 260),
           "latent_only": (50, 23), "latent_full": (80,), "retention_only": (70, 5), "dense_only": (20,),
           "moe_only": (40,), "no_router": (30,), "odd2": (44, 3, 21)}


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    made = {}

    def get(name, store=torch.bfloat16):
        key = (name, store)
        if key not in made:
            made[key] = Case(name, tmp_path_factory.mktemp("lalepel"), store, requests=LENGTHS[name])
        return made[key]

    return get


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(LENGTHS))
def test_every_schedule_agrees_with_plain(name, dtype, cases):
    case = cases(name)
    runner, cache = make_runner(case, dtype, "cuda:0", page_tokens=16, n_pages=40, max_tokens=320)
    for sched_name, steps in schedules(case).items():
        got, routed = run_steps(runner, cache, case, steps)
        compare(case, got, routed, *TOL[dtype], NEAR_TIE[dtype])
        assert cache.free_pages() == cache.total_pages() and cache.state_slots.free == cache.state_slots.total, sched_name


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("page_tokens", [8, 64])
def test_other_page_sizes_and_the_cuda_core_products(page_tokens, dtype, cases, monkeypatch):
    import locus_b200.kernels as K

    case = cases("mix")
    if page_tokens == 8:
        monkeypatch.setattr(K, "USE_TENSOR_CORES", False)   # bfloat16 on the CUDA-core products, 64-row head tiles
    runner, cache = make_runner(case, dtype, "cuda:0", page_tokens=page_tokens, n_pages=24 if page_tokens == 64 else 70,
                                max_tokens=320, max_seq=1024)
    sch = schedules(case)
    for steps in (sch["mixed"], sch["chunked"]):
        got, routed = run_steps(runner, cache, case, steps)
        compare(case, got, routed, *TOL[dtype], NEAR_TIE[dtype])


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_window_edges_in_prompts_and_in_decoding(dtype, tmp_path_factory):
    """A token that the rest of the sequence attends to strongly sits just inside the window of one query and just
    outside the next one's: the two logit rows must differ as the oracle's do.  The marker's key is made to stand out
    by scaling its embedding; the probes are the positions around marker + window, once inside a prompt's portion
    and once decoded one by one."""
    def tweak(name, w):
        from lalepel_cases import sharpen
        sharpen(name, w)
        w["embed"][7] = w["embed"][7] * 6.0

    case = Case("latent_only", tmp_path_factory.mktemp("edge"), torch.bfloat16, requests=(64, 64), tweak=tweak)
    window = case.cfg["layers"][0]["mixer"]["mask"]["size"]
    for rid in case.tokens:
        t = [x if x != 7 else 8 for x in case.tokens[rid]]
        t[30] = 7
        case.tokens[rid] = t
    ref, _ = case.ref("r0")
    inside, outside = 30 + window - 1, 30 + window
    top = float(ref.abs().max())
    # the oracle itself tells the two positions apart by much more than the tolerance (else the test shows nothing)
    cfg_longer = json.loads(json.dumps(case.cfg))
    cfg_longer["layers"][0]["mixer"]["mask"]["size"] = window + 1
    longer, _ = plain.forward(cfg_longer, case.weights, case.tokens["r0"])
    assert float((longer[outside] - ref[outside]).abs().max()) > 20 * TOL[torch.float32][0] * top
    runner, cache = make_runner(case, dtype, "cuda:0", page_tokens=16, n_pages=16, max_tokens=128)
    steps = [[("r0", 45), ("r1", inside - 2)]] + [[("r0", 19), ("r1", 1)]] + [[("r1", 1)]] * 5 + [[("r1", 64 - inside - 4)]]
    got, routed = run_steps(runner, cache, case, steps)
    compare(case, got, routed, *TOL[dtype], NEAR_TIE[dtype])


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_long_decoding_through_graphs_keeps_state_and_window(dtype, cases):
    """300 tokens decoded one by one for two requests side by side, replayed from CUDA graphs: the retention state
    is carried in its slot, the window's pages go back, the far keys of the layer without a window stay."""
    from lalepel_cases import tokens as draw

    case = cases("no_router")   # (an observer of the router's picks would copy to the host inside the capture)
    case.tokens["long0"] = draw(20 + 290, case.cfg["vocab"], 77)
    case.tokens["long1"] = draw(3 + 290, case.cfg["vocab"], 78)
    runner, cache = make_runner(case, dtype, "cuda:0", page_tokens=16, n_pages=60, max_tokens=64, use_graphs=True)
    steps = [[("long0", 20), ("long1", 3)]] + [[("long0", 1), ("long1", 1)]] * 290
    try:
        got, routed = run_steps(runner, cache, case, steps)
        assert runner.stats["graph_replays"] > 200
        compare(case, {r: got[r] for r in ("long0", "long1")}, routed, *TOL[dtype], NEAR_TIE[dtype])
    finally:
        del case.tokens["long0"], case.tokens["long1"]


def _rand(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("kv_rank,rot_dim,heads,window", [(32, 8, 3, 12), (28, 6, 1, 0), (128, 32, 4, 100), (512, 64, 2, 0),
                                                          (64, 16, 5, 37), (32, 0, 1, 7), (256, 48, 20, 33)])
def test_latent_attention_kernel_against_its_twin(kv_rank, rot_dim, heads, window, dtype):
    """latent_attn alone at several sizes, segments of one token and of many behind contexts that straddle pages,
    against the plain twin in float64."""
    import locus_b200.kernels as K

    P, R = 16, kv_rank + rot_dim
    segs = [(0, 37), (90, 1), (33, 20), (15, 1), (200, 17)]      # (cached tokens, new tokens)
    T = sum(n for _, n in segs)
    n_pages = sum(-(-(c + n) // P) for c, n in segs)
    pool = _rand((n_pages, 1, 1, P, R), 1, 0.7, dtype)
    table = torch.full((len(segs), 16), -1, dtype=torch.int32)
    page = 0
    for s, (c, n) in enumerate(segs):
        for i in range(-(-(c + n) // P)):
            table[s, i] = page
            page += 1
    q0 = [sum(n for _, n in segs[:i]) for i in range(len(segs))]
    dev = lambda v: torch.tensor(v, dtype=torch.int32).cuda()  # noqa: E731
    seg_q0, seg_qn, seg_ctx = dev(q0), dev([n for _, n in segs]), dev([c for c, _ in segs])
    items = dev([[s, a] for s, (c, n) in enumerate(segs) for a in range(0, n, K.LATENT_QUERY_TILE)])
    q_abs, q_rot = _rand((heads * T, kv_rank), 2, 0.5, dtype), _rand((T, heads * rot_dim), 3, 0.5, dtype)
    sink = _rand((heads,), 4, 1.0)
    out = torch.zeros(heads * T, kv_rank, dtype=dtype, device="cuda")
    kw = dict(seg_q0=seg_q0, seg_qn=seg_qn, seg_ctx=seg_ctx, block_table=table.cuda(), items=items, n_items=items.shape[0],
              n_tokens=T, n_heads=heads, kv_rank=kv_rank, rot_dim=rot_dim, page_tokens=P, window=window, scale=0.3)
    K.latent_attn(q_abs, q_rot, pool, sink, out, **kw)
    EK.PRECISE = True
    try:
        want = torch.zeros(heads * T, kv_rank, dtype=torch.float64)
        cpu = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in kw.items()}
        EK.latent_attn(q_abs.cpu(), q_rot.cpu(), pool.cpu(), sink.cpu(), want, **cpu)
    finally:
        EK.PRECISE = False
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert float((out.cpu().double() - want).abs().max()) <= tol * float(want.abs().max())
    if K.latent_attn_mma_takes(dtype, kv_rank, rot_dim):
        # the tensor-core kernel: its own query tiles (a block's 64 rows are queries x heads)
        shift = K.latent_mma_head_shift(heads)
        items = dev([[s, a] for s, (c, n) in enumerate(segs) for a in range(0, n, 64 >> shift)])
        out2 = torch.zeros(heads * T, kv_rank, dtype=dtype, device="cuda")
        K.latent_attn_mma(q_abs, q_rot, pool, sink, out2, head_shift=shift, **dict(kw, items=items, n_items=items.shape[0]))
        assert float((out2.cpu().double() - want).abs().max()) <= 1.5e-2 * float(want.abs().max())
        K.latent_attn_mma(q_abs, q_rot, pool, None, out2, head_shift=shift, **dict(kw, items=items, n_items=items.shape[0]))
        K.latent_attn(q_abs, q_rot, pool, None, out, **kw)
        assert float((out2.double() - out.double()).abs().max()) <= 1.5e-2 * float(out.double().abs().max())
        # the keys cut into ranges (more ranges than some items have tiles), with and without the sink
        units = items.shape[0] * (-(-heads // (1 << shift))) * 5
        part_o, part_ml = torch.zeros(units * 64 * kv_rank, device="cuda"), torch.zeros(units * 128, device="cuda")
        for sk, ref in ((sink, want), (None, out.cpu().double())):
            for n_splits in (2, 5):
                out3 = torch.zeros(heads * T, kv_rank, dtype=dtype, device="cuda")
                K.latent_attn_mma(q_abs, q_rot, pool, sk, out3, head_shift=shift, n_splits=n_splits, part_o=part_o,
                                  part_ml=part_ml, **dict(kw, items=items, n_items=items.shape[0]))
                assert float((out3.cpu().double() - ref).abs().max()) <= 1.5e-2 * float(ref.abs().max()), n_splits


@pytest.mark.parametrize("heads,dim,v_dim", [(2, 16, 8), (3, 12, 10), (1, 72, 40), (2, 256, 33)])
def test_retention_kernels_against_their_twins(heads, dim, v_dim):
    """The scan over segments of unequal length from states that are not zero, cut in two launches (the state
    handed on through its slot), and the gate-norm, against the plain twins in float64."""
    import locus_b200.kernels as K

    width = 2 * heads * dim + 2 * heads * v_dim
    segs = [19, 1, 40, 2]
    T = sum(segs)
    qkvg = _rand((T, width), 5, 0.6)
    decay = torch.tensor([0.9, 0.999, 1.0][:heads], dtype=torch.float32).cuda()
    slots = torch.tensor([2, 0, 3, 1], dtype=torch.int32).cuda()
    state0 = _rand((4, heads, dim, v_dim), 6, 0.3)
    q0 = torch.tensor([0, 19, 20, 60], dtype=torch.int32).cuda()
    qn = torch.tensor(segs, dtype=torch.int32).cuda()
    state, o_raw = state0.clone(), torch.zeros(T, heads * v_dim, device="cuda")
    K.retention_scan(qkvg, state, slots, q0, qn, 4, decay, dim ** -0.5, o_raw, n_heads=heads, dim=dim, v_dim=v_dim)
    EK.PRECISE = True
    try:
        st_w, o_w = state0.cpu().double(), torch.zeros(T, heads * v_dim, dtype=torch.float64)
        EK.retention_scan(qkvg.cpu(), st_w, slots.cpu(), q0.cpu(), qn.cpu(), 4, decay.cpu(), dim ** -0.5, o_w,
                          n_heads=heads, dim=dim, v_dim=v_dim)
        out_w = torch.zeros(T, heads * v_dim, dtype=torch.float64)
        EK.retention_gate_norm(o_w, qkvg.cpu(), 2 * heads * dim + heads * v_dim, 1e-5, out_w, n_heads=heads, v_dim=v_dim)
    finally:
        EK.PRECISE = False
    assert float((o_raw.cpu().double() - o_w).abs().max()) <= 2e-5 * float(o_w.abs().max())
    assert float((state.cpu().double() - st_w).abs().max()) <= 2e-5 * float(st_w.abs().max())
    # the same tokens in two launches: the first halves of the segments, then the rest
    state2, o2 = state0.clone(), torch.zeros(T, heads * v_dim, device="cuda")
    first = [n // 2 for n in segs]
    K.retention_scan(qkvg, state2, slots, q0, torch.tensor(first, dtype=torch.int32).cuda(), 4, decay, dim ** -0.5, o2,
                     n_heads=heads, dim=dim, v_dim=v_dim)
    q0b = torch.tensor([a + f for a, f in zip([0, 19, 20, 60], first)], dtype=torch.int32).cuda()
    K.retention_scan(qkvg, state2, slots, q0b, torch.tensor([n - f for n, f in zip(segs, first)], dtype=torch.int32).cuda(),
                     4, decay, dim ** -0.5, o2, n_heads=heads, dim=dim, v_dim=v_dim)
    # (a half may be short enough for the token-by-token kernel where the whole went chunk by chunk: rounding only)
    assert float((o2 - o_raw).abs().max()) <= 2e-5 * float(o_raw.abs().max())
    assert float((state2 - state).abs().max()) <= 2e-5 * float(state.abs().max())
    for odt in DTYPES:
        out = torch.zeros(T, heads * v_dim, dtype=odt, device="cuda")
        K.retention_gate_norm(o_raw, qkvg, 2 * heads * dim + heads * v_dim, 1e-5, out, n_heads=heads, v_dim=v_dim)
        tol = 2e-5 if odt == torch.float32 else 1e-2
        assert float((out.cpu().double() - out_w).abs().max()) <= tol * float(out_w.abs().max())


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_squared_relu_products_and_the_output_norm(dtype):
    """The squared-ReLU epilogue on every product kernel (row counts that pick each of them) and x += norm(y)."""
    import locus_b200.kernels as K

    for M, N, Kd in ((3, 40, 64), (12, 96, 64), (200, 136, 128), (70, 52, 36)):
        x, w = _rand((M, Kd), 7, 1.0, dtype), _rand((N, Kd), 8, 0.2, dtype)
        out = torch.zeros(M, N, dtype=dtype, device="cuda")
        K.linear(x, w, out, act="relu2")
        want = torch.clamp(x.double() @ w.double().T, min=0) ** 2
        tol = 2e-5 if dtype == torch.float32 else 1.5e-2
        assert float((out.double() - want).abs().max()) <= tol * float(want.abs().max()), (M, N, Kd)
    y, x0, w = _rand((33, 52), 9, 3.0), _rand((33, 52), 10, 1.0), _rand((52,), 11, 1.0, dtype)
    x = x0.clone()
    K.rmsnorm_add(y, w, 1e-5, x)
    want = x0.double() + plain.rmsnorm(y.double(), w.double(), 1e-5)
    assert float((x.double() - want).abs().max()) <= 1e-5 * float(want.abs().max())
    h = torch.zeros(33, 52, dtype=dtype, device="cuda")
    K.cast_rows(x0, h)
    assert torch.equal(h, x0.to(dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_greedy_generation_through_the_entry_point(dtype, cases):
    from locus_b200.engine.engine import Engine

    case = cases("mix")
    eng = Engine.from_model_dir(case.dir, dtype="float32" if dtype == torch.float32 else "bfloat16", ctx=512,
                                page_tokens=16, max_batch_tokens=64, chunk=32, max_running=3)
    prompts = [case.tokens[r] for r in ("r2", "r3", "r5", "r1")]
    outs = eng.generate(prompts, max_new_tokens=12)
    gap = 1e-3 if dtype == torch.float32 else 5e-2
    for p, o in zip(prompts, outs):
        seq = list(p)
        assert len(o) == 12
        for tok in o:
            lg, _ = plain.forward(case.cfg, case.weights, seq)
            top2 = torch.topk(lg[-1], 2).values
            if float(top2[0] - top2[1]) > gap * float(lg[-1].abs().max()):
                assert int(torch.argmax(lg[-1])) == tok
            seq.append(tok)
    assert eng.cache.free_pages() == eng.cache.total_pages()


def test_trace_replay_as_a_program(cases, tmp_path):
    """bin/trace_run on a model folder of this design: portions beside single tokens with four live requests and a
    pool that only holds them when pages are used again; logits against the oracle."""
    case = cases("mix")
    steps = schedules(case)["mixed"]
    fed, lines, want_rows = {}, [], []
    for n, step in enumerate(steps):
        entries, end = [], []
        for rid, k in step:
            a = fed.get(rid, 0)
            entries.append({"id": rid, "tokens": case.tokens[rid][a:a + k], "want": [k - 1]})
            want_rows.append((n, rid, a + k - 1))
            fed[rid] = a + k
            if fed[rid] == len(case.tokens[rid]):
                end.append(rid)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", case.dir, "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "320", "--page-tokens", "16"],
                           input="\n".join(lines) + "\n", text=True, capture_output=True, timeout=900)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {n}" for n in range(len(steps))]
        tol = TOL[torch.float32 if dtype == "float32" else torch.bfloat16][0]
        V, at = case.cfg["vocab"], {}
        for n, rid, pos in want_rows:
            rows = torch.from_file(str(out / f"{n}.f32"), size=os.path.getsize(out / f"{n}.f32") // 4,
                                   dtype=torch.float32).view(-1, V).double()
            i = at.get(n, 0)
            at[n] = i + 1
            ref = case.ref(rid)[0][pos]
            d = rows[i] - ref
            # a near-tie of the router may go either way here; such rows are judged in the schedule tests above
            if float((d - d.mean()).abs().max()) > tol * float(ref.abs().max()) and dtype == "float32":
                raise AssertionError(f"step {n} {rid} position {pos}: off by {float((d - d.mean()).abs().max()):.2e}")


def test_the_command_line_generates_from_a_folder_of_this_design(cases):
    """bin/locus-run: the architecture is found by config.json, the weights by name, and greedy generation gives the
    oracle's tokens (where its two best logits are not a near-tie)."""
    case = cases("no_router")
    prompt = case.tokens["r0"][:12]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "locus-run"), case.dir, ",".join(map(str, prompt)), "8",
                        "--dtype", "float32", "--page-tokens", "16", "--ctx", "128"], capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(x) for x in p.stdout.replace(",", " ").split() if x.lstrip("-").isdigit()]
    assert len(out) >= 8
    seq = list(prompt)
    for tok in out[-8:]:
        lg, _ = plain.forward(case.cfg, case.weights, seq)
        top2 = torch.topk(lg[-1], 2).values
        if float(top2[0] - top2[1]) > 1e-3 * float(lg[-1].abs().max()):
            assert int(torch.argmax(lg[-1])) == tok
        seq.append(tok)
    archs = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "locus-run"), "--archs"], capture_output=True, text=True)
    assert "Lalepel" in archs.stdout
