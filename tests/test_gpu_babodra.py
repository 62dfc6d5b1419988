"""Babodra on the GPU against the plain restatement of tests/babodra_oracle.py: every mechanism alone, prompts against
token-by-token decoding, portions down to two tokens, mixed batches, re-used pages, far keys and page borders, the first
tokens of a sequence, long decoding, sizes where head counts / groups collapse to 1, and greedy generation."""
import copy
import ctypes as C

import pytest
import torch

import babodra_oracle as O

pytestmark = pytest.mark.gpu

TOL32, TOL16 = 2e-4, 5e-2


def make(cfg=None, seed=0, dtype="float32", edit=None, **kw):
    from proxy_inference_engine_b200.babodra import BabodraArgs, BabodraModel, random_weights
    cfg = copy.deepcopy(cfg) if cfg else O.random_config(**kw)
    args = BabodraArgs.from_dict(cfg)
    w = random_weights(args, seed=seed)
    for name, fn in (edit or {}).items():
        w[name] = fn(w[name].float()).to(torch.bfloat16)
    return cfg, w, BabodraModel(args, w, "cuda", dtype)


def engine(model, max_tokens=1024, max_seqs=4, graph=True):
    from proxy_inference_engine_b200.engine import HybridEngine
    return HybridEngine(model, max_tokens, max_seqs, use_graph=graph)


def toks(n, vocab=96, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def err(got, want):
    got, want = got.double().cpu(), want.double()
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)).max())


def rows_err(got, want):
    got, want = got.double().cpu(), want.double()
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)


def ok16(got, want, margins):
    """bf16 against the restatement when the model routes: a token whose routing margin is within rounding may take
    another expert than the restatement did (and nudges the tokens that attend to it), so rows with a tiny margin are
    left out, nine rows in ten must be within TOL16 and no other row may be off by more than four times that."""
    e = rows_err(got, want)
    keep = torch.stack(margins).min(0).values > 0.02 if margins else torch.ones_like(e, dtype=torch.bool)
    e = e[keep[-len(e):]]
    return float(e.quantile(0.9)) < TOL16 and float(e.max()) < 4 * TOL16


def oracle16(cfg, w, ids):
    mg = []
    return O.forward(cfg, w, ids, rnd=O.bf16_round, margins=mg), mg


def whole(eng, ids, sid="w"):
    out = eng.forward([(sid, ids, list(range(len(ids))))])
    eng.finish(sid)
    return out


def lib():
    from proxy_inference_engine_b200 import _lib
    return _lib.load_hybrid(build_if_missing=True)


p_ = lambda t: None if t is None else C.c_void_p(t.data_ptr())


# ---- mechanisms alone -------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kinds", [[None], ["dense"], ["moe"], ["moe", "dense", None, "moe"]],
                         ids=["attention", "dense", "moe", "stack"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_match_the_oracle(kinds, dtype):
    cfg, w, model = make(dtype=dtype, kinds=kinds, n_layers=len(kinds))
    ids = toks(41)
    trace, want_layers = [], []
    got = engine(model).forward([("a", ids, list(range(len(ids))))], trace=trace)
    mg = []
    want = O.forward(cfg, w, ids, layers_out=want_layers, rnd=O.ident if dtype == "float32" else O.bf16_round, margins=mg)
    if dtype == "float32":
        for i, t in enumerate(trace):
            assert err(t, want_layers[i]) < TOL32, f"residual after layer {i}"
        assert err(got, want) < TOL32
    else:
        for i, t in enumerate(trace):
            assert ok16(t, want_layers[i], mg), f"residual after layer {i}"
        assert ok16(got, want, mg)


def test_gated_pair_epilogue_in_every_linear_kernel():
    """pieh_linear_glu over interleaved rows: few rows, tiles, ragged edges, the tensor-core path; clamped and plain."""
    from proxy_inference_engine_b200.babodra import interleave_pairs
    L = lib()
    g = torch.Generator().manual_seed(0)
    for M, ff, K in [(1, 48, 64), (3, 25, 200), (9, 64, 72), (70, 50, 99), (200, 160, 256), (130, 96, 128)]:
        for exact in (True, False):
            for alpha, limit, off in ((1.702, 0.9, 1.0), (1.0, 0.0, 0.0)):
                x = torch.randn((M, K), generator=g)
                wg, wu = [(2 * torch.randn((ff, K), generator=g) / K ** 0.5).to(torch.bfloat16) for _ in range(2)]
                wd = interleave_pairs(wg, wu)
                wd = wd.float().cuda() if exact else wd.cuda()
                xd = x.cuda() if exact else x.to(torch.bfloat16).cuda()
                out = torch.empty((M, ff), dtype=torch.float32, device="cuda")
                code = 1 if exact else 0
                assert L.pieh_linear_glu(p_(out), 1, ff, p_(xd), code, K, p_(wd), code, M, 2 * ff, K, alpha, limit, off, None) == 0
                xr = xd.double().cpu()
                gg, uu = xr @ wg.double().T, xr @ wu.double().T
                if limit > 0:
                    gg, uu = gg.clamp(max=limit), uu.clamp(-limit, limit)
                want = gg * torch.sigmoid(alpha * gg) * (uu + off)
                assert err(out, want) < 1e-5, (M, ff, K, exact, alpha)


def test_router_sized_products():
    """pieh_linear with many rows and a handful of outputs (the kernel with a warp per row), both precisions, with bias."""
    L = lib()
    g = torch.Generator().manual_seed(5)
    for M, N, K in [(100, 17, 256), (70, 7, 64), (40, 32, 200), (33, 1, 72), (4096, 9, 128)]:
        for exact in (True, False):
            x = torch.randn((M, K), generator=g)
            wt = (torch.randn((N, K), generator=g) / K ** 0.5).to(torch.bfloat16)
            bias = torch.randn((N,), generator=g).cuda()
            code, dt = (1, torch.float32) if exact else (0, torch.bfloat16)
            xd, wd = x.to(dt).cuda(), wt.to(dt).cuda()
            out = torch.empty((M, N), dtype=torch.float32, device="cuda")
            assert L.pieh_linear(p_(out), 1, N, p_(xd), code, K, p_(wd), code, p_(bias), M, N, K, 0, 0.0, None, None, 0, None) == 0
            assert err(out, xd.double().cpu() @ wt.double().T + bias.double().cpu()) < 1e-5, (M, N, K, exact)


@pytest.mark.parametrize("E,top,groups,keep", [(6, 2, 3, 2), (8, 4, 2, 1), (5, 1, 1, 1), (4, 4, 4, 4), (12, 3, 6, 2), (64, 6, 8, 3)])
def test_routing_alone(E, top, groups, keep):
    """pieh_moe_route against the restatement: choices, weights, and a plan whose slots are a permutation sorted by expert."""
    from proxy_inference_engine_b200._lib import HybMoePlan
    L = lib()
    T = 77
    g = torch.Generator().manual_seed(E)
    z = 3 * torch.randn((T, E + 1), generator=g)
    r = {"experts": E, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}
    s = torch.sigmoid(z[:, :E].double())
    idx, wt = O.route(z[:, :E].double(), torch.eye(E, dtype=torch.float64), r)     # router weight = identity: logits = z
    P = T * top
    i32 = lambda n: torch.zeros((n,), dtype=torch.int32, device="cuda")
    bufs = [i32(P), i32(P), i32(P), torch.zeros((P,), device="cuda"), i32(1 + 3 * (P // 64 + E)), i32(1 + 3 * (P // 128 + E))]
    counters = i32(2 * E + 2)
    plan = HybMoePlan(E, top, groups, keep, 2.5, *[b.data_ptr() for b in bufs], counters.data_ptr())
    zd = z.cuda()
    for _ in range(2):          # twice: the counters must come back to zero
        assert L.pieh_moe_route(p_(zd), E + 1, C.byref(plan), T, None) == 0
    slot_row, slot_expert, pair_slot, pair_w, t64, t128 = [b.cpu() for b in bufs]
    got_e = slot_expert[pair_slot.long()].view(T, top)
    assert sorted(pair_slot.tolist()) == list(range(P))
    assert torch.equal(slot_row[pair_slot.long()].view(T, top), torch.arange(T, dtype=torch.int32)[:, None].expand(T, top))
    assert torch.equal(got_e.sort(-1).values.long(), idx.sort(-1).values)
    assert torch.allclose(pair_w.view(T, top).double(), s.gather(1, got_e.long()) * 2.5, rtol=1e-5)
    assert slot_expert.tolist() == sorted(slot_expert.tolist())
    for tiles, rows in ((t64, 64), (t128, 128)):
        covered = []
        for k in range(int(tiles[0])):
            e, first, n = tiles[1 + 3 * k: 4 + 3 * k].tolist()
            assert 0 < n <= rows and set(slot_expert[first: first + n].tolist()) == {e}
            covered += list(range(first, first + n))
        assert covered == list(range(P))
    assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("T,E,top,K,ff", [(5, 4, 2, 64, 24), (16, 8, 2, 200, 33), (70, 6, 2, 72, 40), (300, 4, 2, 128, 96),
                                          (513, 16, 4, 64, 64)], ids=["few-slots", "few-slots-odd", "tiles", "tensor-core", "many-experts"])
@pytest.mark.parametrize("exact", [True, False], ids=["float32", "bfloat16"])
def test_grouped_products_alone(T, E, top, K, ff, exact):
    """pieh_moe_linear over a routed plan: the gathered gate / up product with the silu pair, then the down product per
    slot, against a loop over tokens and their experts."""
    from proxy_inference_engine_b200._lib import HybMoePlan
    from proxy_inference_engine_b200.babodra import interleave_pairs
    L = lib()
    g = torch.Generator().manual_seed(T)
    z = 2 * torch.randn((T, E), generator=g)
    x = torch.randn((T, K), generator=g)
    wg, wu = [(2 * torch.randn((E, ff, K), generator=g) / K ** 0.5).to(torch.bfloat16) for _ in range(2)]
    wdn = (torch.randn((E, K, ff), generator=g) / ff ** 0.5).to(torch.bfloat16)
    P = T * top
    i32 = lambda n: torch.zeros((n,), dtype=torch.int32, device="cuda")
    bufs = [i32(P), i32(P), i32(P), torch.zeros((P,), device="cuda"), i32(1 + 3 * (P // 64 + E)), i32(1 + 3 * (P // 128 + E))]
    counters = i32(2 * E + 2)
    plan = HybMoePlan(E, top, 1, 1, 1.0, *[b.data_ptr() for b in bufs], counters.data_ptr())
    zd = z.cuda()
    assert L.pieh_moe_route(p_(zd), E, C.byref(plan), T, None) == 0
    code, dt = (1, torch.float32) if exact else (0, torch.bfloat16)
    xd = x.to(dt).cuda()
    gu = torch.stack([interleave_pairs(wg[e], wu[e]) for e in range(E)]).to(dt).cuda().contiguous()
    dn = wdn.to(dt).cuda().contiguous()
    hid = torch.empty((P, ff), dtype=dt, device="cuda")
    assert L.pieh_moe_linear(p_(hid), code, ff, p_(xd), code, K, p_(gu), code, 2 * ff * K, P, 2 * ff, K, 1, 1, 1.0, 0.0, 0.0,
                             C.byref(plan), None) == 0
    ys = torch.empty((P, K), dtype=torch.float32, device="cuda")
    assert L.pieh_moe_linear(p_(ys), 1, K, p_(hid), code, ff, p_(dn), code, K * ff, P, K, ff, 0, 0, 1.0, 0.0, 0.0,
                             C.byref(plan), None) == 0
    torch.cuda.synchronize()
    assert L.pieh_pipeline_error() == 0
    slot_row, slot_expert = bufs[0].cpu().long(), bufs[1].cpu().long()
    xr = xd.double().cpu()
    want_h = torch.stack([O.lin(xr[slot_row[s]], wg[slot_expert[s]].double()) for s in range(P)])
    want_h = want_h * torch.sigmoid(want_h) * torch.stack([O.lin(xr[slot_row[s]], wu[slot_expert[s]].double()) for s in range(P)])
    assert err(hid, want_h) < (1e-5 if exact else 1e-2)
    want_y = torch.stack([O.lin(hid[s].double().cpu(), wdn[slot_expert[s]].double()) for s in range(P)])
    assert err(ys, want_y) < 1e-5


def test_distance_bias_and_sink_show_in_one_head():
    """One query is made to match one far key strongly: the output then depends on the exact distance term and on the
    sink's share, which random weights would drown among hundreds of keys."""
    cfg, w, model = make(kinds=[None], n_layers=1, heads=4, kv_heads=4, dim=16, width=64, scale=2.0,
                         edit={"l0.mix.q.norm": lambda t: t * 2, "l0.mix.k.norm": lambda t: t * 2})
    ids = toks(300)
    assert err(whole(engine(model), ids), O.forward(cfg, w, ids)) < TOL32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_planted_far_keys_in_the_attention_operator(dtype):
    """pieh_bias_attn_prepare / _run on given projections, no norms: chosen queries are made to match ONE far key (the
    first position, the last and first slot of a page, the key just before the query), so every output row is that key's
    value times a weight set by the exact distance term and the sink.  Scattered pages; the prompt in portions and single
    rows, which takes the tile kernel (bf16), the row kernel and its cluster form through the same positions."""
    from proxy_inference_engine_b200._lib import HybBiasAttn
    from proxy_inference_engine_b200.ragged import BatchDetails
    L = lib()
    H, G, d, T, scale = 4, 2, 64, 450, 0.125
    g = torch.Generator().manual_seed(11)
    q, k = 0.3 * torch.randn((T, H, d), generator=g), torch.randn((T, G, d), generator=g)
    v, gate = torch.randn((T, G, d), generator=g), torch.randn((T, H * d), generator=g)
    plant = {449: 0, 448: 63, 447: 64, 446: 127, 445: 128, 444: 443, 300: 1, 200: 199, 129: 128, 128: 127, 65: 64, 64: 0}
    for i, j in plant.items():
        for h in range(H):
            kj = k[j, h // (H // G)]
            q[i, h] = (6.0 + 2.0 * h) / scale * kj / kj.norm() ** 2      # score 6 + 2 h before the distance term
    exact = dtype == "float32"
    rnd = O.ident if exact else O.bf16_round
    slopes = O.head_slopes(H)
    want = O.sink_attention(rnd(q.double()), rnd(k.double()), rnd(v.double()), scale, slopes, H // G)
    want = want.reshape(T, H * d) * torch.sigmoid(gate.double())
    # the restatement itself must rest on the planted key: row 449 of the flattest head is mostly the value at position 0
    flat = want.view(T, H, d)[449, H - 1] / torch.sigmoid(gate.double()).view(T, H, d)[449, H - 1]
    v0 = rnd(v.double())[0, G - 1]
    assert float((flat @ v0) / (v0 @ v0)) > 0.5
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gate], 1).cuda().contiguous()
    ld = proj.shape[1]
    code, dt = (1, torch.float32) if exact else (0, torch.bfloat16)
    pages = [5, 2, 7, 0, 3, 1, 6, 4]
    kp = torch.zeros((8, 64, G, d), dtype=dt, device="cuda")
    vp = torch.zeros_like(kp)
    sl = slopes.float().cuda()
    at = HybBiasAttn(H, G, d, d, H * d, H * d + G * d, H * d + 2 * G * d, None, None, 1e-5, scale, 0.0, 0.0, p_(sl), 1, 0,
                     p_(kp), p_(vp), code)
    got, ctx = [], 0
    for n in [200, 3] + [1] * 12 + [229] + [1] * 6:
        batch = BatchDetails.build([("s", [0] * n, ctx, pages)], device="cuda")
        desc, keep = batch.hybrid_descriptor()
        rows = proj[ctx: ctx + n]
        qo = torch.empty((n, H * d), dtype=torch.float32, device="cuda")
        out = torch.empty((n, H * d), dtype=dt, device="cuda")
        assert L.pieh_bias_attn_prepare(p_(qo), p_(rows), ld, C.byref(at), C.byref(desc), None) == 0
        assert L.pieh_bias_attn_run(p_(out), code, p_(qo), p_(rows), ld, C.byref(at), C.byref(desc), None) == 0
        torch.cuda.synchronize()
        got.append(out.float())
        ctx += n
    got = torch.cat(got).double().cpu()
    assert ctx == T
    tol = 1e-5 if exact else 2e-2
    for i in plant:
        assert float((got[i] - want[i]).abs().max()) < tol * float(want[i].abs().max()), i
    assert float((got - want).abs().max()) < tol * float(want.abs().max())


# ---- schedules --------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_against_token_by_token_decoding(dtype):
    cfg, w, model = make(dtype=dtype)
    ids = toks(150)
    eng = engine(model)
    got = [eng.forward([("s", ids[:70], list(range(70)))])]
    for t in range(70, 150):                   # crosses the page borders at 128 and the temperature steps at 24 k - 1
        got.append(eng.forward([("s", [ids[t]], [0])]).clone())
    if dtype == "float32":
        assert err(torch.cat(got), O.forward(cfg, w, ids)) < TOL32
    else:
        assert ok16(torch.cat(got), *oracle16(cfg, w, ids))


@pytest.mark.parametrize("sizes", [[2, 2, 3, 61, 2, 64, 1, 1, 65], [63, 1, 1, 63, 2, 69], [1] * 5 + [194]])
def test_portions_of_several_sizes(sizes):
    cfg, w, model = make()
    ids = toks(sum(sizes))
    eng, got, at = engine(model), [], 0
    for n in sizes:
        got.append(eng.forward([("s", ids[at: at + n], list(range(n)))]))
        at += n
    assert err(torch.cat(got), O.forward(cfg, w, ids)) < TOL32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_match_each_request_alone(dtype):
    """Four requests of unequal length advance together -- portions beside single tokens -- through a pool too small for
    all of them at once, so pages and slots are handed on; each must match the same request run alone."""
    cfg, w, model = make(dtype=dtype)
    reqs = {n: toks(m, seed=10 + i) for i, (n, m) in enumerate((("a", 200), ("b", 90), ("c", 33), ("d", 130), ("e", 70)))}
    want = {n: (O.forward(cfg, w, ids), None) if dtype == "float32" else oracle16(cfg, w, ids) for n, ids in reqs.items()}
    eng = engine(model, max_tokens=576, max_seqs=4)
    plan = [[("a", 64), ("b", 2)], [("a", 1), ("b", 50), ("c", 33)], [("a", 100), ("b", 1), ("d", 3)],
            [("a", 35), ("b", 37), ("d", 61)], [("d", 2), ("e", 30)], [("d", 64), ("e", 1)], [("e", 39)]]
    at, got = {n: 0 for n in reqs}, {n: [] for n in reqs}
    for step in plan:
        entries = []
        for n, m in step:
            entries.append((n, reqs[n][at[n]: at[n] + m], list(range(m))))
            at[n] += m
        out = eng.forward(entries)
        o = 0
        for n, m in step:
            got[n].append(out[o: o + m])
            o += m
        for n, _ in step:
            if at[n] == len(reqs[n]):
                eng.finish(n)
    for n in reqs:
        assert at[n] == len(reqs[n])
        if dtype == "float32":
            assert err(torch.cat(got[n]), want[n][0]) < TOL32, n
        else:
            assert ok16(torch.cat(got[n]), *want[n]), n


def test_pages_and_slots_are_used_again():
    cfg, w, model = make(kinds=["moe", "dense"], n_layers=2)
    eng = engine(model, max_tokens=192, max_seqs=1)
    for k in range(4):
        ids = toks(100 + 20 * k, seed=k)
        got = whole(eng, ids, sid=f"r{k}")
        assert err(got, O.forward(cfg, w, ids)) < TOL32
    assert eng.cache.allocator.get_num_free_pages() == eng.cache.n_pages


def test_first_tokens_and_single_token_sequences():
    cfg, w, model = make()
    eng = engine(model)
    for n in (1, 2, 3):
        ids = toks(n, seed=n)
        assert err(whole(eng, ids), O.forward(cfg, w, ids)) < TOL32
    a, b = toks(1, seed=7), toks(1, seed=8)
    out = eng.forward([("a", a, [0]), ("b", b, [0])])
    assert err(out[:1], O.forward(cfg, w, a)) < TOL32 and err(out[1:], O.forward(cfg, w, b)) < TOL32


def test_long_decoding_through_captured_steps():
    """300 single-token steps of two sequences side by side (the captured decode graph), bf16, against the restatement."""
    cfg, w, model = make(dtype="bfloat16", kinds=["moe", "dense"], n_layers=2)
    a, b = toks(330, seed=3), toks(310, seed=4)
    eng = engine(model, graph=True)
    eng.forward([("a", a[:30], []), ("b", b[:10], [])])
    ga, gb = [], []
    for t in range(300):
        out = eng.forward([("a", [a[30 + t]], [0]), ("b", [b[10 + t]], [0])])
        ga.append(out[:1].clone())
        gb.append(out[1:].clone())
    wa, ma = oracle16(cfg, w, a)
    wb, mb = oracle16(cfg, w, b)
    assert ok16(torch.cat(ga), wa[30:], ma) and ok16(torch.cat(gb), wb[10:], mb)


@pytest.mark.parametrize("kw", [dict(heads=1, kv_heads=1, dim=8, width=24), dict(heads=6, kv_heads=1, dim=24),
                                dict(heads=3, kv_heads=3, dim=40, width=56, ff=33, expert_ff=17, shared_ff=9),
                                dict(experts=4, top=4, groups=(1, 1), shared_ff=0), dict(experts=7, top=1, groups=(7, 1)),
                                dict(q_temp=None), dict(q_temp=(1.3, 1)), dict(q_temp=(0.4, 2.5)), dict(heads=2, kv_heads=1, dim=64, width=128),
                                dict(heads=2, kv_heads=2, dim=128, width=64, kinds=[None, "dense"], n_layers=2)],
                         ids=["one-head", "one-kv-head", "odd-sizes", "all-experts", "top-1", "no-temperature",
                              "temperature-every-1", "temperature-every-2.5", "tile-head-size", "tile-head-size-128"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(kw, dtype):
    cfg, w, model = make(dtype=dtype, **kw)
    ids = toks(83)
    if dtype == "float32":
        assert err(whole(engine(model), ids), O.forward(cfg, w, ids)) < TOL32
    else:
        assert ok16(whole(engine(model), ids), *oracle16(cfg, w, ids))


def test_tile_attention_against_the_row_kernel(monkeypatch):
    """bf16 prompt portions at a head size the tensor-core tiles serve: far keys, page borders, a portion that starts
    in the middle of a page."""
    cfg, w, model = make(dtype="bfloat16", heads=4, kv_heads=2, dim=64, width=128, kinds=[None, "dense"], n_layers=2)
    ids = toks(333)
    want = O.forward(cfg, w, ids, rnd=O.bf16_round)
    eng = engine(model)
    got = [eng.forward([("s", ids[:37], list(range(37)))]), eng.forward([("s", ids[37:229], list(range(192)))]),
           eng.forward([("s", ids[229:], list(range(104)))])]
    assert err(torch.cat(got), want) < TOL16


def test_greedy_generation_through_the_engine():
    cfg, w, model = make(dtype="float32")
    prompts = [toks(40, seed=1), toks(7, seed=2), toks(90, seed=3)]
    eng = engine(model, max_tokens=512, max_seqs=2)
    outs = eng.generate(prompts, max_new_tokens=12, step_tokens=48)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:                           # every generated token is the oracle's argmax given what came before
            lg = O.forward(cfg, w, seq)[-1]
            top2 = lg.topk(2).values
            if float(top2[0] - top2[1]) > 1e-3:
                assert int(lg.argmax()) == tok
            seq.append(tok)


def test_decode_attention_spread_over_a_cluster():
    """Few (token, head) pairs make clusters of CTAs share a pair's keys; contexts that do not fill every CTA's slice,
    end inside a 32-key block or leave whole CTAs without keys must give what one CTA alone gives (a prompt run)."""
    cfg, w, model = make(kinds=[None], n_layers=1, heads=2, kv_heads=1, dim=24, width=40, max_positions=700)
    ids = toks(640)
    want = O.forward(cfg, w, ids)
    eng = engine(model, graph=False)
    for start in (1, 30, 33, 255, 257, 600):
        eng.forward([("s", ids[:start], [])])
        got = [eng.forward([("s", [ids[t]], [0])]) for t in range(start, start + 36)]
        eng.finish("s")
        assert err(torch.cat(got), want[start: start + 36]) < TOL32, start


def test_checkpoint_on_disk_through_the_command_line(tmp_path):
    """config.json + model.safetensors -> registry -> bin/trace_run (a sequence ended and its slot re-used) and the
    `generate` command."""
    import json, os, subprocess, sys
    import numpy as np
    from safetensors.torch import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, w, model = make(dtype="float32")
    del model
    mdir, out = tmp_path / "m", tmp_path / "o"
    mdir.mkdir()
    save_file({k: v.contiguous() for k, v in w.items()}, str(mdir / "model.safetensors"))
    (mdir / "config.json").write_text(json.dumps(cfg))
    a, b = toks(70, seed=90), toks(9, seed=91)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b, "want": [8]}],
              "end": ["b"]},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "c", "tokens": b[:4], "want": [3]}, {"id": "a", "tokens": [a[0]], "want": [0]}],
              "end": ["a", "c"]}]
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192", "--max-seqs", "2"], input="\n".join(json.dumps(x) for x in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    ra, rb = O.forward(cfg, w, a + [a[0]]), O.forward(cfg, w, b)
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, -1).copy())
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1).copy())
    assert err(got0, torch.stack([ra[0], ra[65], rb[8]])) < TOL32
    assert err(got2, torch.stack([rb[3], ra[70]])) < TOL32
    g = subprocess.run([sys.executable, "-m", "proxy_inference_engine_b200", "generate", "--model", str(mdir), "--prompt-ids",
                        ",".join(map(str, b)), "--max-new-tokens", "5", "--dtype", "float32"], cwd=root, capture_output=True,
                       text=True, timeout=600)
    assert g.returncode == 0, g.stderr[-2000:]
    rec = json.loads(g.stdout.strip().splitlines()[-1])
    assert rec["prompt_ids"] == b and len(rec["generated_ids"]) == 5
    ref = O.forward(cfg, w, b + rec["generated_ids"])
    for jj, tok in enumerate(rec["generated_ids"]):
        row = ref[len(b) - 1 + jj]
        assert float(row.max() - row[tok]) < 1e-3
