"""Golitar on the GPU against the plain float64 restatement of tests/golitar_oracle.py: every mechanism in a model of
its own, prompts against token-by-token decoding, portions, mixed batches, re-used pages and slots, the edges of
windows and pages, long-range memory of the recurrence, odd sizes, and greedy generation through the engine."""
import copy

import pytest
import torch

import golitar_oracle as O

pytestmark = pytest.mark.gpu

DELTA = {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "conv": 3}, "mlp": None}
ATTN = {"type": "attention", "mlp": None,
        "mixer": {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 40, "diff": 0.2, "scale": 0.3, "softcap": 30.0,
                  "mask": {"size": 9},
                  "rot": {"base": 10000.0, "dims": 12,
                          "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}}}
FF = {"kind": "dense", "ff": 136}


def make(layers, width=72, vocab=203, streams=3, seed=0, dtype="float32", cap=12.0, **kw):
    from proxy_inference_engine_b200.golitar import GolitarArgs, GolitarModel, random_weights
    cfg = {"architecture": "Golitar", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": 1e-5},
           "layers": copy.deepcopy(layers)}
    if cap:
        cfg["logit_softcap"] = cap
    args = GolitarArgs.from_dict(cfg)
    w = random_weights(args, seed=seed)
    for name, fn in (kw.get("edit") or {}).items():
        w[name] = fn(w[name]).to(torch.bfloat16)
    return cfg, w, GolitarModel(args, w, "cuda", dtype)


def engine(model, max_tokens=1024, max_seqs=4):
    from proxy_inference_engine_b200.engine import HybridEngine
    return HybridEngine(model, max_tokens, max_seqs)


def toks(n, vocab=203, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def err(got, want):
    """rms of the difference over rms of the reference, per row, worst row."""
    got, want = got.double().cpu(), want.double()
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)).max())


def whole(eng, ids, sid="w"):
    out = eng.forward([(sid, ids, list(range(len(ids))))])
    eng.finish(sid)
    return out


TOL32, TOL16 = 2e-4, 4e-2


# ---- each mechanism in a model of its own ---------------------------------------------------------------------------
@pytest.mark.parametrize("layers", [[DELTA], [ATTN], [dict(DELTA, mlp=FF)], [dict(ATTN, mlp=FF)], [DELTA, ATTN, DELTA]],
                         ids=["delta", "attention", "delta+ff", "attention+ff", "stack"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_match_the_oracle(layers, dtype):
    cfg, w, model = make(layers, dtype=dtype)
    ids = toks(37)
    trace = []
    eng = engine(model)
    got = eng.forward([("a", ids, list(range(len(ids))))], trace=trace)
    want, want_layers = O.forward(cfg, w, ids, return_layers=True)
    tol = TOL32 if dtype == "float32" else TOL16
    for i, t in enumerate(trace):
        assert err(t, want_layers[i]) < tol, f"residual after layer {i}"
    assert err(got, want) < tol


@pytest.mark.parametrize("streams", [1, 2, 5])
def test_residual_streams(streams):
    cfg, w, model = make([dict(DELTA, mlp=FF), dict(ATTN, mlp=FF)], streams=streams)
    ids = toks(20)
    assert err(whole(engine(model), ids), O.forward(cfg, w, ids)) < TOL32


def test_plain_residual_without_stream_weights():
    from proxy_inference_engine_b200.golitar import GolitarArgs, GolitarModel, random_weights
    cfg = {"architecture": "Golitar", "vocab": 120, "width": 64, "norm": {"eps": 1e-6}, "layers": [dict(DELTA, mlp=FF), ATTN]}
    w = {k: v for k, v in random_weights(GolitarArgs.from_dict(cfg), seed=3).items() if ".hc" not in k}
    model = GolitarModel(GolitarArgs.from_dict(cfg), w, "cuda", "float32")
    ids = toks(19, 120)
    assert err(whole(engine(model), ids), O.forward(cfg, w, ids)) < TOL32


def test_linear_kernels_agree_with_a_plain_product():
    """The three shapes of pieh_linear (few rows, tiles, ragged edges) in both precisions, with bias and epilogues."""
    import ctypes as C
    from proxy_inference_engine_b200 import _lib
    L = _lib.load_hybrid(build_if_missing=True)
    g = torch.Generator().manual_seed(0)
    for M, N, K in [(1, 96, 64), (3, 50, 200), (8, 130, 72), (9, 64, 64), (70, 100, 99), (200, 300, 256)]:
        for exact in (True, False):
            x = torch.randn((M, K), generator=g).cuda()
            wt = (torch.randn((N, K), generator=g) / K ** 0.5).to(torch.bfloat16)
            bias = torch.randn((N,), generator=g).cuda()
            wd = wt.float().cuda() if exact else wt.cuda()
            for epi in (0, 1, 2):
                out = torch.empty((M, N), dtype=torch.float32, device="cuda")
                st = L.pieh_linear(C.c_void_p(out.data_ptr()), 1, N, C.c_void_p(x.data_ptr()), 1, K, C.c_void_p(wd.data_ptr()),
                                   1 if exact else 0, C.c_void_p(bias.data_ptr()), M, N, K, epi, 5.0, None, None, 0, None)
                assert st == 0
                xr = x.double().cpu() if exact else x.to(torch.bfloat16).double().cpu()
                y = xr @ wt.double().T + bias.double().cpu()
                y = torch.relu(y) ** 2 if epi == 1 else (5.0 * torch.tanh(y / 5.0) if epi == 2 else y)
                assert err(out, y) < 1e-5, (M, N, K, exact, epi)


def test_stream_operators_alone():
    """pieh_stream_norm (weighted stream sum, RMS norm, offset weight, row gather) and pieh_stream_update against the
    restatement's hyper_step, at stream counts 1, 3 and 8 and a width that is not a multiple of the block."""
    import ctypes as C
    from proxy_inference_engine_b200 import _lib
    L = _lib.load_hybrid(build_if_missing=True)
    p = lambda t: C.c_void_p(t.data_ptr())
    g = torch.Generator().manual_seed(4)
    for S, W, T in ((1, 72, 5), (3, 300, 9), (8, 64, 2)):
        xs = torch.randn((T, S, W), generator=g)
        hc = {"h.in": torch.randn((S,), generator=g), "h.out": torch.randn((S,), generator=g),
              "h.mix": torch.randn((S, S), generator=g)}
        nw, y = 0.2 * torch.randn((W,), generator=g), torch.randn((T, W), generator=g)
        seen = {}

        def sub(u):
            seen["normed"] = O.norm_centered(u, nw.double(), 1e-5)
            return y.double()
        want = O.hyper_step(xs.double().permute(1, 0, 2), hc, "h.", sub).permute(1, 0, 2)
        rows = torch.tensor([T - 1, 0], dtype=torch.int32).cuda()
        xd, out = xs.cuda().contiguous(), torch.empty((2, W), dtype=torch.float32, device="cuda")
        assert L.pieh_stream_norm(p(out), 1, p(xd), p(rows), p(hc["h.in"].cuda()), p(nw.cuda()), 1.0, 1e-5, 2, S, W, None) == 0
        assert err(out, seen["normed"][[T - 1, 0]]) < 1e-5
        assert L.pieh_stream_update(p(xd), p(y.cuda()), p(hc["h.mix"].cuda().contiguous()), p(hc["h.out"].cuda()), T, S, W, None) == 0
        assert err(xd.reshape(T, -1), want.reshape(T, -1)) < 1e-5


@pytest.mark.parametrize("H,G,dk,dv,taps", [(2, 1, 16, 16, 4), (3, 3, 40, 24, 2), (4, 2, 130, 70, 1), (1, 1, 300, 8, 5)])
def test_delta_operators_alone(H, G, dk, dv, taps):
    """pieh_delta_prepare / _scan / _gate fed with given projections (no matrix products), against the restatement's
    delta mixer with selector matrices: whole sequences, single tokens, uneven portions, two sequences interleaved in one
    step, and slots that hold another sequence's state when a new one starts."""
    import ctypes as C
    from proxy_inference_engine_b200 import _lib
    from proxy_inference_engine_b200.ragged import BatchDetails
    L = _lib.load_hybrid(build_if_missing=True)
    p = lambda t: C.c_void_p(t.data_ptr())
    g = torch.Generator().manual_seed(dk)
    nq, nv = G * dk, H * dv
    P = 2 * nq + 2 * nv + 2 * H
    sel = torch.eye(P)
    w = {"q": sel[:nq], "k": sel[nq:2 * nq], "v": sel[2 * nq:2 * nq + nv], "g": sel[2 * nq + nv:2 * nq + 2 * nv],
         "b": sel[2 * nq + 2 * nv:2 * nq + 2 * nv + H], "a": sel[2 * nq + 2 * nv + H:], "o": torch.eye(nv),
         "A_log": torch.log(0.2 + torch.rand(H, generator=g)), "dt_bias": torch.randn(H, generator=g) - 1.0,
         "norm": 1 + 0.1 * torch.randn(dv, generator=g)}
    if taps > 1:
        for n, rows in (("q", nq), ("k", nq), ("v", nv)):
            w[n + ".conv"] = torch.randn((rows, taps), generator=g) / taps ** 0.5
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv}
    seqs = {"a": torch.randn((61, P), generator=g), "b": torch.randn((23, P), generator=g)}
    want = {k: O.delta_mixer(v.double(), {"x." + n: t for n, t in w.items()}, "x.", m, 1e-5) for k, v in seqs.items()}
    C_ = 2 * nq + nv
    conv_w = (torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]]) if taps > 1 else torch.ones((C_, 1))).cuda().contiguous()
    state = torch.full((3, H, dk, dv), 9.0, device="cuda")                     # slots start full of someone else's state
    hist = torch.full((3, max(taps - 1, 1), C_), -7.0, device="cuda")
    d = _lib.HybDelta(H, G, dk, dv, taps, conv_w.data_ptr(), w["A_log"].cuda().data_ptr(), w["dt_bias"].cuda().data_ptr(),
                      w["norm"].cuda().data_ptr(), 1e-5, hist.data_ptr(), state.data_ptr())
    keep = [w["A_log"].cuda(), w["dt_bias"].cuda(), w["norm"].cuda()]
    d.A_log, d.dt_bias, d.out_norm = (t.data_ptr() for t in keep)

    def step(parts):
        """parts: [(name, rows lo..hi, slot)] -> outputs per part"""
        b = BatchDetails.build([(n, [0] * (hi - lo), lo, [0], slot) for n, lo, hi, slot in parts], device="cuda")
        desc, ka = b.hybrid_descriptor()
        proj = torch.cat([seqs[n][lo:hi] for n, lo, hi, _ in parts]).cuda().contiguous()
        T = proj.shape[0]
        f = lambda *sh: torch.empty(sh, dtype=torch.float32, device="cuda")
        q, k, v, be, de, o, out = f(T, G, dk), f(T, G, dk), f(T, H, dv), f(T, H), f(T, H), f(T, H, dv), f(T, nv)
        assert L.pieh_delta_prepare(p(q), p(k), p(v), p(be), p(de), p(proj), P, C.byref(d), C.byref(desc), None) == 0
        assert L.pieh_delta_scan(p(o), p(q), p(k), p(v), p(be), p(de), C.byref(d), C.byref(desc), None) == 0
        assert L.pieh_delta_gate(p(out), 1, p(o), p(proj), P, 2 * nq + nv, C.byref(d), T, None) == 0
        torch.cuda.synchronize()
        res, at = [], 0
        for n, lo, hi, _ in parts:
            res.append(out[at:at + hi - lo].cpu())
            at += hi - lo
        return res

    assert err(step([("a", 0, 61, 0)])[0], want["a"]) < 1e-4                                   # whole, slot 0
    got = torch.cat([step([("a", t, t + 1, 1)])[0] for t in range(61)])                          # token by token, slot 1
    assert err(got, want["a"]) < 1e-4
    # slot 0 now holds a's final state: b starts there from zero, interleaved with a restarting in slot 2
    cuts_a, cuts_b = [0, 5, 6, 26, 61], [0, 2, 3, 20, 23]
    ga, gb = [], []
    for i in range(4):
        ra, rb = step([("b", cuts_b[i], cuts_b[i + 1], 0), ("a", cuts_a[i], cuts_a[i + 1], 2)])[::-1]
        ga.append(ra); gb.append(rb)
    assert err(torch.cat(ga), want["a"]) < 1e-4 and err(torch.cat(gb), want["b"]) < 1e-4


def test_tensor_core_linear_matches_a_plain_product():
    """bf16 activations, M >= 64, K a multiple of 64: the tcgen05 kernel, both tile heights, ragged M and N, every epilogue."""
    import ctypes as C
    from proxy_inference_engine_b200 import _lib
    L = _lib.load_hybrid(build_if_missing=True)
    g = torch.Generator().manual_seed(1)
    p = lambda t: C.c_void_p(t.data_ptr())
    for M, N, K in [(64, 256, 64), (130, 300, 192), (300, 77, 128), (1000, 520, 256), (2100, 5000, 64)]:
        x = torch.randn((M, K), generator=g).to(torch.bfloat16).cuda()
        wt = (torch.randn((N, K), generator=g) / K ** 0.5).to(torch.bfloat16).cuda()
        bias = torch.randn((N,), generator=g).cuda()
        y = x.double().cpu() @ wt.double().cpu().T + bias.double().cpu()
        for epi, odt in ((0, 1), (1, 0), (2, 1)):
            out = torch.empty((M, N), dtype=torch.float32 if odt else torch.bfloat16, device="cuda")
            assert L.pieh_linear(p(out), odt, N, p(x), 0, K, p(wt), 0, p(bias), M, N, K, epi, 5.0, None, None, 0, None) == 0
            ref = torch.relu(y) ** 2 if epi == 1 else (5.0 * torch.tanh(y / 5.0) if epi == 2 else y)
            assert err(out.float(), ref) < (1e-5 if odt else 5e-3), (M, N, K, epi)
        S = 3
        xs = torch.randn((M, S, N), generator=g).cuda()
        mix, ow = torch.randn((S, S), generator=g).cuda(), torch.randn((S,), generator=g).cuda()
        ref = torch.einsum("su,msn->mun", mix.double().cpu(), xs.double().cpu()) + ow.double().cpu()[None, :, None] * y[:, None]
        assert L.pieh_linear(p(xs), 1, 0, p(x), 0, K, p(wt), 0, p(bias), M, N, K, 3, 0.0, p(mix), p(ow), S, None) == 0
        assert err(xs.reshape(M, -1), ref.reshape(M, -1)) < 1e-5
    assert L.pieh_pipeline_error() == 0


def test_long_portions_run_on_the_tensor_cores():
    cfg, w, model = make([dict(DELTA, mlp=FF), dict(ATTN, mlp=FF)], width=128, dtype="bfloat16")
    ids = toks(200)
    want = O.forward(cfg, w, ids)
    eng = engine(model)
    got = torch.cat([eng.forward([("a", ids[:150], list(range(150)))]), eng.forward([("a", ids[150:], list(range(50)))])])
    assert err(got, want) < TOL16 and model.L.pieh_pipeline_error() == 0


# ---- schedules ------------------------------------------------------------------------------------------------------
HYBRID = [dict(DELTA, mlp=None), dict(ATTN, mlp=FF), DELTA]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token(dtype):
    cfg, w, model = make(HYBRID, dtype=dtype)
    ids = toks(90)
    want = O.forward(cfg, w, ids)
    eng = engine(model)
    rows = [eng.forward([("a", ids[:50], None)])]
    for t in range(50, 90):
        rows.append(eng.forward([("a", [ids[t]], [0])]))
    tol = TOL32 if dtype == "float32" else TOL16
    assert err(torch.cat(rows), want[49:]) < tol


@pytest.mark.parametrize("sizes", [[2] * 20, [1, 2, 3, 5, 7, 11, 2, 9], [63, 2, 64, 1], [64, 64], [5, 70, 2]])
def test_portions_of_any_size(sizes):
    cfg, w, model = make(HYBRID)
    ids = toks(sum(sizes))
    want = O.forward(cfg, w, ids)
    eng = engine(model)
    at, got = 0, []
    for n in sizes:
        got.append(eng.forward([("a", ids[at:at + n], list(range(n)))]))
        at += n
    assert err(torch.cat(got), want) < TOL32


def test_unequal_requests_in_one_batch_equal_each_alone():
    cfg, w, model = make(HYBRID)
    seqs = {"a": toks(130, seed=2), "b": toks(7, seed=3), "c": toks(66, seed=4), "d": toks(1, seed=5)}
    want = {k: O.forward(cfg, w, v) for k, v in seqs.items()}
    eng = engine(model, max_tokens=64 * 7)
    # step 1: portions of a, b (whole), c; step 2: the rest of a and c beside d's only token; step 3: single tokens
    s1 = eng.forward([("a", seqs["a"][:100], [99]), ("b", seqs["b"], [0, 6]), ("c", seqs["c"][:3], [2])])
    s2 = eng.forward([("a", seqs["a"][100:129], [0, 28]), ("d", seqs["d"], [0]), ("c", seqs["c"][3:65], [61])])
    s3 = eng.forward([("c", seqs["c"][65:], [0]), ("a", seqs["a"][129:], [0])])
    got = torch.cat([s1, s2, s3])
    ref = torch.stack([want["a"][99], want["b"][0], want["b"][6], want["c"][2], want["a"][100], want["a"][128],
                       want["d"][0], want["c"][64], want["c"][65], want["a"][129]])
    assert err(got, ref) < TOL32


def test_pages_and_slots_are_used_again():
    """Two slots and four pages for six requests in turn: every later request lands on a slot and pages that still hold
    an earlier one's state, and must not see it."""
    cfg, w, model = make(HYBRID)
    eng = engine(model, max_tokens=64 * 4, max_seqs=2)
    used_slots, used_pages = set(), set()
    for r in range(6):
        ids = toks(70 + 9 * r, seed=10 + r)
        want = O.forward(cfg, w, ids)
        a = eng.forward([(r, ids[:33], [32])])
        used_slots.add(eng.cache.seqs[r]["slot"]); used_pages.update(eng.cache.seqs[r]["pages"])
        b = eng.forward([(r, ids[33:], None)])
        assert err(torch.cat([a, b]), torch.stack([want[32], want[-1]])) < TOL32, r
        if r % 2:                      # keep one alive over the next admission so slots alternate
            eng.finish(r)
            eng.finish(r - 1)
    assert len(used_slots) == 2 and len(used_pages) <= 4


def test_a_freed_slot_does_not_leak_its_state():
    cfg, w, model = make([DELTA])
    eng = engine(model, max_seqs=1)
    eng.forward([("x", toks(40, seed=7), None)])
    eng.finish("x")
    ids = toks(5, seed=8)
    assert err(whole(eng, ids), O.forward(cfg, w, ids)) < TOL32


# ---- edges ----------------------------------------------------------------------------------------------------------
def _peaky(window, gain=4.0):
    """One attention layer whose scores are large, so that a single key inside or outside the window shows."""
    a = copy.deepcopy(ATTN)
    a["mixer"]["mask"] = {"size": window}
    a["mixer"]["scale"] = 1.0
    a["mixer"]["softcap"] = 40.0
    big = lambda t: t.float() * gain
    return [a], {"l0.mix.q.norm": big, "l0.mix.k.norm": big}


@pytest.mark.parametrize("window,n", [(9, 30), (64, 140), (65, 140), (1, 12), (100, 260)])
def test_window_edge_in_prompt_and_in_decoding(window, n):
    layers, edit = _peaky(window)
    cfg, w, model = make(layers, edit=edit)
    base = toks(n, seed=20)
    last = n - 1
    for back, seen in ((window - 1, True), (window, False)):
        if last - back < 0:
            continue
        alt = list(base)
        alt[last - back] = (alt[last - back] + 17) % 203
        ref_a, ref_b = O.forward(cfg, w, base)[last], O.forward(cfg, w, alt)[last]
        moved = float((ref_a - ref_b).abs().max())
        if seen and window > 1:
            assert moved > 1e-3, "the planted key must matter for this test to mean anything"
        if not seen:
            assert moved < 1e-12
        for ids, ref in ((base, ref_a), (alt, ref_b)):
            eng = engine(model)
            p = eng.forward([("p", ids, [last])])                          # as a prompt
            eng.forward([("d", ids[:last - 3], [])])                          # decoded: last 4 tokens one by one
            for t in range(last - 3, last + 1):
                d = eng.forward([("d", [ids[t]], [0])])
            assert err(p, ref[None]) < TOL32 and err(d, ref[None]) < TOL32, (back, seen)


@pytest.mark.parametrize("d,dv,window", [(64, 64, 9), (64, 128, 64), (32, 128, 65), (32, 64, 100), (64, 128, 200), (64, 64, 0)])
def test_prompt_tiles_on_tensor_cores(d, dv, window):
    """bf16, head sizes the tile kernel takes: whole prompts, portions that start inside a page and inside a tile, a
    decoding sequence in the same step, against the restatement; and the window's edge must show."""
    layers, edit = _peaky(window or 7, gain=2.5)   # bf16 keys: moderate peaks, looser bound
    tol = 5e-2
    layers[0]["mixer"].update(dim=d, vdim=dv, heads=4, kv_heads=2, rot={"base": 1e4, "dims": d // 2})
    if not window:
        layers[0]["mixer"].pop("mask")
    cfg, w, model = make(layers, edit=edit, dtype="bfloat16", width=64)
    n = 330
    ids, other = toks(n, seed=21), toks(40, seed=22)
    want, want_o = O.forward(cfg, w, ids), O.forward(cfg, w, other)
    eng = engine(model)
    assert err(eng.forward([("w", ids, list(range(n)))]), want) < tol
    got = [eng.forward([("p", ids[:37], list(range(37)))])]
    eng.forward([("o", other[:39], [])])
    mixed = eng.forward([("p", ids[37:237], list(range(200))), ("o", other[39:], [0])])    # 200 rows + one decode row
    got += [mixed[:200], eng.forward([("p", ids[237:], list(range(n - 237)))])]
    assert err(torch.cat(got), want) < tol and err(mixed[200:], want_o[39:]) < tol


def _attention_op(q, k, v, window, portions, act=torch.bfloat16, lam=0.4, cap=30.0, scale=0.5):
    """pieh_attn_prepare + pieh_attn_run on given q [T, H, 2, d], k [T, G, 2, d], v [T, G, dv] (no norm, no rotation),
    one sequence fed in the given portions over scattered pages; returns [T, H, dv] float."""
    import ctypes as C
    from proxy_inference_engine_b200 import _lib
    from proxy_inference_engine_b200.ragged import BatchDetails
    L = _lib.load_hybrid(build_if_missing=True)
    T, H, _, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).float().cuda().contiguous()
    n_pages = (T + 63) // 64 + 3
    pages = list(range(n_pages - 1, 1, -1))                       # descending ids: a page table that is not the identity
    kp = torch.full((n_pages, 64, G, 2 * d), 7.0, dtype=act, device="cuda")     # stale finite contents everywhere
    vp = torch.full((n_pages, 64, G, dv), -3.0, dtype=act, device="cuda")
    code = 0 if act == torch.bfloat16 else 1
    at = _lib.HybAttn(H, G, d, dv, 0, None, None, None, 1e-6, scale, cap, window, lam, 0.8, kp.data_ptr(), vp.data_ptr(), code)
    outs, ctx = [], 0
    for n in portions:
        b = BatchDetails.build([("s", [0] * n, ctx, pages, 0)], device="cuda")
        desc, keep = b.hybrid_descriptor()
        qo = torch.empty((n, H, 2, d), dtype=torch.float32, device="cuda")
        out = torch.empty((n, H * dv), dtype=act, device="cuda")
        part = proj[ctx:ctx + n].contiguous()
        p = lambda t: C.c_void_p(t.data_ptr())
        assert L.pieh_attn_prepare(p(qo), p(part), part.stride(0), C.byref(at), C.byref(desc), None) == 0
        assert L.pieh_attn_run(p(out), code, p(qo), C.byref(at), C.byref(desc), None) == 0
        torch.cuda.synchronize()
        outs.append(out.float().view(n, H, dv))
        ctx += n
    return torch.cat(outs).cpu()


def _attention_ref(q, k, v, window, lam=0.4, cap=30.0, scale=0.5):
    rep = q.shape[1] // k.shape[1]
    kk, vv = k.double().repeat_interleave(rep, 1), v.double().repeat_interleave(rep, 1)
    m = [O.windowed_softmax_attention(q.double()[:, :, i], kk[:, :, i], vv, scale, cap, window) for i in (0, 1)]
    return O.unit_rms(m[0] - lam * m[1], 1e-6) * 0.8


@pytest.mark.parametrize("act", [torch.bfloat16, torch.float32], ids=["tiles-bf16", "rows-fp32"])
@pytest.mark.parametrize("d,dv", [(64, 128), (32, 64)])
@pytest.mark.parametrize("window", [5, 64, 65, 128, 130, 300])
def test_attention_operator_window_edge_with_a_dominant_key(act, d, dv, window):
    """One key per probe scores far above the rest and carries a value unlike the others: the probe row's output is that
    value exactly when the key is the oldest one inside the window, and is not when it is one step further back.  Probes
    sit at tile and page borders; prompt portions start inside pages; bf16 runs the tensor-core tiles, fp32 the row kernel."""
    g = torch.Generator().manual_seed(window)
    T, H, G = 400, 4, 2
    q = 0.1 * torch.randn((T, H, 2, d), generator=g)
    k = 0.1 * torch.randn((T, G, 2, d), generator=g)
    v = torch.randn((T, G, dv), generator=g)
    plan = [(window - 1, window - 1), (T - 1, window), (255, window - 1), (320, window)]
    plants = {}                                                # probe row -> planted key: just inside / just outside
    for r, back in plan:
        if r < T and r - back >= 0 and r not in plants:
            plants[r] = r - back
    for r, j in plants.items():
        q[r, :, :, :] = 0
        q[r, :, 0, 3] = 8.0                                    # map 1 of the probe row looks along feature 3
        k[j, :, 0, 3] = 8.0
        v[j] = 4.0 + torch.arange(dv)[None] * 0.01            # a value row that is easy to recognise
    sees = lambda r: any(0 <= r - j < window for j in plants.values())
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    ref = _attention_ref(q, k, v, window)
    tol = 3e-2 if act == torch.bfloat16 else 1e-4
    for portions in ([T], [37, 200, 163], [64, 64, 272]):
        got = _attention_op(q, k, v, window, portions, act)
        assert err(got.reshape(T, -1), ref.reshape(T, -1)) < tol, portions
    flat = lambda r: float(ref[r].std(-1).mean())             # a row dominated by the planted value is almost constant
    edge_in = [r for r, j in plants.items() if r - j == window - 1]
    edge_out = [r for r, j in plants.items() if r - j == window and not sees(r)]
    assert edge_in and all(flat(r) < 0.2 for r in edge_in)
    assert edge_out and all(flat(r) > 0.5 for r in edge_out)


def test_no_window_no_rotation_no_caps():
    a = copy.deepcopy(ATTN)
    for k in ("mask", "rot", "softcap"):
        a["mixer"].pop(k)
    cfg, w, model = make([a], cap=None)
    ids = toks(150)
    assert err(whole(engine(model), ids), O.forward(cfg, w, ids)) < TOL32


def test_recurrence_remembers_the_first_token_over_hundreds():
    """Decay close to one: the first token's write is still read 400 tokens later, through prompt portions and decoding."""
    slow = {"l0.mix.A_log": lambda t: torch.full_like(t.float(), -9.0)}
    wide = {"type": "delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 16, "conv": 3}, "mlp": None}
    cfg, w, model = make([wide], edit=slow)   # wide keys: later writes overlap the first one little
    base = toks(400, seed=30)
    alt = [(base[0] + 5) % 203] + base[1:]
    ref_a, ref_b = O.forward(cfg, w, base)[-1], O.forward(cfg, w, alt)[-1]
    assert float((ref_a - ref_b).abs().max()) > 1e-2
    for ids, ref in ((base, ref_a), (alt, ref_b)):
        eng = engine(model)
        eng.forward([("s", ids[:3], []), ])
        eng.forward([("s", ids[3:350], [])])
        for t in range(350, 400):
            out = eng.forward([("s", [ids[t]], [0])])
        assert err(out, ref[None]) < TOL32


def test_first_tokens_and_single_token_sequences():
    cfg, w, model = make(HYBRID)
    for n in (1, 2, 3):
        ids = toks(n, seed=40 + n)
        assert err(whole(engine(model), ids), O.forward(cfg, w, ids)) < TOL32
    ids = toks(6, seed=44)
    eng = engine(model)
    got = torch.cat([eng.forward([("a", [t], [0])]) for t in ids])       # decoding from the very first token
    assert err(got, O.forward(cfg, w, ids)) < TOL32


def test_long_decoding():
    cfg, w, model = make(HYBRID, dtype="bfloat16")
    ids = toks(300, seed=50)
    eng = engine(model)
    eng.forward([("a", ids[:20], [])])
    got = torch.cat([eng.forward([("a", [t], [0])]) for t in ids[20:]])
    assert err(got, O.forward(cfg, w, ids)[20:]) < TOL16


@pytest.mark.parametrize("case", range(4))
def test_other_sizes(case):
    d = {"type": "delta", "mlp": None}
    a = {"type": "attention", "mlp": None}
    cases = [
        dict(layers=[dict(d, mixer={"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 2}),
                     dict(a, mixer=dict(ATTN["mixer"], heads=1, kv_heads=1, dim=8, vdim=16, rot={"base": 100.0, "dims": 8}))],
             width=64, vocab=64, streams=1),
        dict(layers=[dict(d, mixer={"heads": 6, "kv_heads": 3, "dim": 80, "vdim": 48, "conv": 5}, mlp={"kind": "dense", "ff": 50})],
             width=100, vocab=77, streams=2),
        dict(layers=[dict(a, mixer=dict(ATTN["mixer"], heads=8, kv_heads=8, dim=16, vdim=128, mask={"size": 33}), mlp=FF),
                     dict(d, mixer={"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 130})],
             width=128, vocab=300, streams=4),
        dict(layers=[dict(a, mixer=dict(ATTN["mixer"], heads=2, kv_heads=1, dim=64, vdim=200, rot={"base": 5e5, "dims": 64})),
                     dict(d, mixer={"heads": 3, "kv_heads": 1, "dim": 17, "vdim": 33, "conv": 4})],
             width=88, vocab=97, streams=2),
    ]
    c = cases[case]
    cfg, w, model = make(c["layers"], width=c["width"], vocab=c["vocab"], streams=c["streams"])
    ids = toks(75, c["vocab"], seed=60 + case)
    want = O.forward(cfg, w, ids)
    eng = engine(model)
    got = [eng.forward([("a", ids[:41], list(range(41)))]), eng.forward([("a", ids[41:70], list(range(29)))])]
    got += [eng.forward([("a", [t], [0])]) for t in ids[70:]]
    assert err(torch.cat(got), want) < TOL32


# ---- the engine's own entry point -----------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler():
    """Six prompts, two slots, small steps: prompts are cut into portions beside decoding sequences, and slots and pages
    go round.  Every generated token must be the oracle's greedy choice given the same history (ties within rounding)."""
    cfg, w, model = make(HYBRID, dtype="bfloat16")
    eng = engine(model, max_tokens=64 * 5, max_seqs=2)
    prompts = [toks(n, seed=70 + n) for n in (5, 90, 33, 64, 1, 17)]
    outs = eng.generate(prompts, max_new_tokens=12, step_tokens=40)
    assert not eng.cache.seqs and len(eng.cache.free_slots) == 2
    assert eng.cache.allocator.get_num_free_pages() == eng.cache.n_pages
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        ref = O.forward(cfg, w, p + o)
        for j, tok in enumerate(o):
            row = ref[len(p) - 1 + j]
            assert float(row.max() - row[tok]) < 0.15, (len(p), j)


def test_sampled_generation_is_reproducible():
    from proxy_inference_engine_b200.samplers import make_sampler
    cfg, w, model = make([DELTA, ATTN], dtype="bfloat16")
    prompts = [toks(9, seed=80), toks(20, seed=81)]
    a = engine(model).generate(prompts, 8, sampler=make_sampler(temp=0.8, top_p=0.9, seed=3))
    b = engine(model).generate(prompts, 8, sampler=make_sampler(temp=0.8, top_p=0.9, seed=3))
    assert a == b and all(0 <= t < 203 for o in a for t in o)


def test_checkpoint_on_disk_through_the_command_line(tmp_path):
    """config.json + model.safetensors -> registry -> bin/trace_run (two steps, a sequence ended and its slot re-used)
    and `python -m proxy_inference_engine_b200 generate`."""
    import json, os, subprocess, sys
    import numpy as np
    from safetensors.torch import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, w, model = make([DELTA, dict(ATTN, mlp=FF)], dtype="float32")
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
        assert float(row.max() - row[tok]) < 0.15
