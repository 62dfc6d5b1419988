"""Babodra: a decoder-only model with learned absolute positions, post-norm residual sublayers, attention whose values
are its projected keys (distance bias per head, softmax sink, query temperature, sigmoid output gate) and feed-forward
sublayers that are either a clamped gated unit or a group-limited mixture of experts with a gated shared expert.  Served
through the ragged step of libpie_b200_hybrid.so like ``golitar.GolitarModel``: same ``BatchDetails``, same
``cache.HybridCache`` pages, same ``engine.HybridEngine``.

config.json: ``architecture`` "Babodra"; ``vocab``, ``width``, ``max_positions``, ``norm.eps`` and ``layers``, a list of
``{"type": "attention", "mixer": {heads, kv_heads, dim, vdim, scale, q_temp: {coef, every}}, "mlp": ... | null}`` with
``mlp`` = ``{"kind": "dense", "ff", "limit"}`` or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top",
"scale", "groups": {"count", "keep"}}, "shared": {"ff"} | null}``.
Tensors: ``embed``, ``pos``, ``head``, ``final.norm``, per layer i ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|g|o`` (+ ``q.b``,
``k.b``, ``q.norm``, ``k.norm``), ``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``,
``l<i>.mlp.shared.gate|up|down|sg``.

One step over a ``ragged.BatchDetails`` (x: fp32 residual [T, W]; xa: the same rows in the act dtype, written by whichever
kernel last changed x):

    x, xa  = embed_positions(tokens, positions)                               embed[token] + pos[position]
    p      = linear(xa; [q | k | gate] fused, biases of q and k)              fp32
    q      = bias_attn_prepare(p)       whole-projection norms, query temperature; normed k -> key pages, raw k -> value pages
    o      = bias_attn_run(q, p)        s = q.k scale - slope_h (i - j), softmax with a sink, times sigmoid(gate)
    x, xa  = postnorm_add(x, linear(o; output projection), norm1)             x += rms_norm(.) * w
    dense:   h = linear_glu(xa; [gate, up] interleaved)  ->  x, xa = postnorm_add(x, linear(h; down), norm2)
    moe:     z = linear(xa; [router | shared gate])  ->  moe_route (choices, slots sorted by expert)
             ys = moe_linear(moe_linear(xa gathered; experts' [gate, up], silu pair); experts' down)
             x, xa = postnorm_add(x, sum_k w_k ys[slot_k] + sigmoid(z_shared) shared(xa), norm2)
    logits = linear(stream_norm(x[wanted rows]; final norm); head)             fp32

dtype "bfloat16": matrix-product inputs and the pages are bf16, accumulation, residual, norms, softmax and routing fp32.
dtype "float32": weights are widened once and every product is a plain fp32 multiply-add.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import torch

from . import _lib
from ._lib import DTYPE_BF16, DTYPE_F32, EPI_NONE, HybBiasAttn, HybMixSum, HybMoePlan
from .cache import HybridCache
from .golitar import _Linear, _p, _stream
from .ragged import BatchDetails

GLU_SLOPE = 1.702        # dense feed-forward: gate * sigmoid(1.702 gate) * (up + 1)
SLOPE_EXPONENT = 8.0     # head h of H: slope 2^(-8 (h + 1) / H)


@dataclass
class BabodraArgs:
    vocab: int
    width: int
    layers: list
    max_positions: int
    norm_eps: float = 1e-5
    architecture: str = "Babodra"
    raw: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, cfg: dict) -> "BabodraArgs":
        for key in ("vocab", "width", "layers", "max_positions"):
            if key not in cfg:
                raise ValueError(f"Babodra config: '{key}' is missing")
        for i, ly in enumerate(cfg["layers"]):
            if ly.get("type") != "attention":
                raise ValueError(f"Babodra config: layer {i} has unknown type {ly.get('type')!r}")
            m = ly.get("mixer") or {}
            for key in ("heads", "kv_heads", "dim", "vdim", "scale"):
                if key not in m:
                    raise ValueError(f"Babodra config: layer {i} mixer lacks '{key}'")
            if int(m["heads"]) % int(m["kv_heads"]):
                raise ValueError(f"Babodra config: layer {i}: heads is not a multiple of kv_heads")
            if int(m["vdim"]) != int(m["dim"]):
                raise ValueError(f"Babodra config: layer {i}: the values are the projected keys, so vdim must equal dim")
            mlp = ly.get("mlp")
            if mlp and mlp.get("kind") not in ("dense", "moe"):
                raise ValueError(f"Babodra config: layer {i} has unknown feed-forward kind {mlp.get('kind')!r}")
            if mlp and mlp["kind"] == "moe":
                r = mlp["router"]
                g = r.get("groups") or {"count": 1, "keep": 1}
                if int(r["experts"]) % int(g["count"]) or int(g["keep"]) * (int(r["experts"]) // int(g["count"])) < int(r["top"]):
                    raise ValueError(f"Babodra config: layer {i}: the kept groups hold fewer experts than 'top'")
        return cls(vocab=int(cfg["vocab"]), width=int(cfg["width"]), layers=list(cfg["layers"]),
                   max_positions=int(cfg["max_positions"]), norm_eps=float((cfg.get("norm") or {}).get("eps", 1e-5)),
                   architecture=cfg.get("architecture", "Babodra"), raw=cfg)

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps}, "layers": self.layers}


def interleave_pairs(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[ff, K] x 2 -> [2 ff, K] with row 2 j = gate row j and row 2 j + 1 = up row j: the layout pieh_linear_glu reads, so
    that a gated pair lands in neighbouring accumulator columns of one thread."""
    return torch.stack([gate, up], 1).reshape(2 * gate.shape[0], gate.shape[1])


class BabodraModel:
    def __init__(self, args: BabodraArgs, weights: dict, device="cuda", dtype: str = "bfloat16"):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.args, self.device, self.dtype = args, device, dtype
        self.exact = dtype == "float32"
        self.act_torch = torch.float32 if self.exact else torch.bfloat16
        self.act = DTYPE_F32 if self.exact else DTYPE_BF16
        self.L = _lib.load_hybrid(build_if_missing=True)
        self.W = args.width
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        get = lambda name: weights[name]
        lin = lambda w, b=None: _Linear(w, b, self.exact, device)
        self.embed = get("embed").to(device=device, dtype=self.act_torch).contiguous()
        self.pos = get("pos").to(device=device, dtype=self.act_torch).contiguous()
        if self.pos.shape[0] < args.max_positions:
            raise ValueError("the position table is shorter than max_positions")
        self.head = lin(get("head"))
        self.final_norm = f32(get("final.norm"))
        self.layers, self.cache_specs = [], []
        for i, cfg in enumerate(args.layers):
            p, m = f"l{i}.", cfg["mixer"]
            H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            mw = lambda n: get(p + "mix." + n)
            bias = torch.cat([mw("q.b").float(), mw("k.b").float(), torch.zeros(H * dv, device=mw("q.b").device)])
            qt = m.get("q_temp") or {}
            ly = {"norm1": f32(get(p + "norm1")), "dims": (H, G, d, dv),
                  "proj": lin(torch.cat([mw("q"), mw("k"), mw("g")], 0), bias), "out": lin(mw("o")),
                  "q_norm": f32(mw("q.norm")), "k_norm": f32(mw("k.norm")), "scale": float(m["scale"]),
                  "temp": (float(qt.get("coef") or 0.0), float(qt.get("every") or 0.0)),
                  "slopes": torch.tensor([2.0 ** (-SLOPE_EXPONENT * (h + 1) / H) for h in range(H)], dtype=torch.float32,
                                         device=device),
                  "mlp": None}
            self.cache_specs.append({"kind": "attention", "G": G, "d": d, "dv": dv, "key_width": d})
            mlp = cfg.get("mlp")
            if mlp:
                ly["norm2"] = f32(get(p + "norm2"))
                q = p + "mlp."
                if mlp["kind"] == "dense":
                    ly["mlp"] = {"kind": "dense", "limit": float(mlp["limit"]),
                                 "gu": lin(interleave_pairs(get(q + "gate"), get(q + "up"))), "down": lin(get(q + "down"))}
                else:
                    r = mlp["router"]
                    E = int(r["experts"])
                    grp = r.get("groups") or {"count": 1, "keep": 1}
                    shared = mlp.get("shared") or None
                    rows = [get(q + "router")] + ([get(q + "shared.sg")] if shared else [])
                    wdt = torch.float32 if self.exact else torch.bfloat16
                    stack = lambda ts: torch.stack(ts, 0).to(device=device, dtype=wdt).contiguous()
                    ly["mlp"] = {"kind": "moe", "E": E, "top": int(r["top"]), "groups": (int(grp["count"]), int(grp["keep"])),
                                 "scale": float(r["scale"]), "router": lin(torch.cat(rows, 0)),
                                 "gu": stack([interleave_pairs(get(f"{q}e{e}.gate"), get(f"{q}e{e}.up")) for e in range(E)]),
                                 "down": stack([get(f"{q}e{e}.down") for e in range(E)]),
                                 "counters": torch.zeros(2 * E + 2, dtype=torch.int32, device=device), "shared": None}
                    if shared:
                        ly["mlp"]["shared"] = {"gu": lin(interleave_pairs(get(q + "shared.gate"), get(q + "shared.up"))),
                                               "down": lin(get(q + "shared.down"))}
            self.layers.append(ly)

    # ------------------------------------------------------------------------------------------------
    def make_cache(self, max_tokens: int, max_seqs: int = 4) -> HybridCache:
        return HybridCache(self.cache_specs, max_tokens, max_seqs, self.device, self.act_torch, lib=self.L)

    def _empty(self, shape, dtype=None):
        return torch.empty(shape, dtype=dtype or torch.float32, device=self.device)

    def _linear(self, lin: _Linear, x, M, out_dtype=None):
        out_dtype = DTYPE_F32 if out_dtype is None else out_dtype
        out = self._empty((M, lin.N), torch.float32 if out_dtype == DTYPE_F32 else torch.bfloat16)
        _lib.check_hybrid(self.L.pieh_linear(_p(out), out_dtype, out.stride(0), _p(x), self.act, x.stride(0), _p(lin.w),
                                             lin.w_dtype, _p(lin.bias), M, lin.N, lin.K, EPI_NONE, 0.0, None, None, 0,
                                             _stream()), "linear")
        return out

    def _glu(self, lin: _Linear, x, M, alpha, limit, offset):
        out = self._empty((M, lin.N // 2), self.act_torch)
        _lib.check_hybrid(self.L.pieh_linear_glu(_p(out), self.act, out.stride(0), _p(x), self.act, x.stride(0), _p(lin.w),
                                                 lin.w_dtype, M, lin.N, lin.K, alpha, limit, offset, _stream()), "linear_glu")
        return out

    def _postnorm(self, x, xa, y, mix, w, T):
        _lib.check_hybrid(self.L.pieh_postnorm_add(_p(x), _p(xa), self.act, _p(y), C.byref(mix) if mix else None, _p(w),
                                                   float(self.args.norm_eps), T, self.W, _stream()), "postnorm_add")

    def _moe(self, ml, xa, T):
        """-> (pieh_mix_sum describing the sublayer's output, tensors to keep alive until it is consumed)."""
        L, E, top, W = self.L, ml["E"], ml["top"], self.W
        P = T * top
        has_shared = ml["shared"] is not None
        z = self._linear(ml["router"], xa, T)                      # [T, E (+ 1)] fp32 logits
        i32 = lambda n: self._empty((n,), torch.int32)
        bufs = [i32(P), i32(P), i32(P), self._empty((P,)), i32(1 + 3 * (P // 64 + E)), i32(1 + 3 * (P // 128 + E))]
        plan = HybMoePlan(E, top, ml["groups"][0], ml["groups"][1], ml["scale"], *[b.data_ptr() for b in bufs],
                          ml["counters"].data_ptr())
        _lib.check_hybrid(L.pieh_moe_route(_p(z), z.stride(0), C.byref(plan), T, _stream()), "moe_route")
        wdt = DTYPE_F32 if self.exact else DTYPE_BF16
        ff2, ff = ml["gu"].shape[1], ml["gu"].shape[1] // 2
        hid = self._empty((P, ff), self.act_torch)
        _lib.check_hybrid(L.pieh_moe_linear(_p(hid), self.act, ff, _p(xa), self.act, xa.stride(0), _p(ml["gu"]), wdt,
                                            ff2 * W, P, ff2, W, 1, 1, 1.0, 0.0, 0.0, C.byref(plan), _stream()), "moe_gate_up")
        ys = self._empty((P, W))
        _lib.check_hybrid(L.pieh_moe_linear(_p(ys), DTYPE_F32, W, _p(hid), self.act, ff, _p(ml["down"]), wdt, W * ff, P, W,
                                            ff, 0, 0, 1.0, 0.0, 0.0, C.byref(plan), _stream()), "moe_down")
        so = None
        if has_shared:
            sh = self._glu(ml["shared"]["gu"], xa, T, 1.0, 0.0, 0.0)
            so = self._linear(ml["shared"]["down"], sh, T)
        mix = HybMixSum(ys.data_ptr(), bufs[2].data_ptr(), bufs[3].data_ptr(), top, so.data_ptr() if has_shared else None,
                        z.data_ptr() + 4 * E if has_shared else None, z.stride(0))
        return mix, (z, bufs, hid, ys, so)

    def step(self, batch: BatchDetails, cache: HybridCache, rows: torch.Tensor | None = None, trace: list | None = None):
        """One forward step over ``batch``; pages come from ``cache`` through the batch's block table.  rows: int32 device
        tensor of the token rows whose logits are wanted (None: each sequence's last row).  Returns fp32 logits
        [len(rows), vocab].  trace: if a list, the residual after every layer is appended to it (debugging aid)."""
        batch.validate()
        L, T, W, a = self.L, batch.total_tokens_in_step, self.W, self.args
        if max(c + n for c, n in zip(batch.context_lengths, batch.input_lengths)) > a.max_positions:
            raise ValueError(f"a sequence grows past the model's {a.max_positions} positions")
        desc, keep = batch.hybrid_descriptor()
        bref = C.byref(desc)
        x, xa = self._empty((T, W)), self._empty((T, W), self.act_torch)
        _lib.check_hybrid(L.pieh_embed_positions(_p(x), _p(xa), self.act, _p(self.embed), _p(self.pos), self.act,
                                                 _p(batch.token_ids), _p(batch.positions), T, W, a.vocab, a.max_positions,
                                                 _stream()), "embed_positions")
        for ly, st in zip(self.layers, cache.layers):
            H, G, d, dv = ly["dims"]
            proj = self._linear(ly["proj"], xa, T)
            ld = proj.stride(0)
            at = HybBiasAttn(H, G, d, dv, H * d, H * d, H * d + G * d, _p(ly["q_norm"]), _p(ly["k_norm"]), float(a.norm_eps),
                             ly["scale"], ly["temp"][0], ly["temp"][1], _p(ly["slopes"]), 1, 0, _p(st["k"]), _p(st["v"]),
                             self.act)
            q = self._empty((T, H * d))
            _lib.check_hybrid(L.pieh_bias_attn_prepare(_p(q), _p(proj), ld, C.byref(at), bref, _stream()), "attn_prepare")
            mixed = self._empty((T, H * dv), self.act_torch)
            _lib.check_hybrid(L.pieh_bias_attn_run(_p(mixed), self.act, _p(q), _p(proj), ld, C.byref(at), bref, _stream()),
                              "attn_run")
            self._postnorm(x, xa, self._linear(ly["out"], mixed, T), None, ly["norm1"], T)
            ml = ly["mlp"]
            if ml and ml["kind"] == "dense":
                hid = self._glu(ml["gu"], xa, T, GLU_SLOPE, ml["limit"], 1.0)
                self._postnorm(x, xa, self._linear(ml["down"], hid, T), None, ly["norm2"], T)
            elif ml:
                mix, alive = self._moe(ml, xa, T)
                self._postnorm(x, xa, None, mix, ly["norm2"], T)
                del alive
            if trace is not None:
                trace.append(x.clone())
        if rows is None:
            rows = batch.last_token_rows().to(torch.int32)
        R = int(rows.numel())
        xn = self._empty((R, W), self.act_torch)
        _lib.check_hybrid(L.pieh_stream_norm(_p(xn), self.act, _p(x), _p(rows), None, _p(self.final_norm), 0.0,
                                             float(a.norm_eps), R, 1, W, _stream()), "final_norm")
        logits = self._linear(self.head, xn, R)
        del keep
        return logits


def random_weights(args: BabodraArgs, seed: int = 0, device="cpu") -> dict:
    """A synthetic checkpoint of this design (bf16 tensors): matrices U(-1, 1) scaled by 1 / sqrt(in), norm weights
    around 1, small biases, router rows large enough that the choices are not near ties."""
    g = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16
    rnd = lambda *s: torch.rand(s, generator=g, device=device) * 2 - 1
    lin = lambda o, i, gain=1.0: (gain * rnd(o, i) / math.sqrt(i)).to(bf)
    W = args.width
    w = {"embed": torch.randn((args.vocab, W), generator=g, device=device).to(bf),
         "pos": (0.5 * torch.randn((args.max_positions, W), generator=g, device=device)).to(bf),
         "head": lin(args.vocab, W), "final.norm": (1 + 0.1 * rnd(W)).to(bf)}
    for i, cfg in enumerate(args.layers):
        p, m = f"l{i}.", cfg["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w[p + "norm1"] = (1 + 0.1 * rnd(W)).to(bf)
        w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.g"] = lin(H * d, W, 2.0), lin(G * d, W, 2.0), lin(H * dv, W, 2.0)
        w[p + "mix.q.b"], w[p + "mix.k.b"] = (0.1 * rnd(H * d)).to(bf), (0.1 * rnd(G * d)).to(bf)
        w[p + "mix.q.norm"], w[p + "mix.k.norm"] = (1 + 0.2 * rnd(H * d)).to(bf), (1 + 0.2 * rnd(G * d)).to(bf)
        w[p + "mix.o"] = lin(W, H * dv)
        mlp = cfg.get("mlp")
        if not mlp:
            continue
        w[p + "norm2"] = (1 + 0.1 * rnd(W)).to(bf)
        q = p + "mlp."
        if mlp["kind"] == "dense":
            w[q + "gate"], w[q + "up"], w[q + "down"] = lin(mlp["ff"], W, 2.0), lin(mlp["ff"], W, 2.0), lin(W, mlp["ff"])
        else:
            w[q + "router"] = lin(mlp["router"]["experts"], W, 3.0)
            sizes = [(f"e{e}.", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                sizes.append(("shared.", mlp["shared"]["ff"]))
                w[q + "shared.sg"] = lin(1, W, 2.0)
            for name, ff in sizes:
                w[q + name + "gate"], w[q + name + "up"], w[q + name + "down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
    return w
