"""Golitar: a decoder-only hybrid of gated-delta-rule layers and differential sliding-window attention layers over
hyper-connected residual streams, served through the ragged step of libpie_b200_hybrid.so (csrc/hyb_*.cu).

config.json: ``architecture`` "Golitar"; ``vocab``, ``width``, ``streams``, ``norm.eps``, ``logit_softcap`` and ``layers``,
a list of ``{"type": "delta" | "attention", "mixer": {...sizes...}, "mlp": {"kind": "dense", "ff": n} | null}``.
Tensors: ``embed``, ``head``, ``final.norm`` and per layer i ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``,
``l<i>.hc1|hc2.in|out|mix``.  Every size and constant is read from the config; a missing optional entry (rotation,
frequency scaling, window, soft caps, biases, stream weights) switches that piece off.

One model step over a ``ragged.BatchDetails`` (prompt portions and single decoded tokens side by side), per sublayer:

    u   = stream_norm(xs; in-weights, norm weight)               residual streams -> one normed input   (act dtype)
    p   = linear(u; fused projection)                            fp32
    delta:      delta_prepare (conv + silu, unit q / k, beta, decay) -> delta_scan (state in the slot) -> delta_gate
    attention:  attn_prepare (q / k norm, rotation, append to pages) -> attn_run (two maps, window, combine, norm)
    xs  = linear(o; output projection, STREAMS epilogue)         mixes the streams and adds the output in place
    feed-forward:  linear(u; up, relu^2 epilogue) -> linear(.; down, STREAMS epilogue)
    logits = linear(stream_norm(sum of streams; final norm)[wanted rows]; head, soft-cap epilogue)     fp32

dtype "bfloat16": matrix-product inputs and the key / value pages are bf16, accumulation and everything between the
products fp32.  dtype "float32": weights are widened once and every product is a plain fp32 multiply-add.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import torch

from . import _lib
from ._lib import (DTYPE_BF16, DTYPE_F32, EPI_NONE, EPI_RELU2, EPI_SOFTCAP, EPI_STREAMS, HybAttn, HybDelta)
from .cache import HybridCache
from .ragged import BatchDetails


@dataclass
class GolitarArgs:
    vocab: int
    width: int
    layers: list
    norm_eps: float = 1e-6
    streams: int = 1
    logit_softcap: float | None = None
    architecture: str = "Golitar"
    raw: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, cfg: dict) -> "GolitarArgs":
        for key in ("vocab", "width", "layers"):
            if key not in cfg:
                raise ValueError(f"Golitar config: '{key}' is missing")
        for i, ly in enumerate(cfg["layers"]):
            if ly.get("type") not in ("delta", "attention"):
                raise ValueError(f"Golitar config: layer {i} has unknown type {ly.get('type')!r}")
            mlp = ly.get("mlp")
            if mlp and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"Golitar config: layer {i} has unknown feed-forward kind {mlp.get('kind')!r}")
        return cls(vocab=int(cfg["vocab"]), width=int(cfg["width"]), layers=list(cfg["layers"]),
                   norm_eps=float((cfg.get("norm") or {}).get("eps", 1e-6)), streams=int(cfg.get("streams") or 1),
                   logit_softcap=cfg.get("logit_softcap") or None, architecture=cfg.get("architecture", "Golitar"), raw=cfg)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "streams": self.streams,
               "norm": {"eps": self.norm_eps}, "layers": self.layers}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out


def scaled_rotary_frequencies(rot: dict) -> list:
    """Angle per position of each rotated pair: base^(-2i/dims), with the long wavelengths slowed down by ``factor`` and
    a linear blend between the ``original/high`` and ``original/low`` wavelengths when ``scaling`` is given."""
    dims = int(rot["dims"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = float(rot["base"]) ** (-2.0 * i / dims)
        if sc:
            wl = 2.0 * math.pi / f
            if wl > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wl >= sc["original"] / sc["high"]:
                s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


class _Linear:
    """A dense matrix [out, in] in the product dtype of the model (+ optional fp32 bias)."""

    def __init__(self, w: torch.Tensor, bias, exact: bool, device):
        self.w = w.to(device=device, dtype=torch.float32 if exact else torch.bfloat16).contiguous()
        self.bias = None if bias is None else bias.to(device=device, dtype=torch.float32).contiguous()
        self.N, self.K = self.w.shape
        self.w_dtype = DTYPE_F32 if exact else DTYPE_BF16


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class GolitarModel:
    def __init__(self, args: GolitarArgs, weights: dict, device="cuda", dtype: str = "bfloat16"):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.args, self.device, self.dtype = args, device, dtype
        self.exact = dtype == "float32"
        self.act_torch = torch.float32 if self.exact else torch.bfloat16
        self.act = DTYPE_F32 if self.exact else DTYPE_BF16
        self.L = _lib.load_hybrid(build_if_missing=True)
        S, W = args.streams, args.width
        self.S, self.W = S, W
        if S > 8:
            raise ValueError("at most 8 residual streams are built")
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        get = lambda name: weights[name]
        self.embed = get("embed").to(device=device, dtype=self.act_torch).contiguous()
        self.embed_dtype = self.act
        self.head = _Linear(get("head") if "head" in weights else get("embed"), None, self.exact, device)
        self.final_norm = f32(get("final.norm"))
        self.layers, self.cache_specs = [], []
        for i, cfg in enumerate(args.layers):
            p, m = f"l{i}.", cfg["mixer"]
            ly = {"type": cfg["type"], "norm1": f32(get(p + "norm1")), "hc1": self._hc(weights, p + "hc1.", f32)}
            mw = lambda n: get(p + "mix." + n)
            opt = lambda n: weights.get(p + "mix." + n)
            if cfg["type"] == "delta":
                H, G, dk, dv, taps = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m.get("conv") or 1)
                ly["proj"] = _Linear(torch.cat([mw("q"), mw("k"), mw("v"), mw("g"), mw("b"), mw("a")], 0), None,
                                     self.exact, device)
                if opt("q.conv") is not None:
                    conv = torch.cat([mw("q.conv"), mw("k.conv"), mw("v.conv")], 0)
                    taps = int(conv.shape[1])
                else:
                    taps, conv = 1, torch.ones((2 * G * dk + H * dv, 1))
                ly["conv_w"] = f32(conv)
                ly["A_log"], ly["dt_bias"], ly["out_norm"] = f32(mw("A_log")), f32(mw("dt_bias")), f32(mw("norm"))
                ly["out"] = _Linear(mw("o"), None, self.exact, device)
                ly["dims"] = (H, G, dk, dv, taps)
                self.cache_specs.append({"kind": "delta", "H": H, "dk": dk, "dv": dv, "taps": taps,
                                         "channels": 2 * G * dk + H * dv})
            else:
                H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
                parts, biases = [mw("q"), mw("k"), mw("v")], [opt("q.b"), opt("k.b"), opt("v.b")]
                bias = None
                if any(b is not None for b in biases):
                    bias = torch.cat([b.float() if b is not None else torch.zeros(w.shape[0]) for w, b in zip(parts, biases)])
                ly["proj"] = _Linear(torch.cat(parts, 0), bias, self.exact, device)
                ly["out"] = _Linear(mw("o"), opt("o.b"), self.exact, device)
                ly["q_norm"] = f32(mw("q.norm")) if opt("q.norm") is not None else None
                ly["k_norm"] = f32(mw("k.norm")) if opt("k.norm") is not None else None
                rot = m.get("rot") or None
                ly["rot_dims"] = int(rot["dims"]) if rot else 0
                ly["rot_freqs"] = (torch.tensor(scaled_rotary_frequencies(rot), dtype=torch.float64).to(device)
                                   if rot else None)
                diff = float(m.get("diff") or 0.0)
                dot = lambda a, b: float((mw(a).double() * mw(b).double()).sum())
                ly["lambda"] = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + diff
                ly["out_scale"] = 1.0 - diff
                ly["scale"] = float(m.get("scale") or d ** -0.5)
                ly["softcap"] = float(m.get("softcap") or 0.0)
                ly["window"] = int((m.get("mask") or {}).get("size") or 0)
                ly["dims"] = (H, G, d, dv)
                self.cache_specs.append({"kind": "attention", "G": G, "d": d, "dv": dv})
            if cfg.get("mlp"):
                ly["norm2"] = f32(get(p + "norm2"))
                ly["hc2"] = self._hc(weights, p + "hc2.", f32)
                ly["up"] = _Linear(get(p + "mlp.up"), None, self.exact, device)
                ly["down"] = _Linear(get(p + "mlp.down"), None, self.exact, device)
            self.layers.append(ly)

    def _hc(self, weights, p, f32):
        S = self.S
        if (p + "in") in weights:
            return {"in": f32(weights[p + "in"]), "out": f32(weights[p + "out"]), "mix": f32(weights[p + "mix"])}
        if S != 1:
            raise ValueError(f"{p}in is missing although the model has {S} residual streams")
        one = torch.ones((1,), dtype=torch.float32, device=self.device)
        return {"in": one, "out": one, "mix": one.view(1, 1)}

    # ------------------------------------------------------------------------------------------------
    def make_cache(self, max_tokens: int, max_seqs: int = 4) -> HybridCache:
        return HybridCache(self.cache_specs, max_tokens, max_seqs, self.device, self.act_torch, lib=self.L)

    def _linear(self, lin: _Linear, x, M, out=None, out_dtype=None, epi=EPI_NONE, epi_a=0.0, hc=None):
        out_dtype = DTYPE_F32 if out_dtype is None else out_dtype
        if out is None:
            out = torch.empty((M, lin.N), dtype=torch.float32 if out_dtype == DTYPE_F32 else torch.bfloat16, device=self.device)
        x_dtype = DTYPE_F32 if x.dtype == torch.float32 else DTYPE_BF16
        _lib.check_hybrid(self.L.pieh_linear(_p(out), out_dtype, out.stride(0) if epi != EPI_STREAMS else 0, _p(x), x_dtype,
                                             x.stride(0), _p(lin.w), lin.w_dtype, _p(lin.bias), M, lin.N, lin.K, epi,
                                             float(epi_a), _p(hc["mix"]) if hc else None, _p(hc["out"]) if hc else None,
                                             self.S if hc else 0, _stream()), "linear")
        return out

    def _norm(self, xs, hc_in, w, R, rows=None, S=None):
        out = torch.empty((R, self.W), dtype=self.act_torch, device=self.device)
        _lib.check_hybrid(self.L.pieh_stream_norm(_p(out), self.act, _p(xs), _p(rows), _p(hc_in), _p(w), 1.0,
                                                  float(self.args.norm_eps), R, self.S if S is None else S, self.W,
                                                  _stream()), "stream_norm")
        return out

    def step(self, batch: BatchDetails, cache: HybridCache, rows: torch.Tensor | None = None, trace: list | None = None):
        """One forward step over ``batch``; the sequences' pages and slots come from ``cache`` (the block table and the
        ``state_slots`` of the batch name them).  rows: int32 device tensor of the token rows whose logits are wanted
        (None: each sequence's last row).  Returns fp32 logits [len(rows), vocab].  trace: if a list, the summed residual
        after every layer is appended to it (debugging aid)."""
        batch.validate()
        L, T, S, W, dev = self.L, batch.total_tokens_in_step, self.S, self.W, self.device
        desc, keep = batch.hybrid_descriptor()
        bref = C.byref(desc)
        f32 = torch.float32
        xs = torch.empty((T, S, W), dtype=f32, device=dev)
        _lib.check_hybrid(L.pieh_embed_streams(_p(xs), _p(self.embed), self.embed_dtype, _p(batch.token_ids), T, S, W,
                                               self.args.vocab, _stream()), "embed")
        for ly, st in zip(self.layers, cache.layers):
            u = self._norm(xs, ly["hc1"]["in"], ly["norm1"], T)
            proj = self._linear(ly["proj"], u, T)
            ld = proj.stride(0)
            if ly["type"] == "delta":
                H, G, dk, dv, taps = ly["dims"]
                d = HybDelta(H, G, dk, dv, taps, _p(ly["conv_w"]), _p(ly["A_log"]), _p(ly["dt_bias"]), _p(ly["out_norm"]),
                             float(self.args.norm_eps), _p(st["conv"]), _p(st["state"]))
                q = torch.empty((T, G, dk), dtype=f32, device=dev)
                k = torch.empty_like(q)
                v = torch.empty((T, H, dv), dtype=f32, device=dev)
                beta = torch.empty((T, H), dtype=f32, device=dev)
                decay = torch.empty_like(beta)
                o = torch.empty_like(v)
                _lib.check_hybrid(L.pieh_delta_prepare(_p(q), _p(k), _p(v), _p(beta), _p(decay), _p(proj), ld, C.byref(d),
                                                       bref, _stream()), "delta_prepare")
                _lib.check_hybrid(L.pieh_delta_scan(_p(o), _p(q), _p(k), _p(v), _p(beta), _p(decay), C.byref(d), bref,
                                                    _stream()), "delta_scan")
                mixed = torch.empty((T, H * dv), dtype=self.act_torch, device=dev)
                _lib.check_hybrid(L.pieh_delta_gate(_p(mixed), self.act, _p(o), _p(proj), ld, 2 * G * dk + H * dv,
                                                    C.byref(d), T, _stream()), "delta_gate")
            else:
                H, G, dd, dv = ly["dims"]
                a = HybAttn(H, G, dd, dv, ly["rot_dims"], _p(ly["rot_freqs"]), _p(ly["q_norm"]), _p(ly["k_norm"]),
                            float(self.args.norm_eps), ly["scale"], ly["softcap"], ly["window"], ly["lambda"],
                            ly["out_scale"], _p(st["k"]), _p(st["v"]), self.act)
                q = torch.empty((T, H, 2, dd), dtype=f32, device=dev)
                _lib.check_hybrid(L.pieh_attn_prepare(_p(q), _p(proj), ld, C.byref(a), bref, _stream()), "attn_prepare")
                mixed = torch.empty((T, H * dv), dtype=self.act_torch, device=dev)
                _lib.check_hybrid(L.pieh_attn_run(_p(mixed), self.act, _p(q), C.byref(a), bref, _stream()), "attn_run")
            self._linear(ly["out"], mixed, T, out=xs, epi=EPI_STREAMS, hc=ly["hc1"])
            if "up" in ly:
                u = self._norm(xs, ly["hc2"]["in"], ly["norm2"], T)
                hid = self._linear(ly["up"], u, T, out_dtype=self.act, epi=EPI_RELU2)
                self._linear(ly["down"], hid, T, out=xs, epi=EPI_STREAMS, hc=ly["hc2"])
            if trace is not None:
                trace.append(xs.sum(1))
        if rows is None:
            rows = batch.last_token_rows().to(torch.int32)
        R = int(rows.numel())
        x = self._norm(xs, None, self.final_norm, R, rows=rows)
        cap = self.args.logit_softcap
        logits = self._linear(self.head, x, R, epi=EPI_SOFTCAP if cap else EPI_NONE, epi_a=cap or 0.0)
        del keep
        return logits


def random_weights(args: GolitarArgs, seed: int = 0, device="cpu") -> dict:
    """A synthetic checkpoint of this design (bf16 tensors): matrices U(-1, 1) / sqrt(in), norm offsets and biases
    small, stream weights near the plain residual, decays spread over (0, 1).  device: where the values are drawn
    (the CPU stream is the reproducible one the tests use; large benchmark models draw on the GPU)."""
    g = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16
    rnd = lambda *s: torch.rand(s, generator=g, device=device) * 2 - 1
    lin = lambda o, i: (rnd(o, i) / math.sqrt(i)).to(bf)
    S, W = args.streams, args.width
    w = {"embed": torch.randn((args.vocab, W), generator=g, device=device).to(bf), "head": lin(args.vocab, W),
         "final.norm": (0.1 * rnd(W)).to(bf)}
    for i, cfg in enumerate(args.layers):
        p, m = f"l{i}.", cfg["mixer"]
        subs = ["1"] + (["2"] if cfg.get("mlp") else [])
        for q in subs:
            w[p + "norm" + q] = (0.1 * rnd(W)).to(bf)
            w[p + f"hc{q}.in"] = (1.0 / S + 0.1 * rnd(S)).to(bf)
            w[p + f"hc{q}.out"] = (1.0 + 0.2 * rnd(S)).to(bf)
            w[p + f"hc{q}.mix"] = (torch.eye(S, device=device) + 0.1 * rnd(S, S)).to(bf)
        if cfg["type"] == "delta":
            H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m.get("conv") or 1
            for n, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                w[p + "mix." + n] = lin(rows, W)
                if m.get("conv"):
                    w[p + f"mix.{n}.conv"] = (rnd(rows, taps) / math.sqrt(taps) + torch.eye(taps, device=device)[-1]).to(bf)
            w[p + "mix.g"], w[p + "mix.b"], w[p + "mix.a"] = lin(H * dv, W), lin(H, W), lin(H, W)
            w[p + "mix.A_log"] = torch.log(0.5 + 4 * torch.rand(H, generator=g, device=device)).to(bf)
            w[p + "mix.dt_bias"] = (rnd(H) - 2.0).to(bf)
            w[p + "mix.norm"] = (1 + 0.1 * rnd(dv)).to(bf)
            w[p + "mix.o"] = lin(W, H * dv)
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * 2 * d), ("k", G * 2 * d), ("v", G * dv)):
                w[p + "mix." + n] = lin(rows, W)
                w[p + f"mix.{n}.b"] = (0.1 * rnd(rows)).to(bf)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = (1 + 0.2 * rnd(d)).to(bf), (1 + 0.2 * rnd(d)).to(bf)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                w[p + "mix." + n] = (0.3 * rnd(d)).to(bf)
            w[p + "mix.o"], w[p + "mix.o.b"] = lin(W, H * dv), (0.1 * rnd(W)).to(bf)
        if cfg.get("mlp"):
            w[p + "mlp.up"], w[p + "mlp.down"] = lin(cfg["mlp"]["ff"], W), lin(W, cfg["mlp"]["ff"])
    return w
