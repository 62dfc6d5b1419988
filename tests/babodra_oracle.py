"""Slow plain restatement of the Babodra design in float64 / float32 torch on the CPU, one function per mechanism.
It shares no code with proxy_inference_engine_b200: the tests compare the served model with it.

Notation: x residual [T, W]; a sublayer reads x and the residual takes its NORMED output, x <- x + rms(f(x)) * w.
Linear weights are [out, in].  ``rnd`` is the rounding applied to the inputs of matrix products (identity for the
exact mode, bf16 round trip to imitate the served mode)."""
from __future__ import annotations

import math

import torch


def ident(t):
    return t


def bf16_round(t):
    return t.to(torch.bfloat16).to(t.dtype)


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def lin(x, w, b=None, rnd=ident):
    y = rnd(x) @ rnd(w).T
    return y if b is None else y + b


def head_slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float64)


def query_temperature(pos, coef, every):
    return 1.0 + coef * torch.log(torch.floor((pos + 1) / every) + 1.0)


def sink_attention(q, k, v, scale, slopes, group):
    """q [T, H, d], k [T, G, d], v [T, G, dv]: causal softmax over s_ij = q_i.k_j scale - slope_h (i - j) with one extra
    term of score 0 in the denominator that carries no value."""
    T, H, _ = q.shape
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    i = torch.arange(T)
    dist = (i[:, None] - i[None, :]).to(q.dtype)
    for h in range(H):
        g = h // group
        s = (q[:, h] @ k[:, g].T) * scale - slopes[h].to(q.dtype) * dist
        s = s.masked_fill(dist < 0, float("-inf"))
        m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - m)
        out[:, h] = (e / (torch.exp(-m) + e.sum(-1, keepdim=True))) @ v[:, g]
    return out


def attention_mixer(x, w, p, cfg, eps, rnd=ident):
    """The whole mixer on one sequence from position 0: x [T, W] -> [T, W]."""
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    T = x.shape[0]
    q = lin(x, w[p + "q"], w[p + "q.b"], rnd)
    k = lin(x, w[p + "k"], w[p + "k.b"], rnd)
    v = k                                              # the values are the projected keys, before their norm
    q = rms(q, eps) * w[p + "q.norm"]                  # one norm over all heads' features together
    k = rms(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T, dtype=x.dtype)
    qt = cfg.get("q_temp")
    if qt:
        q = q * query_temperature(pos, qt["coef"], qt["every"])[:, None]
    o = sink_attention(rnd(q).view(T, H, d), rnd(k).view(T, G, d), rnd(v).view(T, G, dv), cfg["scale"], head_slopes(H),
                       H // G)
    gate = torch.sigmoid(lin(x, w[p + "g"], None, rnd))
    return lin(o.reshape(T, H * dv) * gate, w[p + "o"], None, rnd)


def dense_ff(x, w, p, cfg, rnd=ident):
    lim = cfg["limit"]
    g = torch.clamp(lin(x, w[p + "gate"], None, rnd), max=lim)
    u = torch.clamp(lin(x, w[p + "up"], None, rnd), min=-lim, max=lim)
    return lin(g * torch.sigmoid(1.702 * g) * (u + 1.0), w[p + "down"], None, rnd)


def silu_expert(x, w, p, rnd=ident):
    g = lin(x, w[p + "gate"], None, rnd)
    return lin(g * torch.sigmoid(g) * lin(x, w[p + "up"], None, rnd), w[p + "down"], None, rnd)


def route(x, w_router, r, rnd=ident, margins=None):
    """-> (chosen expert ids [T, top], their weights [T, top]).  margins: if a list, gets per token the smallest gap by
    which a choice was made (last kept group against the next one, last chosen expert against the next eligible one):
    a token with a tiny margin may legitimately be routed otherwise by an implementation that rounds differently."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(lin(x, w_router, None, rnd))
    grp = r.get("groups") or {"count": 1, "keep": 1}
    n, keep = grp["count"], grp["keep"]
    per = E // n
    gs = s.view(-1, n, per)
    gscore = gs.topk(min(2, per), -1).values.sum(-1)                 # a group counts by its two best experts
    kept = gscore.topk(keep, -1).indices
    allowed = torch.zeros((x.shape[0], n), dtype=torch.bool).scatter_(1, kept, True)
    masked = torch.where(allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), s, torch.full_like(s, -1.0))
    idx = masked.topk(top, -1).indices
    if margins is not None:
        m = torch.full((x.shape[0],), float("inf"), dtype=s.dtype)
        if keep < n:
            gv = gscore.sort(-1, descending=True).values
            m = torch.minimum(m, gv[:, keep - 1] - gv[:, keep])
        if top < keep * per:
            ev = masked.sort(-1, descending=True).values
            m = torch.minimum(m, ev[:, top - 1] - ev[:, top])
        margins.append(m)
    return idx, s.gather(1, idx) * r["scale"]


def moe_ff(x, w, p, cfg, rnd=ident, margins=None):
    idx, wt = route(x, w[p + "router"], cfg["router"], rnd, margins)
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            y[t] += a * silu_expert(x[t:t + 1], w, f"{p}e{e}.", rnd)[0]
    if cfg.get("shared"):
        y = y + torch.sigmoid(lin(x, w[p + "shared.sg"], None, rnd)) * silu_expert(x, w, p + "shared.", rnd)
    return y


def forward(config, weights, tokens, dtype=torch.float64, rnd=ident, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence fed whole from position 0.  margins: if a list, one tensor [T] per mixture
    layer is appended (see route)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    T = len(tokens)
    x = w["embed"][torch.tensor(tokens)] + w["pos"][:T]
    for i, ly in enumerate(config["layers"]):
        p = f"l{i}."
        x = x + rms(attention_mixer(x, w, p + "mix.", ly["mixer"], eps, rnd), eps) * w[p + "norm1"]
        mlp = ly.get("mlp")
        if mlp:
            f = dense_ff(x, w, p + "mlp.", mlp, rnd) if mlp["kind"] == "dense" else moe_ff(x, w, p + "mlp.", mlp, rnd, margins)
            x = x + rms(f, eps) * w[p + "norm2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(rms(x, eps) * w["final.norm"], w["head"], None, rnd)


def random_config(vocab=96, width=48, n_layers=3, heads=4, kv_heads=2, dim=16, ff=40, experts=6, top=2, groups=(3, 2),
                  expert_ff=24, shared_ff=20, max_positions=512, scale=None, q_temp=(0.37, 24), kinds=None):
    """A small configuration of the design; kinds: per layer "dense" | "moe" | None."""
    kinds = kinds or (["dense", "moe", None] * n_layers)[:n_layers]
    layers = []
    for kind in kinds:
        mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale or dim ** -0.5}
        if q_temp:
            mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
        if kind == "dense":
            mlp = {"kind": "dense", "ff": ff, "limit": 0.8}
        elif kind == "moe":
            mlp = {"kind": "moe", "expert": {"ff": expert_ff},
                   "router": {"experts": experts, "top": top, "scale": 1.7, "groups": {"count": groups[0], "keep": groups[1]}},
                   "shared": {"ff": shared_ff} if shared_ff else None}
        else:
            mlp = None
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Babodra", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": 1e-5}, "layers": layers}
