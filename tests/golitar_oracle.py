"""Plain, slow restatement of the Golitar design in float64 torch on the CPU: one function per mechanism, whole
sequences at a time, no cache, no batching.  The tests compare the engine with it; it shares no code with the package.

Notation: x [T, W] residual (or S streams of it), weights stored [out, in] and applied as x @ W.T.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def _w(weights, name):
    return weights[name].to(F64)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_centered(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(x, taps_w):
    """x [T, C], taps_w [C, taps] (last column multiplies the current token); zeros before the start."""
    T, C = x.shape
    n = taps_w.shape[1]
    pad = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + pad[j:j + T] * taps_w[:, j]
    return y


def delta_recurrence(q, k, v, beta, g):
    """q, k [T, H, dk]; v [T, H, dv]; beta, g [T, H].  One matrix state per head, start at zero.  For each token:
    decay, then write the error-corrected value under key k, then read with q (the read sees the write)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = S * g[t][:, None, None]
        pred = torch.einsum("hkv,hk->hv", S, k[t])
        u = beta[t][:, None] * (v[t] - pred)
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def delta_mixer(h, weights, p, m, eps):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    proj = {}
    for n in ("q", "k", "v"):
        z = h @ _w(weights, p + n).T
        proj[n] = silu(causal_conv(z, _w(weights, p + n + ".conv")) if (p + n + ".conv") in weights else z)
    q = proj["q"].view(T, G, dk)
    k = proj["k"].view(T, G, dk)
    v = proj["v"].view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q = q.repeat_interleave(rep, 1)
    k = k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(h @ _w(weights, p + "b").T)
    dt = torch.nn.functional.softplus(h @ _w(weights, p + "a").T + _w(weights, p + "dt_bias"))
    g = torch.exp(-torch.exp(_w(weights, p + "A_log")) * dt)
    o = delta_recurrence(q, k, v, beta, g)
    o = unit_rms(o, eps) * _w(weights, p + "norm")
    gate = silu(h @ _w(weights, p + "g").T).view(T, H, dv)
    return (o * gate).reshape(T, H * dv) @ _w(weights, p + "o").T


def rotary_freqs(rot):
    d = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / d) for i in range(d // 2)], dtype=F64)
    sc = rot.get("scaling")
    if sc:
        fac, lo, hi, orig = sc["factor"], sc["low"], sc["high"], sc["original"]
        out = []
        for fi in f.tolist():
            lam = 2 * math.pi / fi
            if lam < orig / hi:
                out.append(fi)
            elif lam > orig / lo:
                out.append(fi / fac)
            else:
                s = (orig / lam - lo) / (hi - lo)
                out.append((1 - s) * fi / fac + s * fi)
        f = torch.tensor(out, dtype=F64)
    return f


def rotate_pairs(x, pos, freqs):
    """x [T, ..., D]; the first 2 * len(freqs) features are rotated in adjacent pairs."""
    d = 2 * freqs.numel()
    ang = pos.to(F64)[:, None] * freqs[None]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [d // 2]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    a, b = x[..., 0:d:2], x[..., 1:d:2]
    y = x.clone()
    y[..., 0:d:2] = a * c - b * s
    y[..., 1:d:2] = b * c + a * s
    return y


def windowed_softmax_attention(q, k, v, scale, cap, window):
    """q [T, H, d], k [T, H, d], v [T, H, dv] (already expanded to query heads).  Causal; window = visible keys or None."""
    T = q.shape[0]
    s = torch.einsum("thd,shd->hts", q, k) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None]
    vis = (j <= i)
    if window:
        vis = vis & (i - j < window)
    s = s.masked_fill(~vis, float("-inf"))
    return torch.einsum("hts,shv->thv", torch.softmax(s, -1), v)


def diff_attention_mixer(h, weights, p, m, eps, pos=None):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T) if pos is None else pos

    def lin(n):
        y = h @ _w(weights, p + n).T
        return y + _w(weights, p + n + ".b") if (p + n + ".b") in weights else y
    q = lin("q").view(T, H, 2, d)
    k = lin("k").view(T, G, 2, d)
    v = lin("v").view(T, G, dv)
    q = unit_rms(q, eps) * _w(weights, p + "q.norm")
    k = unit_rms(k, eps) * _w(weights, p + "k.norm")
    if m.get("rot"):
        fr = rotary_freqs(m["rot"])
        q, k = rotate_pairs(q, pos, fr), rotate_pairs(k, pos, fr)
    rep = H // G
    k = k.repeat_interleave(rep, 1)
    v = v.repeat_interleave(rep, 1)
    window = (m.get("mask") or {}).get("size")
    maps = [windowed_softmax_attention(q[:, :, i], k[:, :, i], v, m["scale"], m.get("softcap"), window) for i in (0, 1)]
    diff = m["diff"]
    lam = (torch.exp((_w(weights, p + "lq1") * _w(weights, p + "lk1")).sum())
           - torch.exp((_w(weights, p + "lq2") * _w(weights, p + "lk2")).sum()) + diff)
    o = maps[0] - lam * maps[1]
    o = unit_rms(o, eps) * (1.0 - diff)
    y = o.reshape(T, H * dv) @ _w(weights, p + "o").T
    return y + _w(weights, p + "o.b") if (p + "o.b") in weights else y


def dense_ff(h, weights, p):
    z = torch.relu(h @ _w(weights, p + "up").T)
    return (z * z) @ _w(weights, p + "down").T


def hyper_step(xs, weights, p, fn):
    """xs [S, T, W]: read one input as a weighted sum of the streams, run the sublayer, mix the streams and add its
    output to each with its own weight."""
    a, o, mx = _w(weights, p + "in"), _w(weights, p + "out"), _w(weights, p + "mix")
    u = torch.einsum("s,stw->tw", a, xs)
    y = fn(u)
    return torch.einsum("st,sqw->tqw", mx, xs) + o[:, None, None] * y[None]


def forward(cfg, weights, tokens, return_layers=False):
    """tokens: list of ints -> logits [T, vocab] (float64); optionally also the summed residual after every layer."""
    eps = cfg["norm"]["eps"]
    S = cfg.get("streams") or 1
    x = _w(weights, "embed")[torch.tensor(tokens)]
    xs = x[None].repeat(S, 1, 1)
    layers = []
    for i, ly in enumerate(cfg["layers"]):
        p = f"l{i}."
        mixer = {"delta": delta_mixer, "attention": diff_attention_mixer}[ly["type"]]
        subs = [("1", lambda u, p=p, ly=ly, mixer=mixer: mixer(norm_centered(u, _w(weights, p + "norm1"), eps), weights,
                                                                 p + "mix.", ly["mixer"], eps))]
        if ly.get("mlp"):
            subs.append(("2", lambda u, p=p: dense_ff(norm_centered(u, _w(weights, p + "norm2"), eps), weights, p + "mlp.")))
        for tag, fn in subs:
            if (p + f"hc{tag}.in") in weights:
                xs = hyper_step(xs, weights, p + f"hc{tag}.", fn)
            else:
                xs = xs + fn(xs.sum(0))[None]
        layers.append(xs.sum(0))
    x = norm_centered(xs.sum(0), _w(weights, "final.norm"), eps)
    logits = x @ _w(weights, "head" if "head" in weights else "embed").T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(layers)) if return_layers else logits
