"""Plain, slow restatement of the Vilosun design: one function per mechanism, whole sequences, float64, no cache.

It is the oracle of the Vilosun tests and shares nothing with ``nanorlhf_b200``: weights come in as a dict
``name -> tensor`` with the checkpoint's names, the configuration as the dict ``config.json`` holds.
Every function works on ONE sequence ``[T, ...]`` and loops over time where the design is recurrent.

Notation: x is the residual stream [T, width]; h the (normed) input of a sublayer; i, j are positions from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def lin(w, x, b=None):
    y = x @ w.to(F64).T
    return y if b is None else y + b.to(F64)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def group_rmsnorm(x, w, groups, eps):
    """The vector is cut into ``groups`` equal consecutive parts; each is divided by sqrt(mean(part^2) + eps); then times w."""
    T, n = x.shape
    xp = x.view(T, groups, n // groups)
    xp = xp / torch.sqrt((xp * xp).mean(-1, keepdim=True) + eps)
    return xp.reshape(T, n) * w.to(F64)


def embed(tokens, W, cfg):
    """Token row times a constant plus a hashed row for the (previous, current) pair; the first token takes the spare row."""
    e = cfg["embedding"]
    x = W["embed"].to(F64)[tokens] * e["scale"]
    bg = e.get("bigram")
    if bg is not None:
        rows = []
        for i, t in enumerate(tokens):
            rows.append(bg["buckets"] if i == 0 else (tokens[i - 1] * bg["mul_prev"] + t * bg["mul_cur"]) % bg["buckets"])
        x = x + W["bigram"].to(F64)[rows]
    return x


def causal_conv(u, w):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start.  u [T, C], w [C, taps]."""
    T, C = u.shape
    taps = w.shape[1]
    up = torch.cat([torch.zeros(taps - 1, C, dtype=F64), u], 0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y = y + up[j:j + T] * w[:, j].to(F64)
    return y


def distance_slopes(H):
    """Head h of H (from 0) loses 2^(-8 (h + 1) / H) of score per position between query and key."""
    return [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]


def chunk_softmax_attention(q, k, v, size, scale, temp=None, slopes=None):
    """Core of the attention mixer on given q [T, H, D], k [T, G, D], v [T, G, Dv]: position i attends to j <= i with
    floor(i / size) == floor(j / size); score = q.k * scale * temp[h] - slopes[h] * (i - j); ordinary softmax."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(T):
        lo = (i // size) * size
        dist = torch.arange(i - lo, -1, -1, dtype=F64)       # i - j for j = lo .. i
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hh]) * scale
            if temp is not None:
                s = s * temp[hh]
            if slopes is not None:
                s = s - slopes[hh] * dist
            out[i, hh] = torch.softmax(s, 0) @ v[lo:i + 1, g]
    return out


def chunk_attention(h, W, p, m, v_first=None):
    """The attention mixer: biased projections, short convolutions, value blending, chunked attention, a sigmoid gate per head.
    Returns (mixer output, the values that were attended = what a cache would hold)."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(lin(W[p + "q"], h, W[p + "q.b"]), W[p + "q.conv"]).view(T, H, D)
    k = causal_conv(lin(W[p + "k"], h, W[p + "k.b"]), W[p + "k.conv"]).view(T, G, D)
    v = causal_conv(lin(W[p + "v"], h, W[p + "v.b"]), W[p + "v.conv"]).view(T, G, Dv)
    if v_first is not None:
        lam = W[p + "vmix"].to(F64)
        v = (1 - lam) * v + lam * v_first
    out = chunk_softmax_attention(q, k, v, m["mask"]["size"], m["scale"], W[p + "temp"].to(F64), distance_slopes(H))
    out = out * torch.sigmoid(lin(W[p + "g"], h)).unsqueeze(-1)
    return lin(W[p + "o"], out.reshape(T, H * Dv)), v


def gated_delta(h, W, p, m, eps):
    """Gated delta rule, one decay per head; state [dim, vdim] per head, read after the token's own write."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(lin(W[p + "q"], h), W[p + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(lin(W[p + "k"], h), W[p + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(lin(W[p + "v"], h), W[p + "v.conv"])).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(W[p + "b"], h))
    decay = torch.exp(-torch.exp(W[p + "A_log"].to(F64)) * softplus(lin(W[p + "a"], h) + W[p + "dt_bias"].to(F64)))
    S = torch.zeros(H, D, Dv, dtype=F64)
    o = torch.zeros(T, H, Dv, dtype=F64)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = decay[t, hh] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ k[t, g])
            S[hh] = S[hh] + torch.outer(k[t, g], u)
            o[t, hh] = S[hh].T @ q[t, g]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * W[p + "norm"].to(F64)
    o = o.reshape(T, H * Dv) * silu(lin(W[p + "g"], h))
    return lin(W[p + "o"], o)


def moe(h, W, p, mlp):
    """Each token goes to the ``top`` experts with the largest router logits, weighted by the softmax over those logits only."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = lin(W[p + "router"], h, W[p + "router.b"])
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(z[t, e]), e))[:top]
        wts = torch.softmax(z[t, order], 0)
        for wt, e in zip(wts, order):
            q = f"{p}e{e}."
            a = silu(lin(W[q + "gate"], h[t:t + 1])) * lin(W[q + "up"], h[t:t + 1])
            out[t] += wt * lin(W[q + "down"], a)[0]
    return out


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer)."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = embed(list(tokens), W, cfg)
    v_first = None
    per_layer = []
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        h = group_rmsnorm(x, W[L + "norm1"], groups, eps)
        if layer["type"] == "attention":
            mix = layer["mixer"]
            use = bool(mix.get("v_mix"))
            y, v = chunk_attention(h, W, L + "mix.", mix, v_first if use else None)
            if use and v_first is None:
                v_first = v
        elif layer["type"] == "delta":
            y = gated_delta(h, W, L + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        y = y * torch.sigmoid(lin(W[L + "rg1"], h, W[L + "rg1.b"]))
        x = x + group_rmsnorm(y, W[L + "norm1b"], groups, eps)
        if layer.get("mlp") is not None:
            h = group_rmsnorm(x, W[L + "norm2"], groups, eps)
            y = moe(h, W, L + "mlp.", layer["mlp"])
            y = y * torch.sigmoid(lin(W[L + "rg2"], h, W[L + "rg2.b"]))
            x = x + group_rmsnorm(y, W[L + "norm2b"], groups, eps)
        per_layer.append(x.clone())
    xf = group_rmsnorm(x, W["final.norm"], groups, eps)
    logits = lin(W["head"], xf) * cfg["logit_scale"]
    return (logits, per_layer) if return_layers else logits


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Random tensors under the checkpoint's names for a config dict (tests make their own small models)."""
    g = torch.Generator().manual_seed(seed)
    W, width = {}, cfg["width"]

    def rn(*shape, s=1.0):
        return torch.randn(*shape, generator=g) * s

    def gain(n):
        return torch.rand(n, generator=g) * 0.5 + 0.75
    W["embed"] = rn(cfg["vocab"], width, s=0.5)
    bg = cfg["embedding"].get("bigram")
    if bg is not None:
        W["bigram"] = rn(bg["buckets"] + 1, width, s=0.5)
    for i, layer in enumerate(cfg["layers"]):
        L, m = f"l{i}.", layer["mixer"]
        has_ff = layer.get("mlp") is not None
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if has_ff else ()):
            W[L + n] = gain(width)
        for r in ("rg1",) + (("rg2",) if has_ff else ()):
            W[L + r] = rn(width, width, s=width ** -0.5)
            W[L + r + ".b"] = rn(width, s=0.5)
        p = L + "mix."
        H, G, D, Dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        if layer["type"] == "attention":
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                W[p + n] = rn(rows, width, s=width ** -0.5)
                W[p + n + ".b"] = rn(rows, s=0.2)
                W[p + n + ".conv"] = rn(rows, taps, s=taps ** -0.5)
            W[p + "vmix"] = torch.rand((), generator=g) * 0.6 + 0.2
            W[p + "temp"] = torch.rand(H, generator=g) + 0.5
            W[p + "g"] = rn(H, width, s=width ** -0.5)
            W[p + "o"] = rn(width, H * Dv, s=(H * Dv) ** -0.5)
        else:
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                W[p + n] = rn(rows, width, s=width ** -0.5)
                W[p + n + ".conv"] = rn(rows, taps, s=taps ** -0.5)
            W[p + "b"] = rn(H, width, s=width ** -0.5)
            W[p + "a"] = rn(H, width, s=width ** -0.5)
            W[p + "A_log"] = torch.rand(H, generator=g) * 2.0 - 1.5
            W[p + "dt_bias"] = torch.rand(H, generator=g) * 2.5 - 3.0
            W[p + "norm"] = gain(Dv)
            W[p + "g"] = rn(H * Dv, width, s=width ** -0.5)
            W[p + "o"] = rn(width, H * Dv, s=(H * Dv) ** -0.5)
        mlp = layer.get("mlp")
        if mlp is not None:
            q, ff = L + "mlp.", mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                W[f"{q}e{e}.gate"] = rn(ff, width, s=width ** -0.5)
                W[f"{q}e{e}.up"] = rn(ff, width, s=width ** -0.5)
                W[f"{q}e{e}.down"] = rn(width, ff, s=ff ** -0.5)
            W[q + "router"] = rn(mlp["router"]["experts"], width, s=2.0 * width ** -0.5)
            W[q + "router.b"] = rn(mlp["router"]["experts"], s=0.3)
    W["final.norm"] = gain(width)
    W["head"] = rn(cfg["vocab"], width, s=width ** -0.5)
    return {k: v.to(dtype) for k, v in W.items()}


def make_config(vocab=97, width=48, layers=("attention", "delta"), groups=2, eps=1e-5, embed_scale=3.0, logit_scale=0.5,
                bigram=(61, 7, 13), attn=None, delta=None, moe=None, v_mix=None, chunk=None):
    """A small config dict.  ``attn`` / ``delta`` / ``moe`` override sizes; ``v_mix`` / ``chunk``: per attention layer (in order)
    lists overriding the flag / the chunk length; ``moe=None`` in a position of ``layers`` spelled "attention-" or "delta-"
    drops that layer's feed-forward."""
    a = dict(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, size=6, scale=0.4)
    a.update(attn or {})
    d = dict(heads=4, kv_heads=2, dim=12, vdim=8, conv=2)
    d.update(delta or {})
    f = dict(ff=16, experts=5, top=2)
    f.update(moe or {})
    out, na = [], 0
    for kind in layers:
        bare = kind.endswith("-")
        kind = kind.rstrip("-")
        mlp = None if bare else {"kind": "moe", "expert": {"ff": f["ff"]}, "router": {"experts": f["experts"], "top": f["top"]}}
        if kind == "attention":
            m = {"heads": a["heads"], "kv_heads": a["kv_heads"], "dim": a["dim"], "vdim": a["vdim"], "conv": a["conv"],
                 "scale": a["scale"], "mask": {"size": chunk[na] if chunk else a["size"]}, "v_mix": v_mix[na] if v_mix else True}
            na += 1
        else:
            m = {"heads": d["heads"], "kv_heads": d["kv_heads"], "dim": d["dim"], "vdim": d["vdim"], "conv": d["conv"]}
        out.append({"type": kind, "mixer": m, "mlp": mlp})
    emb = {"scale": embed_scale}
    if bigram:
        emb["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    return {"architecture": "Vilosun", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "embedding": emb,
            "logit_scale": logit_scale, "layers": out}
