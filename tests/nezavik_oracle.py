"""Plain, slow restatement of the Nezavik design: one function per mechanism, whole sequences, float64, no cache.

It is the oracle of the Nezavik tests and shares nothing with ``nanorlhf_b200``: weights come in as a dict
``name -> tensor`` with the checkpoint's names, the configuration as the dict ``config.json`` holds.
Every function works on ONE sequence ``[T, ...]`` and loops over time where the design is recurrent.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def lin(w, x):
    return x @ w.to(F64).T


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def scalar_rmsnorm(x, g, eps):
    """x / sqrt(mean(x^2) + eps) * g with ONE learned number g."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g.to(F64)


def causal_conv(x, w, bias=None):
    """Depthwise causal convolution over time. x [T, C], w [C, taps]; the last tap multiplies the current token."""
    T, C = x.shape
    taps = w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], 0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y = y + xp[j:j + T] * w[:, j].to(F64)
    if bias is not None:
        y = y + bias.to(F64)
    return y


def window_attention(h, W, p, m, eps):
    """Sliding-window softmax attention with per-head RMS-normed queries and keys, no positional rotation."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(W[p + "q"], h).view(T, H, D)
    k = lin(W[p + "k"], h).view(T, G, D)
    v = lin(W[p + "v"], h).view(T, G, Dv)
    q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * W[p + "q.norm"].to(F64)
    k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * W[p + "k.norm"].to(F64)
    win = m["mask"]["size"]
    out = torch.zeros(T, H, Dv, dtype=F64)
    for i in range(T):
        lo = max(0, i - win + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hh]) * m["scale"]
            out[i, hh] = torch.softmax(s, 0) @ v[lo:i + 1, g]
    return lin(W[p + "o"], out.reshape(T, H * Dv))


def ssd_mixer(h, W, p, m, eps):
    """State-space (Mamba-2 style) mixer: scalar decay per head, state [N, vdim] per head."""
    T = h.shape[0]
    Hh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hh * P
    u = lin(W[p + "in"], h)
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(T, Hh, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"].to(F64))
    A = torch.exp(W[p + "A_log"].to(F64))
    Dk = W[p + "D"].to(F64)
    S = torch.zeros(Hh, N, P, dtype=F64)
    y = torch.zeros(T, Hh, P, dtype=F64)
    for t in range(T):
        for hh in range(Hh):
            g = hh // (Hh // G)
            S[hh] = torch.exp(-A[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + Dk[hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = y.view(T, ng, inner // ng)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    y = y.reshape(T, inner) * W[p + "norm"].to(F64)
    return lin(W[p + "o"], y)


def delta_mixer(h, W, p, m, eps, per_channel):
    """Gated delta rule. ``per_channel``: one decay per head and key channel (low-rank projected) and a sigmoid
    low-rank output gate; otherwise one decay per head and a silu output gate."""
    T = h.shape[0]
    Hh, Hk, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(lin(W[p + "q"], h), W[p + "q.conv"])).view(T, Hk, D)
    k = silu(causal_conv(lin(W[p + "k"], h), W[p + "k.conv"])).view(T, Hk, D)
    v = silu(causal_conv(lin(W[p + "v"], h), W[p + "v.conv"])).view(T, Hh, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(W[p + "b"], h))
    A = torch.exp(W[p + "A_log"].to(F64))
    if per_channel:
        a = lin(W[p + "a2"], lin(W[p + "a1"], h)) + W[p + "dt_bias"].to(F64)
        decay = torch.exp(-A[None, :, None] * softplus(a).view(T, Hh, D))             # [T, Hh, D]
        gate = torch.sigmoid(lin(W[p + "g2"], lin(W[p + "g1"], h))).view(T, Hh, Dv)
    else:
        a = lin(W[p + "a"], h) + W[p + "dt_bias"].to(F64)
        decay = torch.exp(-A[None, :] * softplus(a))[:, :, None].expand(T, Hh, D)
        gate = silu(lin(W[p + "g"], h)).view(T, Hh, Dv)
    S = torch.zeros(Hh, D, Dv, dtype=F64)
    o = torch.zeros(T, Hh, Dv, dtype=F64)
    for t in range(T):
        for hh in range(Hh):
            g = hh // (Hh // Hk)
            S[hh] = decay[t, hh][:, None] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ k[t, g])
            S[hh] = S[hh] + torch.outer(k[t, g], u)
            o[t, hh] = S[hh].T @ q[t, g]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * W[p + "norm"].to(F64)
    return lin(W[p + "o"], (o * gate).reshape(T, Hh * Dv))


def feed_forward(h, W, p):
    return lin(W[p + "down"], torch.relu(lin(W[p + "up"], h)) ** 2)


def mixer(h, W, p, layer, eps):
    m = layer["mixer"]
    if layer["type"] == "parallel":
        left = window_attention(h, W, p + "left.", m["left"], eps)
        right = ssd_mixer(h, W, p + "right.", m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right
    if layer["type"] == "channel_delta":
        return delta_mixer(h, W, p, m, eps, True)
    if layer["type"] == "delta":
        return delta_mixer(h, W, p, m, eps, False)
    raise ValueError(layer["type"])


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    x = W["embed"].to(F64)[torch.as_tensor(tokens)] + W["pos"].to(F64)[:T]
    results = [x]                          # X_0 = embedding output, X_{i+1} = layer i's own result
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = scalar_rmsnorm(x, W[p + "norm1"], eps)
        y = mixer(h, W, p + "mix.", layer, eps)
        if layer.get("mlp") is not None:
            y = y + feed_forward(h, W, p + "mlp.")
        results.append(x + y)
        w = W[p + "dwa"].to(F64)
        x = sum(w[j] * results[j] for j in range(i + 2))
        streams.append(x)
    x = scalar_rmsnorm(x, W["final.norm"], eps)
    logits = lin(W["head"], x)
    return (logits, torch.stack(streams)) if return_layers else logits


# ---- small random models ---------------------------------------------------------------------------------------
def make_config(vocab=97, width=40, max_positions=256, layers=("parallel", "channel_delta", "delta"), eps=1e-5, seed_sizes=None):
    s = dict(heads=6, kv_heads=3, dim=24, vdim=16, window=11, scale=0.31, s_heads=4, s_vdim=12, s_state=20, s_groups=2,
             s_norm_groups=3, s_conv=3, d_heads=4, d_kv=2, d_dim=16, d_vdim=24, d_conv=4, ff=56, left_scale=0.7,
             right_scale=1.3)
    s.update(seed_sizes or {})
    out = []
    for t in layers:
        if t == "parallel":
            mx = {"left": {"dim": s["dim"], "heads": s["heads"], "kv_heads": s["kv_heads"], "mask": {"size": s["window"]},
                           "scale": s["scale"], "vdim": s["vdim"]},
                  "left_scale": s["left_scale"], "right_scale": s["right_scale"],
                  "right": {"conv": s["s_conv"], "groups": s["s_groups"], "heads": s["s_heads"],
                            "norm_groups": s["s_norm_groups"], "state": s["s_state"], "vdim": s["s_vdim"]}}
        else:
            mx = {"conv": s["d_conv"], "dim": s["d_dim"], "heads": s["d_heads"], "kv_heads": s["d_kv"], "vdim": s["d_vdim"]}
        out.append({"type": t, "mixer": mx, "mlp": {"ff": s["ff"], "kind": "dense"} if s["ff"] else None})
    return {"architecture": "Nezavik", "layers": out, "max_positions": max_positions, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


def make_weights(cfg, seed=0, dtype=torch.bfloat16, rank=8):
    """Random weights with the checkpoint's names and shapes, scaled so that activations stay O(1)."""
    g = torch.Generator().manual_seed(seed)
    Wd = cfg["width"]
    W = {}

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(dtype)

    def vec(n, lo, hi):
        return (torch.rand(n, generator=g) * (hi - lo) + lo).to(dtype)

    W["embed"] = (torch.randn(cfg["vocab"], Wd, generator=g)).to(dtype)
    W["pos"] = (torch.randn(cfg["max_positions"], Wd, generator=g) * 0.3).to(dtype)
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = layer["mixer"]
        W[p + "norm1"] = vec(1, 0.8, 1.2).reshape(())
        if layer["type"] == "parallel":
            a, r = m["left"], m["right"]
            q = p + "mix.left."
            W[q + "q"] = mat(a["heads"] * a["dim"], Wd)
            W[q + "k"] = mat(a["kv_heads"] * a["dim"], Wd)
            W[q + "v"] = mat(a["kv_heads"] * a["vdim"], Wd)
            W[q + "q.norm"] = vec(a["dim"], 0.5, 1.5)
            W[q + "k.norm"] = vec(a["dim"], 0.5, 1.5)
            W[q + "o"] = mat(Wd, a["heads"] * a["vdim"])
            q = p + "mix.right."
            inner = r["heads"] * r["vdim"]
            ch = inner + 2 * r["groups"] * r["state"]
            W[q + "in"] = mat(2 * inner + 2 * r["groups"] * r["state"] + r["heads"], Wd)
            W[q + "conv"] = mat(ch, r["conv"], 1.5)
            W[q + "conv.b"] = vec(ch, -0.2, 0.2)
            W[q + "dt_bias"] = vec(r["heads"], -2.0, 0.5)
            W[q + "A_log"] = vec(r["heads"], -1.5, 1.0)
            W[q + "D"] = vec(r["heads"], 0.5, 1.5)
            W[q + "norm"] = vec(inner, 0.5, 1.5)
            W[q + "o"] = mat(Wd, inner)
        else:
            q = p + "mix."
            nk, nv = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            for n, rows in (("q", nk), ("k", nk), ("v", nv)):
                W[q + n] = mat(rows, Wd, 2.0)
                W[q + n + ".conv"] = mat(rows, m["conv"], 1.5)
            W[q + "b"] = mat(m["heads"], Wd)
            W[q + "A_log"] = vec(m["heads"], -2.0, 0.5)
            W[q + "norm"] = vec(m["vdim"], 0.5, 1.5)
            if layer["type"] == "channel_delta":
                r = rank
                W[q + "a1"] = mat(r, Wd)
                W[q + "a2"] = mat(m["heads"] * m["dim"], r)
                W[q + "dt_bias"] = vec(m["heads"] * m["dim"], -3.0, 0.0)
                W[q + "g1"] = mat(r, Wd)
                W[q + "g2"] = mat(nv, r)
            else:
                W[q + "a"] = mat(m["heads"], Wd)
                W[q + "dt_bias"] = vec(m["heads"], -3.0, 0.0)
                W[q + "g"] = mat(nv, Wd)
            W[q + "o"] = mat(Wd, nv)
        if layer.get("mlp") is not None:
            W[p + "mlp.up"] = mat(layer["mlp"]["ff"], Wd)
            W[p + "mlp.down"] = mat(Wd, layer["mlp"]["ff"], 0.5)
        w = torch.rand(i + 2, generator=g) + 0.2
        W[p + "dwa"] = (w / w.sum()).to(dtype)
    W["final.norm"] = vec(1, 0.8, 1.2).reshape(())
    W["head"] = mat(cfg["vocab"], Wd)
    return W
