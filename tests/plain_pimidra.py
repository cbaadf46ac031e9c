"""Pimidra in plain float64 over whole sequences: the oracle of the tests.

One function per mechanism, written from the design's equations, sharing no code with the engine.
``cfg`` is the dictionary of ``config.json``; ``P`` maps tensor names to float64 tensors.  Every
function takes the rows of ONE sequence, positions counted from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ----------------------------------------------------------------------------- state-space mixer
def causal_conv(u, w, b):
    """``u [T, C]``, ``w [C, taps]`` (last column = the current token), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    out = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += u[:T - back] * w[:, j]
    return out + b


def mamba2(h, P, pre, m, eps):
    H, Vd, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * Vd
    p = h @ P[pre + "in"].T
    z, rest = p[:, :inner], p[:, inner:]
    xbc, dt = rest[:, :inner + 2 * G * N], rest[:, inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, P[pre + "conv"], P[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(-1, H, Vd)
    Bm = xbc[:, inner:inner + G * N].reshape(-1, G, N)
    Cm = xbc[:, inner + G * N:].reshape(-1, G, N)
    dt = softplus(dt + P[pre + "dt_bias"])                       # [T, H]
    decay = torch.exp(-torch.exp(P[pre + "A_log"]) * dt)         # [T, H]
    T = h.shape[0]
    y = torch.zeros(T, H, Vd, dtype=F64)
    per = H // G
    for n in range(H):
        g = n // per
        S = torch.zeros(N, Vd, dtype=F64)
        for t in range(T):
            S = decay[t, n] * S + dt[t, n] * torch.outer(Bm[t, g], x[t, n])
            y[t, n] = S.T @ Cm[t, g] + P[pre + "D"][n] * x[t, n]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = y.reshape(T, parts, inner // parts)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    y = y.reshape(T, inner) * P[pre + "norm"]
    return y @ P[pre + "o"].T


# ----------------------------------------------------------------------------- attention
def rotate_half(x, dims, base, factor):
    """``x [T, heads, dim]``: channel i < dims/2 pairs with i + dims/2."""
    T = x.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(half)], dtype=F64)
    a = torch.arange(T, dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def visible(T, chunk):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if chunk:
        ok &= (i // chunk) == (j // chunk)
    return ok


def attention(h, P, pre, m, eps, v_first):
    """Returns ``(output, the layer's values before mixing)``; ``v_first``: the values of the
    first value-mixing layer, or ``None`` in that layer (and in layers that do not mix)."""
    H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = h @ P[pre + "q"].T + P[pre + "q.b"]
    k = h @ P[pre + "k"].T + P[pre + "k.b"]
    v = h @ P[pre + "v"].T + P[pre + "v.b"]
    q = rms_norm(q, P[pre + "q.norm"], eps).reshape(T, H, D)
    k = rms_norm(k, P[pre + "k.norm"], eps).reshape(T, G, D)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_half(q, rot["dims"], rot["base"], factor)
        k = rotate_half(k, rot["dims"], rot["base"], factor)
    own = v
    if v_first is not None:
        lam = P[pre + "vmix"]
        v = (1 - lam) * v + lam * v_first
    v = v.reshape(T, G, Vd)
    ok = visible(T, (m.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, Vd, dtype=F64)
    per = H // G
    for n in range(H):
        s = (q[:, n] @ k[:, n // per].T) * m["scale"]
        s = s.masked_fill(~ok, -math.inf)
        out[:, n] = torch.softmax(s, dim=-1) @ v[:, n // per]
    return out.reshape(T, H * Vd) @ P[pre + "o"].T, own


# ----------------------------------------------------------------------------- gated linear attention
def gla(h, P, pre, m, eps):
    H, D, Vd, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    q = (h @ P[pre + "q"].T * D ** -0.5).reshape(T, H, D)
    k = (h @ P[pre + "k"].T).reshape(T, H, D)
    v = (h @ P[pre + "v"].T).reshape(T, H, Vd)
    z = (h @ P[pre + "a1"].T) @ P[pre + "a2"].T + P[pre + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / tau)).reshape(T, H, D)
    o = torch.zeros(T, H, Vd, dtype=F64)
    for n in range(H):
        S = torch.zeros(D, Vd, dtype=F64)
        for t in range(T):
            S = alpha[t, n][:, None] * S + torch.outer(k[t, n], v[t, n])
            o[t, n] = S.T @ q[t, n]
    o = rms_norm(o, P[pre + "norm"], eps).reshape(T, H * Vd)
    return (o * silu(h @ P[pre + "g"].T)) @ P[pre + "o"].T


# ----------------------------------------------------------------------------- feed-forwards
def dense_ff(h, P, pre):
    return (torch.relu(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def route(logits, top):
    """The ``top`` largest logits of each row (lowest index among equals) and the softmax over
    them alone."""
    vals, idx = torch.sort(logits, dim=-1, descending=True, stable=True)
    return idx[:, :top], torch.softmax(vals[:, :top], dim=-1)


def moe_ff(h, P, pre, mlp):
    top = mlp["router"]["top"]
    idx, w = route(h @ P[pre + "router"].T, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = f"{pre}e{int(idx[t, c])}."
            y = (silu(P[e + "gate"] @ h[t]) * (P[e + "up"] @ h[t]))
            out[t] += w[t, c] * (P[e + "down"] @ y)
    return out


# ----------------------------------------------------------------------------- the model
def forward(cfg, tensors, tokens, without=()):
    """Logits ``[T, vocab]`` and the stream after every layer ``[L, T, width]`` of one sequence.
    ``without``: mechanisms to leave out (tests show that each one matters): ``"alpha"``,
    ``"chunk"``, ``"vmix"``, ``"scaling"``."""
    P = {k: v.to(F64) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    alpha = 1.0 if "alpha" in without else cfg["postln_alpha"]
    x = P["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    v_first, after = None, []
    for i, L in enumerate(cfg["layers"]):
        m, pre = dict(L["mixer"]), f"l{i}.mix."
        if "chunk" in without:
            m.pop("mask", None)
        if "scaling" in without and m.get("rot"):
            m["rot"] = {k: v for k, v in m["rot"].items() if k != "scaling"}
        if L["type"] == "mamba2":
            a = mamba2(x, P, pre, m, eps)
        elif L["type"] == "gla":
            a = gla(x, P, pre, m, eps)
        else:
            mixing = m.get("v_mix") and "vmix" not in without
            a, own = attention(x, P, pre, m, eps, v_first if mixing else None)
            if mixing and v_first is None:
                v_first = own
        x = rms_norm(alpha * x + a, P[f"l{i}.norm1"], eps)
        mlp = L.get("mlp")
        if mlp is not None:
            f = dense_ff(x, P, f"l{i}.mlp.") if mlp["kind"] == "dense" \
                else moe_ff(x, P, f"l{i}.mlp.", mlp)
            x = rms_norm(alpha * x + f, P[f"l{i}.norm2"], eps)
        after.append(x)
    logits = rms_norm(x, P["final.norm"], eps) @ P["head"].T
    return logits, torch.stack(after)
