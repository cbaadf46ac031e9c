"""Bapivik in plain float64 over whole sequences: the oracle of the tests.

One function per mechanism, written from the design's equations, sharing no code with the engine.
``cfg`` is the dictionary of ``config.json``; ``P`` maps tensor names to float64 tensors.  Every
function takes the rows of ONE sequence, positions counted from 0.  ``rnd`` (identity by default)
is applied where the bfloat16 engine stores an activation in 16 bits.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def same(x):
    return x


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------------------- embedding
def embed(tokens, P, positions=True):
    """Token row plus the learned row of the token's position, unscaled."""
    T = len(tokens)
    x = P["embed"][torch.tensor(tokens)]
    return x + P["pos"][:T] if positions else x


# ----------------------------------------------------------------------------- lightning
def lightning(h, P, pre, m, eps, rnd=same):
    """Linear attention with one fixed decay a head: ``S <- a_n S + k v^T``, ``o = S^T q`` with
    q, k, v through SiLU; all heads' outputs normed together, gated by a sigmoid, projected."""
    H, D, Vd = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(rnd(h @ P[pre + "q"].T)).reshape(T, H, D)
    k = silu(rnd(h @ P[pre + "k"].T)).reshape(T, H, D)
    v = silu(rnd(h @ P[pre + "v"].T)).reshape(T, H, Vd)
    o = torch.zeros(T, H, Vd, dtype=F64)
    for n in range(H):
        a = float(m["decay"][n])
        S = torch.zeros(D, Vd, dtype=F64)
        for t in range(T):
            S = a * S + torch.outer(k[t, n], v[t, n])
            o[t, n] = S.T @ q[t, n]
    y = rms_norm(o.reshape(T, H * Vd), P[pre + "norm"], eps)
    y = rnd(y * torch.sigmoid(rnd(h @ P[pre + "g"].T)))
    return y @ P[pre + "o"].T


# ----------------------------------------------------------------------------- latent attention
def latent_of(h, P, pre, eps, rnd=same):
    """The normed latent vector a token keeps."""
    return rnd(rms_norm(rnd(h @ P[pre + "dkv"].T), P[pre + "dkv.norm"], eps))


def latent_attention(h, c, P, pre, m, eps, rnd=same, gated=True):
    """``c``: the latent vectors the layer reads (its own, or another layer's)."""
    H, D, Vd = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    cq = rnd(rms_norm(rnd(h @ P[pre + "dq"].T), P[pre + "dq.norm"], eps))
    q = rnd(cq @ P[pre + "uq"].T).reshape(T, H, D)
    k = (c @ P[pre + "uk"].T).reshape(T, H, D)
    v = (c @ P[pre + "uv"].T).reshape(T, H, Vd)
    gate = torch.sigmoid(rnd(h @ P[pre + "g"].T))             # [T, H]
    out = torch.zeros(T, H, Vd, dtype=F64)
    for n in range(H):
        s = (q[:, n] @ k[:, n].T) * m["scale"]
        i = torch.arange(T)
        s = s.masked_fill(i[None, :] > i[:, None], -math.inf)
        out[:, n] = torch.softmax(s, dim=-1) @ v[:, n]
    out = rnd(out * gate[:, :, None]) if gated else rnd(out)
    return out.reshape(T, H * Vd) @ P[pre + "o"].T


# ----------------------------------------------------------------------------- attention
def query_temperature(T, coef, every):
    p = torch.arange(T, dtype=F64)
    return 1.0 + coef * torch.log(torch.floor((p + 1) / every) + 1.0)


def visible(T, window):
    """``[i, j]`` true where query ``i`` sees key ``j``: itself and the ``window - 1`` before."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window:
        ok = ok & (i - j < window)
    return ok


def attention(h, P, pre, m, eps, rnd=same, without=()):
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = rnd(h @ P[pre + "q"].T).reshape(T, H, D)
    k = rnd(h @ P[pre + "k"].T).reshape(T, G, D)
    v = k                                                     # the keys as projected
    q = rms_norm(q, P[pre + "q.norm"], eps)
    kn = rnd(rms_norm(k, P[pre + "k.norm"], eps))
    qt = m.get("q_temp")
    if qt and "q_temp" not in without:
        q = q * query_temperature(T, qt["coef"], qt["every"])[:, None, None]
    q = rnd(q)
    ok = visible(T, 0 if "window" in without else (m.get("mask") or {}).get("size", 0))
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(F64)
    cap = None if "softcap" in without else m.get("softcap")
    out = torch.zeros(T, H, D, dtype=F64)
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ kn[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        if "slopes" not in without:
            s = s - 2.0 ** (-8.0 * (n + 1) / H) * dist
        s = s.masked_fill(~ok, -math.inf)
        out[:, n] = torch.softmax(s, dim=-1) @ v[:, g]
    return rnd(out.reshape(T, H * D)) @ P[pre + "o"].T


# ----------------------------------------------------------------------------- feed-forward
def dense(h, P, pre, rnd=same):
    u = rnd(h @ P[pre + "up"].T + P[pre + "up.b"])
    return rnd(torch.relu(u) ** 2) @ P[pre + "down"].T + P[pre + "down.b"]


# ----------------------------------------------------------------------------- the model
def forward(cfg, P, tokens, rnd=same, layers_out=None, without=()):
    """Logits ``[T, vocab]`` of one sequence.  ``layers_out``: a list that receives the stream
    after every layer (after the depth average).  ``without``: mechanisms to leave out (``pos``,
    ``dwa``, ``norm_b``, ``gate``, ``shared``, ``q_temp``, ``softcap``, ``slopes``, ``window``,
    ``logit_cap``), so that a test can show that each one moves the logits."""
    eps = cfg["norm"]["eps"]
    x = embed(tokens, P, "pos" not in without)

    def out_norm(y, name):
        return y if "norm_b" in without else rms_norm(y, P[name], eps)
    X = [x]                                      # the embedding output and every layer's result
    latents = {}
    for i, L in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", L["mixer"]
        h = rnd(rms_norm(x, P[pre + "norm1"], eps))
        if L["type"] == "lightning":
            a = lightning(h, P, pre + "mix.", m, eps, rnd)
        elif L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is not None and "shared" in without:      # as if it read the layer before it
                src = max(k for k in latents if k < i)
            if src is None:
                latents[i] = latent_of(h, P, pre + "mix.", eps, rnd)
                src = i
            a = latent_attention(h, latents[src], P, pre + "mix.", m, eps, rnd,
                                 gated="gate" not in without)
        elif L["type"] == "attention":
            a = attention(h, P, pre + "mix.", m, eps, rnd, without)
        else:
            raise ValueError(L["type"])
        x = x + out_norm(a, pre + "norm1b")
        if L.get("mlp") is not None:
            h = rnd(rms_norm(x, P[pre + "norm2"], eps))
            x = x + out_norm(dense(h, P, pre + "mlp.", rnd), pre + "norm2b")
        X.append(x)
        w = P[pre + "dwa"]
        if "dwa" not in without:
            x = sum(w[j] * X[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x)
    y = rnd(rms_norm(x, P["final.norm"], eps))
    logits = y @ P["embed"].T
    cap = cfg.get("logit_softcap")
    if cap and "logit_cap" not in without:
        logits = cap * torch.tanh(logits / cap)
    return logits
