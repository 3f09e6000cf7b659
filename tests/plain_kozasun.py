"""A plain, slow implementation of the Kozasun decoder in float64, one function per mechanism.

It runs a whole sequence at once, keeps no cache and no state (the retention starts from zero and walks every token)
and shares no code with the engine: the engine's kernels, parts and step function are compared with it.  ``weights``
maps checkpoint tensor names to float64 torch tensors on the CPU; ``config`` is the parsed config.json.

Notation: every matrix is stored [out, in] and applied as x @ W.T; positions are 0 .. T - 1.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- small pieces
def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var = mean squared deviation."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    """x over the root of its mean square along the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_half(x, base, dims):
    """x [T, heads, dim]: coordinate i < dims/2 is paired with i + dims/2 and the pair turned by t * base^(-2i/dims)."""
    if not dims:
        return x
    T = x.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = torch.arange(T, dtype=F64)[:, None] * torch.pow(torch.tensor(base, dtype=F64), -2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def visible(T, kind, size):
    """[T, T] mask: query i sees key j.  kind "chunk": j <= i in the same block of ``size`` positions counted from 0;
    "window": 0 <= i - j < size; None: j <= i."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if kind == "chunk":
        ok = ok & (i // size == j // size)
    elif kind == "window":
        ok = ok & (i - j < size)
    return ok


def softmax_with_sink(scores, ok, sink=None):
    """Weights over the visible keys; with ``sink`` [heads] the denominator also holds exp(sink).  scores [H, T, T]."""
    s = scores.masked_fill(~ok[None], -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


# ----------------------------------------------------------------------------- mixers
def attention(h, w, p, m, eps):
    """Grouped-query attention with biased projections, one RMS norm over the whole q (and k) row, a rotated prefix of
    each head, chunked visibility and a sink in the softmax's denominator."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    q, k, v = q.view(T, H, dk), k.view(T, G, dk), v.view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate_half(q, rot["base"], rot["dims"]), rotate_half(k, rot["base"], rot["dims"])
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    mask = m.get("mask")
    ok = visible(T, "chunk" if mask else None, mask["size"] if mask else 0)
    pw = softmax_with_sink(scores, ok, w[p + "sink"])
    o = torch.einsum("hij,jhd->ihd", pw, v).reshape(T, H * dv)
    return o @ w[p + "o"].T


def retention(h, w, p, m, eps):
    """Linear attention with one fixed decay per head: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate_half(q, rot["base"], rot["dims"]), rotate_half(k, rot["base"], rot["dims"])
    k = k * dk ** -0.5
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = unit_rms(o, eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Attention whose keys and values are expanded from a normed low-rank latent, over a sliding window, each head's
    result times a sigmoid gate."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    c = unit_rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).view(T, H, dk)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    mask = m.get("mask")
    ok = visible(T, "window" if mask else None, mask["size"] if mask else 0)
    pw = softmax_with_sink(scores, ok)
    o = torch.einsum("hij,jhd->ihd", pw, v)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


MIXERS = {"attention": attention, "retention": retention, "latent_attention": latent_attention}


# ----------------------------------------------------------------------------- feed-forwards
def gated(h, w, p, act):
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, r):
    """(chosen experts [T, top], their weights [T, top]).  Scores are sigmoids of the router's logits; the choice goes
    by score + correction among the experts of the ``keep`` best groups (a group's worth: its two largest choice
    scores added), the weights are the plain scores times ``scale``."""
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    T, E = s.shape
    groups = r.get("groups")
    if groups:
        n = groups["count"]
        per = choice.view(T, n, E // n)
        worth = per.topk(min(2, E // n), dim=-1).values.sum(dim=-1)
        best = worth.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros(T, n, dtype=torch.bool)
        allowed.scatter_(1, best, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(E // n, dim=1), -math.inf)
    idx = choice.topk(r["top"], dim=-1).indices
    return idx, s.gather(1, idx) * r.get("scale", 1.0)


def feed_forward(h, w, p, ff):
    if ff["kind"] == "dense":
        return gated(h, w, p, gelu_tanh)
    idx, wt = route(h, w, p, ff["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            out[t] += a * gated(h[t:t + 1], w, f"{p}e{e}.", silu)[0]
    if ff.get("shared"):
        out = out + gated(h, w, p + "shared.", silu)
    return out


# ----------------------------------------------------------------------------- the model
def hyper(xs, w, p, sub):
    """One sublayer over the streams xs [S, T, D]: it reads sum_s in[s] x_s and its output y rewrites every stream,
    x_t <- sum_s mix[s, t] x_s + out[t] y."""
    u = torch.einsum("s,std->td", w[p + "in"], xs)
    y = sub(u)
    return torch.einsum("st,sid->tid", w[p + "mix"], xs) + w[p + "out"][:, None, None] * y[None]


def forward(config, weights, tokens, on_layer=None):
    """Logits [T, vocab] of one sequence.  ``on_layer(run, x)`` sees the stream (the streams' sum) after every layer."""
    w = weights
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config.get("embedding", {}).get("scale", 1.0)
    S = config.get("streams")
    xs = x[None].repeat(S, 1, 1) if S else None
    for i, L in enumerate(config["layers"]):
        p = f"l{L.get('weights_of', i)}."
        mix = lambda u: MIXERS[L["type"]](layer_norm(u, w[p + "norm1"], w[p + "norm1.b"], eps), w, p + "mix.", L["mixer"], eps)  # noqa: E731
        ff = lambda u: feed_forward(layer_norm(u, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.", L["mlp"])               # noqa: E731
        if S:
            xs = hyper(xs, w, p + "hc1.", mix)
            if L.get("mlp"):
                xs = hyper(xs, w, p + "hc2.", ff)
            x = xs.sum(dim=0)
        else:
            x = x + mix(x)
            if L.get("mlp"):
                x = x + ff(x)
        if on_layer is not None:
            on_layer(i, x)
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
