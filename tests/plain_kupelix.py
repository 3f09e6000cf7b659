"""A plain, slow implementation of the Kupelix decoder in float64, one function per mechanism.

It runs a whole sequence at once, keeps no cache and no state (recurrences start from zero and walk every token) and
shares no code with the engine: the engine's kernels, parts and step function are compared with it.  ``weights``
maps checkpoint tensor names to float64 torch tensors on the CPU; ``config`` is the parsed config.json.

Notation: every matrix is stored [out, in] and applied as x @ W.T; x is the residual stream [T, D].
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


def unit_length(x, eps):
    """x over its length along the last axis: x / sqrt(sum x^2 + eps)."""
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u, w):
    """out[t] = sum_j w[:, j] * u[t - (taps - 1) + j], zeros before the start.  u [T, C], w [C, taps]."""
    T, C = u.shape
    taps = w.shape[1]
    out = torch.zeros(T, C, dtype=u.dtype)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    ap = softplus(p)
    an = 0.5 + softplus(q)
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


# ----------------------------------------------------------------------------- rotation
def rotary_frequencies(rot):
    """f_i = base^(-2i/dims), rescaled by wavelength as Llama 3.1 does when ``scaling`` is given."""
    dims = int(rot["dims"])
    f = [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < orig / high:
                out.append(fi)
            elif wave > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate_pairs(x, rot):
    """x [T, heads, dim]: neighbouring pairs (2i, 2i+1) of the first ``dims`` coordinates turn by position * f_i."""
    dims = int(rot["dims"])
    T = x.shape[0]
    ang = torch.arange(T, dtype=F64)[:, None] * rotary_frequencies(rot)[None, :]      # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ----------------------------------------------------------------------------- mixers
def attention(h, weights, prefix, m, eps):
    """Causal softmax attention with normed and rotated queries and keys, scores mixed across heads, a sink in the
    denominator and a sigmoid gate per head."""
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    W = lambda n: weights[prefix + n]                                       # noqa: E731
    q = (h @ W("q").T + W("q.b")).reshape(T, H, dk)
    k = (h @ W("k").T + W("k.b")).reshape(T, G, dk)
    v = (h @ W("v").T + W("v.b")).reshape(T, G, dv)
    q = unit_rms(q, eps) * W("q.norm")
    k = unit_rms(k, eps) * W("k.norm")
    if m.get("rot"):
        q, k = rotate_pairs(q, m["rot"]), rotate_pairs(k, m["rot"])
    scores = torch.empty(H, T, T, dtype=F64)
    for hd in range(H):
        scores[hd] = (q[:, hd] @ k[:, hd // (H // G)].T) * float(m["scale"])
    scores = torch.einsum("hg,gij->hij", W("talk"), scores)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        for i in range(T):
            s = scores[hd, i, : i + 1]
            top = max(float(s.max()), float(W("sink")[hd]))
            e = torch.exp(s - top)
            den = e.sum() + math.exp(float(W("sink")[hd]) - top)
            out[i, hd] = (e / den) @ v[: i + 1, hd // (H // G)]
    out = out * torch.sigmoid(h @ W("g").T)[:, :, None]
    return out.reshape(T, H * dv) @ W("o").T


def hgrn2(h, weights, prefix, m, eps):
    """Linear attention whose forget gate also gates the write: S = diag(f) S + (1 - f) v^T, o = S^T q."""
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    W = lambda n: weights[prefix + n]                                       # noqa: E731
    q = silu(h @ W("q").T).reshape(T, H, dk)
    v = (h @ W("v").T).reshape(T, H, dv)
    low = W("lower")
    f = (low + (1.0 - low) * torch.sigmoid(h @ W("f").T + W("f.b"))).reshape(T, H, dk)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = f[t, hd][:, None] * S + (1.0 - f[t, hd])[:, None] * v[t, hd][None, :]
            out[t, hd] = S.T @ q[t, hd]
    out = unit_rms(out, eps) * W("norm")
    return out.reshape(T, H * dv) @ W("o").T


def channel_delta(h, weights, prefix, m, eps):
    """Gated delta rule with a decay per key channel: S = g * S; u = beta (v - S^T k); S += k u^T; o = S^T q."""
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    W = lambda n: weights[prefix + n]                                       # noqa: E731
    q = silu(causal_conv(h @ W("q").T, W("q.conv"))).reshape(T, G, dk)
    k = silu(causal_conv(h @ W("k").T, W("k.conv"))).reshape(T, G, dk)
    v = silu(causal_conv(h @ W("v").T, W("v.conv"))).reshape(T, H, dv)
    q = unit_length(q, 1e-6) * dk ** -0.5
    k = unit_length(k, 1e-6)
    beta = torch.sigmoid(h @ W("b").T)                                       # [T, H]
    rate = torch.exp(W("A_log"))                                             # [H]
    step = softplus((h @ W("a1").T) @ W("a2").T + W("dt_bias")).reshape(T, H, dk)
    g = torch.exp(-rate[None, :, None] * step)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        j = hd // (H // G)
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = g[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, j])
            S = S + k[t, j][:, None] * u[None, :]
            out[t, hd] = S.T @ q[t, j]
    gate = torch.sigmoid((h @ W("g1").T) @ W("g2").T).reshape(T, H, dv)
    out = unit_rms(out, eps) * W("norm") * gate
    return out.reshape(T, H * dv) @ W("o").T


MIXERS = {"attention": attention, "hgrn2": hgrn2, "channel_delta": channel_delta}


# ----------------------------------------------------------------------------- feed-forward
def dense_ff(h, weights, prefix):
    p, q = weights[prefix + "act"][0], weights[prefix + "act"][1]
    return xielu(h @ weights[prefix + "up"].T, p, q) @ weights[prefix + "down"].T


# ----------------------------------------------------------------------------- the model
def run_order(config):
    """The layers in the order they run, with True where a pass over the repeated run begins."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def layer(x, i, weights, config):
    """One parallel layer: both sublayers read the same normed input, and their sum joins the stream."""
    L = config["layers"][i]
    eps = float(config["norm"]["eps"])
    p = f"l{i}."
    h = layer_norm(x, weights[p + "norm1"], weights[p + "norm1.b"], eps)
    y = MIXERS[L["type"]](h, weights, p + "mix.", L["mixer"], eps)
    if L.get("mlp") is not None:
        y = y + dense_ff(h, weights, p + "mlp.")
    return x + y


def forward(tokens, weights, config, layers_out=None):
    """Logits [T, vocab] of a token sequence; ``layers_out`` (a list) receives the stream after every layer run."""
    x0 = weights["embed"][torch.tensor(tokens)].clone()
    x = x0
    for i, begins_pass in run_order(config):
        if begins_pass:
            x = torch.cat([x, x0], dim=1) @ weights["loop.in"].T
        x = layer(x, i, weights, config)
        if layers_out is not None:
            layers_out.append(x.clone())
    eps = float(config["norm"]["eps"])
    x = layer_norm(x, weights["final.norm"], weights["final.norm.b"], eps)
    return (x @ weights["head"].T) * float(config.get("logit_scale", 1.0))
