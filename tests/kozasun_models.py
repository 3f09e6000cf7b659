"""Small Kozasun configurations with weights made here, for the tests.

The tensor names and shapes are derived here from the configuration (not from the engine's manifest, which is thereby
checked too), the values are drawn with numpy and rounded to bfloat16.  ``sharp`` (a strength, 1 or True for the
full one) makes faults visible that random weights would hide: the attention's and the latent attention's queries are scaled up so that each query looks at one
or two keys only, wherever they lie in what it may see, their output weighs more, and the sinks are raised so that
leaving them out changes every output.  ``steady_router`` spaces the router's corrections so far apart that the choice
of experts does not hang on the last bits of a score (the bfloat16 engine rounds the router's input; the weights of
the chosen experts still come from the live scores): powers of two, so that no two experts and no two groups of
experts are worth the same.
"""
from __future__ import annotations

import copy

import numpy as np
import torch

from lokinex_models import write_model  # noqa: F401  (the safetensors writer of the test suite)


def attention(heads, kv_heads, dim, vdim, rot=None, chunk=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if chunk:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m}


def retention(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "retention", "mixer": m}


def latent(heads, dim, vdim, kv_rank, window=None, scale=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": dim ** -0.5 if scale is None else scale}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale=None, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if scale is not None:
        r["scale"] = scale
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def same_as(j):
    return j


def config(vocab, width, layers, eps=1e-6, streams=None, embedding_scale=None):
    """``layers``: (layer, mlp) pairs, or an int j for a layer that uses layer j's tensors."""
    out = []
    for entry in layers:
        if isinstance(entry, int):
            out.append(dict(copy.deepcopy(out[entry]), weights_of=entry))
        else:
            out.append(dict(copy.deepcopy(entry[0]), mlp=copy.deepcopy(entry[1])))
    c = {"architecture": "Kozasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": out}
    if streams is not None:
        c["streams"] = streams
    if embedding_scale is not None:
        c["embedding"] = {"scale": embedding_scale}
    return c


# Sizes that differ from each other in every respect; values that a model may happen to make equal or 1 (kv heads
# against heads, vdim against dim, rot.dims against dim, streams, top, groups kept, scales) are unequal or not 1
# somewhere and equal or 1 elsewhere.
CONFIGS = {
    # three streams, a shared layer in the middle of the order and one at its end, a layer without feed-forward,
    # rows that need padding, a chunk and a window that are no multiple of a page or of a key tile
    "P": config(211, 96, [
        (attention(6, 2, 24, 40, rot=(8, 5000.0), chunk=20, scale=0.3), dense(160)),
        (retention(3, 24, 20, (0.9, 0.97, 0.995), rot=(24, 300.0)), moe(6, 2, 40, scale=1.5, groups=(3, 2), shared=56)),
        (latent(3, 16, 24, 40, window=33, scale=0.25), None),
        0,
        (retention(2, 40, 12, (0.99, 0.5)), moe(5, 1, 24)),
        2,
    ], eps=1e-6, streams=3, embedding_scale=0.25),
    # no streams (the plain residual sum), no embedding scale, no masks, no rotation in the attention, one kv head,
    # one group kept of two, a width the tensor-core products refuse
    "Q": config(130, 100, [
        (attention(5, 1, 32, 8), moe(10, 3, 24, scale=1.75, groups=(2, 1), shared=40)),
        (latent(2, 24, 8, 20), dense(56)),
        (retention(1, 64, 32, (0.98,), rot=(16, 1e4)), None),
    ], eps=1e-5),
    # wider, two streams, heads of the sizes the tensor-core kernels take, for long sequences
    "R": config(320, 256, [
        (attention(4, 2, 64, 64, rot=(32, 1e5), chunk=128), dense(320)),
        (retention(4, 64, 32, (0.97, 0.99, 0.995, 0.999), rot=(32, 5e5)), moe(12, 2, 64, scale=2.5, groups=(4, 2), shared=128)),
        (latent(4, 48, 32, 80, window=200), dense(256)),
        1,
    ], eps=1e-5, streams=2, embedding_scale=2.0),
    # one stream with hyper-connection tensors of size one
    "S": config(97, 64, [
        (latent(2, 16, 16, 24, window=7), dense(72)),
        (attention(2, 2, 16, 16, rot=(16, 100.0), chunk=5), None),
    ], streams=1),
}


def ff_shapes(s, p, mlp, D):
    if mlp is None:
        return
    if mlp["kind"] == "dense":
        s.update({p + "gate": (mlp["ff"], D), p + "up": (mlp["ff"], D), p + "down": (D, mlp["ff"])})
        return
    E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
    s.update({p + "router": (E, D), p + "correction": (E,)})
    for e in range(E):
        s.update({f"{p}e{e}.gate": (ff, D), f"{p}e{e}.up": (ff, D), f"{p}e{e}.down": (D, ff)})
    if mlp.get("shared"):
        sf = mlp["shared"]["ff"]
        s.update({p + "shared.gate": (sf, D), p + "shared.up": (sf, D), p + "shared.down": (D, sf)})


def tensor_shapes(cfg):
    D, V, S = cfg["width"], cfg["vocab"], cfg.get("streams")
    s = {"embed": (V, D), "head": (V, D), "final.norm": (D,), "final.norm.b": (D,)}
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        p = f"l{i}."
        m = L["mixer"]
        s[p + "norm1"] = s[p + "norm1.b"] = (D,)
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            G = m["kv_heads"]
            s.update({p + "mix.q": (H * dk, D), p + "mix.q.b": (H * dk,), p + "mix.k": (G * dk, D), p + "mix.k.b": (G * dk,),
                      p + "mix.v": (G * dv, D), p + "mix.v.b": (G * dv,), p + "mix.q.norm": (H * dk,),
                      p + "mix.k.norm": (G * dk,), p + "mix.sink": (H,), p + "mix.o": (D, H * dv)})
        elif L["type"] == "retention":
            s.update({p + "mix.q": (H * dk, D), p + "mix.k": (H * dk, D), p + "mix.v": (H * dv, D), p + "mix.g": (H * dv, D),
                      p + "mix.o": (D, H * dv)})
        else:
            R = m["kv_rank"]
            s.update({p + "mix.q": (H * dk, D), p + "mix.dkv": (R, D), p + "mix.dkv.norm": (R,), p + "mix.uk": (H * dk, R),
                      p + "mix.uv": (H * dv, R), p + "mix.g": (H, D), p + "mix.o": (D, H * dv)})
        if S is not None:
            s.update({p + "hc1.in": (S,), p + "hc1.out": (S,), p + "hc1.mix": (S, S)})
        if L["mlp"] is not None:
            s[p + "norm2"] = s[p + "norm2.b"] = (D,)
            ff_shapes(s, p + "mlp.", L["mlp"], D)
            if S is not None:
                s.update({p + "hc2.in": (S,), p + "hc2.out": (S,), p + "hc2.mix": (S, S)})
    return s


def draw_weights(cfg, seed, sharp=False, steady_router=False):
    """name → float64 tensor holding bfloat16-representable values."""
    rng = np.random.default_rng(seed)
    sharp = float(sharp)
    kinds = {f"l{i}.": L["type"] for i, L in enumerate(cfg["layers"])}
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        layer = name[: name.index(".") + 1] if name.startswith("l") and name[1].isdigit() else ""
        rest = name[len(layer):]
        kind = kinds.get(layer)
        if rest in ("norm1", "norm2", "final.norm", "mix.q.norm", "mix.k.norm", "mix.dkv.norm"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
            if sharp and rest == "mix.q.norm":
                v = v * (1.0 + 5.0 * sharp)       # peaked attention: the queries are normed, so the norm's weight scales them
        elif rest.endswith(".b"):
            v = 0.3 * rng.standard_normal(shape)
        elif rest == "mix.sink":
            v = 2.0 * min(sharp, 1.0) + rng.standard_normal(shape)
        elif rest in ("hc1.in", "hc2.in"):
            v = 1.0 / shape[0] + 0.2 * rng.standard_normal(shape)
        elif rest in ("hc1.out", "hc2.out"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif rest in ("hc1.mix", "hc2.mix"):
            v = np.eye(shape[0]) + 0.2 * rng.standard_normal(shape)
        elif rest == "mlp.correction":
            v = 4.0 * 2.0 ** rng.permutation(shape[0]) if steady_router else 0.15 * rng.standard_normal(shape)
        elif rest == "mlp.router":
            v = 2.0 * rng.standard_normal(shape) / np.sqrt(shape[-1])
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            v = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if sharp and kind == "latent_attention" and rest == "mix.q":
                v = v * (1.0 + 7.0 * sharp)       # peaked latent attention
            if sharp and kind in ("attention", "latent_attention") and rest == "mix.o":
                v = v * (1.0 + 2.0 * sharp)       # what the attention reads far back weighs on the logits
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16).to(torch.float64)
    return out


def make(path, name_or_cfg, seed=0, sharp=False, steady_router=False):
    cfg = CONFIGS[name_or_cfg] if isinstance(name_or_cfg, str) else name_or_cfg
    w = draw_weights(cfg, seed, sharp, steady_router)
    write_model(path, cfg, w)
    return cfg, w


def with_mask_sizes(cfg, delta):
    """The configuration with every mask's size changed by ``delta``: what a window or a block that is one off computes."""
    c = copy.deepcopy(cfg)
    for L in c["layers"]:
        if L["mixer"].get("mask"):
            L["mixer"]["mask"]["size"] += delta
    return c
