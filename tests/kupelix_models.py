"""Small Kupelix configurations with weights made here, for the tests.

The tensor names and shapes are derived here from the configuration (not from the engine's manifest, which is thereby
checked too), the values are drawn with numpy and rounded to bfloat16.  ``sharp=True`` makes faults visible that random
weights would hide: the attention's queries are scaled up so that each query looks at one or two keys only, wherever
they lie, and its output weighs four times as much, the sinks are raised so that leaving them out changes every output, the forget gates' lower bounds sit just
below one and the delta rule's decays just below one, so that both states last for hundreds of tokens.
"""
from __future__ import annotations

import numpy as np
import torch

from lokinex_models import write_model  # noqa: F401  (the safetensors writer of the test suite)


def attention(heads, kv_heads, dim, vdim, rot_dims=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention", "mixer": m}


def hgrn2(heads, dim, vdim):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank=12, gate_rank=20):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(vocab, width, layers, eps=1e-6, loop=None, logit_scale=None):
    c = {"architecture": "Kupelix", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": [dict(l, mlp=m) for l, m in layers]}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    return c


# Sizes that differ from each other in every respect; values that a model may happen to make equal or 1 (kv heads
# against heads, vdim against dim, rot.dims against dim, taps, times, logit_scale) are unequal or not 1 somewhere and
# equal or 1 elsewhere.
CONFIGS = {
    # a loop in the middle (start > 0, stop < layers), three passes, a layer without feed-forward, rows that need padding
    "P": config(211, 96, [
        (hgrn2(3, 24, 20), dense(160)),
        (attention(6, 2, 24, 40, rot_dims=8, base=5000.0, scaling=(8.0, 1.0, 4.0, 64)), dense(72)),
        (delta(4, 2, 16, 24, 3), None),
        (attention(4, 4, 16, 16, rot_dims=16, base=300.0), dense(48)),
        (delta(2, 2, 40, 12, 2, decay_rank=7, gate_rank=9), dense(64)),
    ], eps=1e-6, loop=(1, 4, 3), logit_scale=0.25),
    # no loop, no rotation in one layer, one kv head, one tap, a width the tensor-core products refuse, logit scale absent
    "Q": config(130, 100, [
        (attention(5, 1, 32, 8), dense(56)),
        (delta(3, 1, 8, 36, 1, decay_rank=4, gate_rank=4), dense(40)),
        (hgrn2(1, 64, 32), None),
    ], eps=1e-5),
    # wider, one pass of a loop over everything, for long sequences
    "R": config(320, 256, [
        (attention(4, 2, 48, 32, rot_dims=24, base=1e5, scaling=(4.0, 1.0, 2.0, 128)), dense(384)),
        (delta(4, 2, 32, 64, 4, decay_rank=16, gate_rank=32), dense(256)),
        (hgrn2(4, 32, 48), dense(320)),
    ], eps=1e-5, loop=(0, 3, 1), logit_scale=1.5),
}


def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "head": (V, D), "final.norm": (D,), "final.norm.b": (D,)}
    if cfg.get("loop") is not None:
        s["loop.in"] = (D, 2 * D)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        s[p + "norm1"] = s[p + "norm1.b"] = (D,)
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            G = m["kv_heads"]
            s.update({p + "mix.q": (H * dk, D), p + "mix.q.b": (H * dk,), p + "mix.k": (G * dk, D), p + "mix.k.b": (G * dk,),
                      p + "mix.v": (G * dv, D), p + "mix.v.b": (G * dv,), p + "mix.q.norm": (dk,), p + "mix.k.norm": (dk,),
                      p + "mix.talk": (H, H), p + "mix.sink": (H,), p + "mix.g": (H, D), p + "mix.o": (D, H * dv)})
        elif L["type"] == "hgrn2":
            s.update({p + "mix.q": (H * dk, D), p + "mix.f": (H * dk, D), p + "mix.f.b": (H * dk,), p + "mix.lower": (H * dk,),
                      p + "mix.v": (H * dv, D), p + "mix.norm": (dv,), p + "mix.o": (D, H * dv)})
        else:
            G, taps, ra, rg = m["kv_heads"], m["conv"], m["decay_rank"], m["gate_rank"]
            s.update({p + "mix.q": (G * dk, D), p + "mix.q.conv": (G * dk, taps), p + "mix.k": (G * dk, D),
                      p + "mix.k.conv": (G * dk, taps), p + "mix.v": (H * dv, D), p + "mix.v.conv": (H * dv, taps),
                      p + "mix.b": (H, D), p + "mix.A_log": (H,), p + "mix.norm": (dv,), p + "mix.a1": (ra, D),
                      p + "mix.a2": (H * dk, ra), p + "mix.dt_bias": (H * dk,), p + "mix.g1": (rg, D),
                      p + "mix.g2": (H * dv, rg), p + "mix.o": (D, H * dv)})
        if L["mlp"] is not None:
            ff = L["mlp"]["ff"]
            s.update({p + "mlp.up": (ff, D), p + "mlp.down": (D, ff), p + "mlp.act": (2,)})
    return s


def draw_weights(cfg, seed, sharp=False):
    """name → float64 tensor holding bfloat16-representable values."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        layer = name[: name.index(".") + 1] if name.startswith("l") and name[1].isdigit() else ""
        rest = name[len(layer):]
        if rest in ("norm1", "final.norm", "mix.q.norm", "mix.k.norm", "mix.norm"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
            if sharp and rest == "mix.q.norm":
                v = v * 6.0                       # peaked attention: a query looks at one or two keys, wherever they lie
                                                  # (the queries are normed, so it is the norm's weight that scales them)
        elif rest in ("norm1.b", "final.norm.b", "mix.q.b", "mix.k.b", "mix.v.b", "mix.f.b"):
            v = 0.3 * rng.standard_normal(shape)
        elif rest == "mix.talk":
            v = np.eye(shape[0]) + 0.3 * rng.standard_normal(shape)
        elif rest == "mix.sink":
            v = (2.0 if sharp else 0.0) + rng.standard_normal(shape)
        elif rest == "mix.lower":
            v = rng.uniform(0.97, 0.999, shape) if sharp else rng.uniform(0.0, 0.9, shape)
        elif rest == "mix.A_log":
            v = (-4.0 if sharp else 0.0) + 0.5 * rng.standard_normal(shape)
        elif rest == "mix.dt_bias":
            v = (-3.0 if sharp else 0.0) + rng.standard_normal(shape)
        elif rest.endswith(".conv"):
            v = 0.5 * rng.standard_normal(shape)
        elif rest == "mlp.act":
            v = rng.standard_normal(shape)
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            v = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if sharp and rest == "mix.o" and (name[: -len("o")] + "talk") in tensor_shapes(cfg):
                v = v * 4.0                       # what the attention reads far back weighs on the logits
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16).to(torch.float64)
    return out


def make(path, name_or_cfg, seed=0, sharp=False):
    cfg = CONFIGS[name_or_cfg] if isinstance(name_or_cfg, str) else name_or_cfg
    w = draw_weights(cfg, seed, sharp)
    on_disk = {k: v for k, v in cfg.items()}
    # the inner widths of the low-rank maps are read from the tensors' shapes, as for a checkpoint from elsewhere
    on_disk["layers"] = [dict(L, mixer={k: v for k, v in L["mixer"].items() if k not in ("decay_rank", "gate_rank")})
                         for L in cfg["layers"]]
    write_model(path, on_disk, w)
    return cfg, w
