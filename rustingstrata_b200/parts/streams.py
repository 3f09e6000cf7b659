"""Several residual streams per token (hyper-connections), the layer norm their readers use, and an embedding that is
a sum of tables.

Streams: a model with S streams keeps x_1 .. x_S per token, all equal to the embedding output at the start.  A
sublayer reads u = sum_s in[s] x_s through its norm, and its output y rewrites all streams at once from the old ones,

    x_t <- sum_s mix[s, t] x_s + out[t] y            (mix indexed [from, to]),

and at the end the model's final norm reads the plain sum of the streams.  One stream with in = out = mix = 1 is the
ordinary residual sum, which is what a layer without the three tensors gets.  The stream buffer is float32
[tokens, S * hidden]; sums, means and variances are float32 in both engines.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block, Norm, Part
from .registry import register_part
from .spec import StateNeed, TensorNeed


@register_part("embedding", "table_sum")
class TableSumEmbedding(Part):
    """Token row + bigram row + learned position row, written to every residual stream.

    params: vocab, width, copies (residual streams to fill, default 1), scale (default 1: multiplies the token row);
    bigram: None or {buckets, mul_prev, mul_cur}: row
    (previous token * mul_prev + token * mul_cur) mod buckets of a [buckets + 1, width] table whose last row serves a
    sequence's first token; positions: rows of a learned [positions, width] table added unscaled, or 0 for none.
    tensors: weight, and bigram / position when the params have them.  Per request it keeps one int32: the last token
    of the request's previous step."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.vocab, self.width = int(p["vocab"]), int(p["width"])
        self.copies = int(p.get("copies", 1))
        self.scale = float(p.get("scale", 1.0))
        big = p.get("bigram")
        self.bigram_params = None if big is None else (int(big["buckets"]), int(big["mul_prev"]), int(big["mul_cur"]))
        if self.bigram_params is not None and self.bigram_params[0] < 1:
            raise ValueError(f"table_sum: a bigram table needs at least one bucket, got {self.bigram_params[0]}")
        self.n_positions = int(p.get("positions") or 0)
        self.weight = self.bigram = self.position = self.state = None

    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["weight"]: TensorNeed((self.vocab, self.width), "embedding")}
        if self.bigram_params is not None:
            needs[t["bigram"]] = TensorNeed((self.bigram_params[0] + 1, self.width), "embedding")
        if self.n_positions:
            needs[t["position"]] = TensorNeed((self.n_positions, self.width), "embedding")
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        self.weight = tensors[t["weight"]].contiguous()
        if self.bigram_params is not None:
            self.bigram = tensors[t["bigram"]].contiguous()
        if self.n_positions:
            self.position = tensors[t["position"]].contiguous()

    def state_need(self):
        return StateNeed(1, "int32") if self.bigram_params is not None else None

    def forward(self, ctx, residual):
        big = self.bigram_params
        ops.embed_sum(self.weight, ctx.token_ids, residual, ctx.n_tokens, ctx.n_seqs, self.copies, ctx.positions,
                      ctx.seq_of_token, ctx.q_start, ctx.state_slots, ctx.status, bigram=self.bigram,
                      mul_prev=big[1] if big else 0, mul_cur=big[2] if big else 0, prev_state=self.state,
                      position_table=self.position, scale=self.scale)


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * weight + bias, var the mean squared deviation.

    params: width, eps, streams (default 1: x is one row of ``width``; more: x holds that many rows side by side and
    the norm reads their sum), bias (default True).  tensors: weight, bias."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.streams = int(spec.params.get("streams", 1))
        self.has_bias = bool(spec.params.get("bias", True))
        self.weight = self.bias = None

    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["weight"]: TensorNeed((self.width,), "norm")}
        if self.has_bias:
            needs[t["bias"]] = TensorNeed((self.width,))
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        self.weight = tensors[t["weight"]].contiguous()
        self.bias = tensors[t["bias"]].contiguous() if self.has_bias else None

    def forward(self, x, out, n_rows, rows=None):
        ops.stream_layernorm(x, self.streams, None, self.weight, self.bias, self.eps, out, n_rows, rows=rows)


@register_part("block", "hyper_connection")
class HyperConnectionBlock(Block):
    """A pre-norm layer over S residual streams: each sublayer reads a weighted sum of the streams through its norm and
    its output rewrites all streams (see the module's text).

    params: hidden, streams.  Made of: mixer_norm, mixer, and optionally feed_forward_norm with feed_forward (both or
    neither); the norms are of kind ``layernorm``.  tensors (all or none per sublayer; none: the plain residual sum of
    one stream): mixer_in [S], mixer_out [S], mixer_mix [S, S], ff_in, ff_out, ff_mix.  The sublayers store their
    output in a float32 buffer of the block; the kernel that rewrites the streams also runs the norm of the stream's
    next reader: the feed-forward's, or the next layer's first norm when that layer is of this kind and shape."""
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    optional = ("feed_forward_norm", "feed_forward")

    def __init__(self, spec, runtime, parts):
        super().__init__(spec, runtime, parts)
        self.hidden = int(spec.params["hidden"])
        self.S = int(spec.params.get("streams", 1))
        if not 1 <= self.S <= ops.MAX_STREAMS:
            raise ValueError(f"hyper_connection: {self.S} streams (1 to {ops.MAX_STREAMS} are supported)")
        if self.hidden > ops.MAX_STREAM_WIDTH:
            raise ValueError(f"hyper_connection: width {self.hidden} exceeds the {ops.MAX_STREAM_WIDTH} the stream kernels hold")
        ff = [r for r in ("feed_forward_norm", "feed_forward") if r in parts]
        if len(ff) == 1:
            raise ValueError("block 'hyper_connection' has a feed-forward with its norm or neither")
        self.has_ff = bool(ff)
        for r in ("mixer_norm", "feed_forward_norm"):
            if r in parts and not isinstance(parts[r], LayerNorm):
                raise ValueError(f"block 'hyper_connection': the {r} part must be of kind 'layernorm'")
            if r in parts and (parts[r].streams != 1 or parts[r].width != self.hidden):
                raise ValueError(f"block 'hyper_connection': the {r} part norms one row of {self.hidden} values")
        t = spec.tensors
        self.named = {q: all(f"{q}_{k}" in t for k in ("in", "out", "mix")) for q in ("mixer", "ff")}
        for q, full in self.named.items():
            if q == "ff" and not self.has_ff:
                continue
            if not full and (any(f"{q}_{k}" in t for k in ("in", "out", "mix")) or self.S != 1):
                raise ValueError(f"block 'hyper_connection': {self.S} streams need the {q} sublayer's in, out and mix tensors")
        self.coef = {}
        runtime.scratch("normed", runtime.max_batch_tokens, self.hidden)
        runtime.scratch("sublayer_out", runtime.max_batch_tokens, self.hidden, torch.float32)

    def tensor_needs(self):
        t, S = self.spec.tensors, self.S
        needs = {}
        for q in ("mixer", "ff"):
            if self.named[q] and (q == "mixer" or self.has_ff):
                needs[t[f"{q}_in"]] = TensorNeed((S,), "average")
                needs[t[f"{q}_out"]] = TensorNeed((S,), "norm")
                needs[t[f"{q}_mix"]] = TensorNeed((S, S), "average")
        return needs

    def load(self, tensors):
        t, S = self.spec.tensors, self.S
        for q in ("mixer", "ff"):
            if q == "ff" and not self.has_ff:
                continue
            if self.named[q]:
                self.coef[q] = tuple(tensors[t[f"{q}_{k}"]].to(torch.float32).contiguous() for k in ("in", "out", "mix"))
            else:
                one = torch.ones(1, dtype=torch.float32, device=self.runtime.device)
                self.coef[q] = (one, one, one.view(1, 1))

    def stream_reader(self):
        """What the block before this one needs to run this block's first norm: (streams, width, in, weight, bias, eps)."""
        n = self.parts["mixer_norm"]
        return (self.S, self.hidden, self.coef["mixer"][0], n.weight, n.bias, n.eps)

    def forward(self, residual, ctx, call):
        rt, p, T, S = self.runtime, self.parts, ctx.n_tokens, self.S
        if ctx.owed is not None:
            ctx.owed.finish()
            ctx.owed = None
        h = rt.get_scratch("normed")[:, : self.hidden]
        delta = rt.get_scratch("sublayer_out", torch.float32)[:, : self.hidden]
        m_in, m_out, m_mix = self.coef["mixer"]
        n1 = p["mixer_norm"]
        if ctx.normed_ready:
            ctx.normed_ready = False             # the block before this one left norm(sum in[s] x_s) in h
        else:
            ops.stream_layernorm(residual, S, m_in, n1.weight, n1.bias, n1.eps, h, T)
        nxt = ctx.next_reader
        fuse_next = nxt is not None and nxt[0] == S and nxt[1] == self.hidden
        tail = dict(next_coef=nxt[2], next_weight=nxt[3], next_bias=nxt[4], next_eps=nxt[5], next_out=h) if fuse_next else {}
        ctx.store_output = True
        try:
            p["mixer"].forward(h, delta, ctx, call.mixers["mixer"])
            if not self.has_ff:
                ops.stream_update(residual, S, delta, m_mix, m_out, T, **tail)
            else:
                f_in, f_out, f_mix = self.coef["ff"]
                n2 = p["feed_forward_norm"]
                ops.stream_update(residual, S, delta, m_mix, m_out, T, next_coef=f_in, next_weight=n2.weight,
                                  next_bias=n2.bias, next_eps=n2.eps, next_out=h)
                p["feed_forward"].forward(h, delta, ctx)
                ops.stream_update(residual, S, delta, f_mix, f_out, T, **tail)
            ctx.normed_ready = fuse_next
        finally:
            ctx.store_output = False
