"""Arrangement of a layer's parts around the residual stream.

Reference ``block`` (src/model.rs:587-599): x += mixer(norm(x)); x += ffn(norm(x)).
The residual stream is float32 in both engines; the norm writes the activation type.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block, Norm
from .registry import register_part
from .spec import TensorNeed


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """params: hidden.  Made of: mixer_norm, mixer, feed_forward_norm, feed_forward (and a position encoding for
    the mixer, if the layer lists one)."""
    chain_safe = True
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, spec, runtime, parts):
        super().__init__(spec, runtime, parts)
        self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
        self.ff_norm, self.feed_forward = parts["feed_forward_norm"], parts["feed_forward"]
        self.hidden = int(spec.params["hidden"])
        runtime.scratch("normed", runtime.max_batch_tokens, self.hidden)

    @property
    def first_reader_takes_owed(self):
        return getattr(self.mixer_norm, "takes_owed", False)

    def forward(self, residual, ctx, call):
        h = self.runtime.get_scratch("normed")[:, : self.hidden]
        self.norm_of_stream(self.mixer_norm, residual, h, ctx)
        ctx.may_owe = getattr(self.ff_norm, "takes_owed", False)
        self.mixer.forward(h, residual, ctx, call.mixers["mixer"])
        ctx.may_owe = False
        self.norm_of_stream(self.ff_norm, residual, h, ctx)
        ctx.may_owe = ctx.next_block_takes_owed
        self.feed_forward.forward(h, residual, ctx)
        ctx.may_owe = False


@register_part("block", "parallel")
class ParallelBlock(Block):
    """One norm whose output both sublayers read: with h = norm(x), x += mixer(h) + feed_forward(h).

    params: hidden.  Made of: norm, mixer, and optionally feed_forward (a position encoding for the mixer, if the layer
    lists one).  Both sublayers add their output into the float32 stream, the mixer first."""
    roles = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}
    optional = ("feed_forward",)

    def __init__(self, spec, runtime, parts):
        super().__init__(spec, runtime, parts)
        self.norm, self.mixer, self.feed_forward = parts["norm"], parts["mixer"], parts.get("feed_forward")
        self.hidden = int(spec.params["hidden"])
        runtime.scratch("normed", runtime.max_batch_tokens, self.hidden)

    @property
    def first_reader_takes_owed(self):
        return getattr(self.norm, "takes_owed", False)

    def forward(self, residual, ctx, call):
        h = self.runtime.get_scratch("normed")[:, : self.hidden]
        self.norm_of_stream(self.norm, residual, h, ctx)
        # neither sublayer may leave a sum owed to the stream: the other one adds into it right after
        ctx.may_owe = False
        self.mixer.forward(h, residual, ctx, call.mixers["mixer"])
        if self.feed_forward is not None:
            self.feed_forward.forward(h, residual, ctx)


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Block):
    """A layer whose sublayers are normed on both sides: x += post(mixer(conv(pre(x)))), x += post'(ff(pre'(x))).

    params: hidden, ignored_tensors (names of scalar tensors a checkpoint may carry for a sublayer the layer lacks).
    Made of: mixer_norm, mixer, mixer_post_norm; optionally input_conv (a convolution over time that
    what the mixer reads passes first; it keeps state like a mixer, hence its category), and feed_forward_norm,
    feed_forward, feed_forward_post_norm (all three or none).  The mixer and the feed-forward store their output in a
    float32 buffer of the block (``ctx.store_output``); the post-norm adds it to the stream and, in the same kernel,
    applies the norm of the stream's next reader inside the layer."""
    roles = {"mixer_norm": "norm", "input_conv": "mixer", "mixer": "mixer", "mixer_post_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    optional = ("input_conv", "feed_forward_norm", "feed_forward", "feed_forward_post_norm")

    def __init__(self, spec, runtime, parts):
        super().__init__(spec, runtime, parts)
        self.hidden = int(spec.params["hidden"])
        ff = [r for r in ("feed_forward_norm", "feed_forward", "feed_forward_post_norm") if r in parts]
        if len(ff) not in (0, 3):
            raise ValueError(f"block 'sandwich_norm' has a feed-forward with both of its norms or none; got {ff}")
        self.has_ff = bool(ff)
        for r in ("mixer_post_norm", "feed_forward_post_norm"):
            if r in parts and type(parts[r]).forward_add is Norm.forward_add:
                raise ValueError(f"block 'sandwich_norm': the {r} part cannot norm a sublayer's output into the stream")
        self.ignored = tuple(spec.params.get("ignored_tensors", ()))
        runtime.scratch("normed", runtime.max_batch_tokens, self.hidden)
        runtime.scratch("conv_out", runtime.max_batch_tokens, self.hidden)
        runtime.scratch("sublayer_out", runtime.max_batch_tokens, self.hidden, torch.float32)

    def tensor_needs(self):
        # gains of norms that a layer without a feed-forward has no use for: taken if the checkpoint has them
        return {name: TensorNeed((), "norm", optional=True) for name in self.ignored}

    def forward(self, residual, ctx, call):
        rt, p, T = self.runtime, self.parts, ctx.n_tokens
        h = rt.get_scratch("normed")[:, : self.hidden]
        delta = rt.get_scratch("sublayer_out", torch.float32)[:, : self.hidden]
        self.norm_of_stream(p["mixer_norm"], residual, h, ctx)
        if "input_conv" in p:
            h2 = rt.get_scratch("conv_out")[:, : self.hidden]
            p["input_conv"].forward(h, h2, ctx, call.mixers["input_conv"])
            h = h2
        ctx.store_output = True
        try:
            p["mixer"].forward(h, delta, ctx, call.mixers["mixer"])
            if not self.has_ff:
                p["mixer_post_norm"].forward_add(delta, residual, T)
                return
            h = rt.get_scratch("normed")[:, : self.hidden]
            p["mixer_post_norm"].forward_add(delta, residual, T, then=p["feed_forward_norm"], out=h)
            p["feed_forward"].forward(h, delta, ctx)
            p["feed_forward_post_norm"].forward_add(delta, residual, T)
        finally:
            ctx.store_output = False


@register_part("block", "stream_reentry")
class StreamReentryBlock(Block):
    """The start of a pass over a run of layers that is repeated with the same weights: the stream is mixed with the
    embedding output again, x <- W [x ; embedding(token)] + step, ``step`` one row of a [passes, hidden] table.

    params: hidden, vocab, n_passes, index (which row of the table).  tensors: in_proj [hidden, 2 * hidden] (x first),
    step [n_passes, hidden] (left out of the tensors: no such term), embedding [vocab, hidden] (the model's token table).
    No parts, no cache, no state."""
    roles = {}

    def __init__(self, spec, runtime, parts):
        super().__init__(spec, runtime, parts)
        p = spec.params
        self.hidden, self.vocab = int(p["hidden"]), int(p["vocab"])
        self.n_passes, self.index = int(p["n_passes"]), int(p["index"])
        if not 0 <= self.index < self.n_passes:
            raise ValueError(f"stream_reentry: pass {self.index} of {self.n_passes}")
        runtime.scratch("stream_cat", runtime.max_batch_tokens, 2 * self.hidden)

    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["in_proj"]: TensorNeed((self.hidden, 2 * self.hidden)),
                 t["embedding"]: TensorNeed((self.vocab, self.hidden), "embedding")}
        if "step" in t:
            needs[t["step"]] = TensorNeed((self.n_passes, self.hidden))
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        self.w_in = tensors[t["in_proj"]].contiguous()
        self.step_row = tensors[t["step"]][self.index].contiguous() if "step" in t else None
        self.table = tensors[t["embedding"]]

    def flops_per_token(self) -> float:
        return 4.0 * self.hidden * self.hidden

    def forward(self, residual, ctx, call):
        T = ctx.n_tokens
        if ctx.owed is not None:
            ctx.owed.finish()
            ctx.owed = None
        cat = self.runtime.get_scratch("stream_cat")[:, : 2 * self.hidden]
        # cat = [x | embedding]; the stream is preset to the pass's row, and the product adds W cat onto it
        ops.concat_embed(residual, self.table, ctx.token_ids, self.step_row, cat, T, ctx.status)
        ops.linear(cat, self.w_in, residual, T, accumulate=True, status=ctx.status)
