"""Feed-forwards beyond the gated one: a plain two-matrix layer with a squared ReLU, and a mixture of experts whose
choice is a table from token id to expert ids (no router to evaluate), with an optional shared expert.

``table_moe``: every token uses the ``top`` experts its id names, each with weight 1 / top; an expert is
down(SiLU(gate h) * (up h)) without biases.  A shared expert of the same form runs for every token and is added,
multiplied by sigmoid(w_sg . h), one number per token.  The step's (token, k) pairs are sorted by expert on the device
(nothing is read back, so a step can be captured), one grouped product per projection serves all experts, and a last
kernel adds a token's pairs in ascending k together with the gated shared expert.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, StepContext
from .registry import register_part
from .spec import TensorNeed

# rows of one expert that a CTA of the grouped product takes, in its row-streaming (True) and its tiled form; the
# launcher checks them against the compiled kernels
_ROWS_PER_TILE = {True: ops.GROUPED_ROWS_SMALL, False: ops.GROUPED_ROWS_TILED}


@register_part("feed_forward", "relu2_mlp")
class SquaredReluMLP(FeedForward):
    """down(relu(up h)^2), no biases.  params: hidden, intermediate.  tensors: up_proj, down_proj."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec.params["hidden"])
        self.inter = int(spec.params["intermediate"])
        runtime.scratch("ff_act", runtime.max_batch_tokens, self.inter)

    def tensor_needs(self):
        t = self.spec.tensors
        return {t["up_proj"]: TensorNeed((self.inter, self.hidden)), t["down_proj"]: TensorNeed((self.hidden, self.inter))}

    def load(self, tensors):
        t = self.spec.tensors
        self.w_up = tensors[t["up_proj"]].contiguous()
        self.w_down = tensors[t["down_proj"]].contiguous()

    def forward(self, h, residual, ctx: StepContext):
        T = ctx.n_tokens
        act = self.runtime.get_scratch("ff_act")[:, : self.inter]
        ops.linear(h, self.w_up, act, T, status=ctx.status)
        ops.relu_squared(act, act, T)
        ops.linear(act, self.w_down, residual, T, accumulate=not ctx.store_output, status=ctx.status)


@register_part("feed_forward", "table_moe")
class TableMoE(FeedForward):
    """params: hidden, vocab, experts, top, expert_ff, shared_ff (0 or None: no shared expert).
    tensors: table [vocab, top]; expert_gate / expert_up / expert_down: name patterns with ``{e}`` for the expert's
    number; shared_gate, shared_up, shared_down, shared_scale [1, hidden] when there is a shared expert."""
    SMALL_PAIRS_PER_EXPERT = 4      # up to this many (token, k) pairs per expert on average the row-streaming form runs
    LARGE_PAIRS_PER_EXPERT = 96     # from this many on average the tensor-core product takes its 128 x 128 tiles

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.vocab = int(p["hidden"]), int(p["vocab"])
        self.n_experts, self.top = int(p["experts"]), int(p["top"])
        self.ff = int(p["expert_ff"])
        self.shared_ff = int(p.get("shared_ff") or 0)
        if not 1 <= self.top <= self.n_experts:
            raise ValueError(f"table_moe: top {self.top} of {self.n_experts} experts")
        rt = runtime
        pairs = rt.max_batch_tokens * self.top
        # the row pitch is the row's own width, so that the rows stay 16-byte aligned whatever other layers ask for
        self.act_name = f"moe_act_{self.ff}"
        rt.scratch(self.act_name, pairs, self.ff)
        rt.scratch("moe_pair_out", pairs, self.hidden, torch.float32)
        rt.scratch("moe_order", 1, pairs, torch.int32)
        rt.scratch("moe_tiles", 1, 3 * self._max_tiles(pairs, min(_ROWS_PER_TILE.values())) + 4, torch.int32)
        rt.scratch("moe_delta", rt.max_batch_tokens, self.hidden, torch.float32)
        if self.shared_ff:
            rt.scratch("moe_shared_act", rt.max_batch_tokens, self.shared_ff)
            rt.scratch("moe_shared_gu", rt.max_batch_tokens, 2 * self.shared_ff)
            rt.scratch("moe_shared_out", rt.max_batch_tokens, self.hidden, torch.float32)

    def _max_tiles(self, pairs: int, rows: int) -> int:
        """Row tiles of ``rows`` the grouped product can meet: full tiles, plus at most one partly filled per expert in use."""
        return pairs // rows + min(self.n_experts, pairs)

    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["table"]: TensorNeed((self.vocab, self.top), "choice_table", limit=self.n_experts)}
        for e in range(self.n_experts):
            needs[t["expert_gate"].format(e=e)] = TensorNeed((self.ff, self.hidden))
            needs[t["expert_up"].format(e=e)] = TensorNeed((self.ff, self.hidden))
            needs[t["expert_down"].format(e=e)] = TensorNeed((self.hidden, self.ff))
        if self.shared_ff:
            needs[t["shared_gate"]] = TensorNeed((self.shared_ff, self.hidden))
            needs[t["shared_up"]] = TensorNeed((self.shared_ff, self.hidden))
            needs[t["shared_down"]] = TensorNeed((self.hidden, self.shared_ff))
            needs[t["shared_scale"]] = TensorNeed((1, self.hidden))
        return needs

    def load(self, tensors):
        t, E = self.spec.tensors, self.n_experts
        self.table = tensors[t["table"]].contiguous()
        # all experts in one tensor each: [E, gate rows then up rows, hidden] and [E, hidden, ff]
        g0 = tensors[t["expert_gate"].format(e=0)]
        # bfloat16 engine with 16-byte aligned rows: gate and up rows alternate, so that the tensor-core grouped product
        # finds a gate and its up in neighbouring accumulator columns; else gate rows first, up rows behind them
        self.interleaved = (g0.dtype == torch.bfloat16 and self.runtime.dtype == torch.bfloat16 and self.hidden % 8 == 0
                            and self.ff % 8 == 0)
        join = (lambda g, u: torch.stack([g, u], dim=1).reshape(2 * self.ff, self.hidden)) if self.interleaved else \
            (lambda g, u: torch.cat([g, u], dim=0))
        self.w_gate_up = torch.stack([join(tensors[t["expert_gate"].format(e=e)], tensors[t["expert_up"].format(e=e)])
                                      for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[t["expert_down"].format(e=e)] for e in range(E)]).contiguous()
        if self.shared_ff:
            g, u = tensors[t["shared_gate"]], tensors[t["shared_up"]]
            self.shared_fused = (g.dtype == torch.bfloat16 and self.runtime.dtype == torch.bfloat16 and self.hidden % 8 == 0)
            if self.shared_fused:      # gate and up rows alternate: the product's epilogue applies SiLU(gate) * up
                self.w_shared_gu = torch.stack([g, u], dim=1).reshape(2 * self.shared_ff, self.hidden).contiguous()
            else:
                self.w_shared_gu = torch.cat([g, u], dim=0).contiguous()
            self.w_shared_down = tensors[t["shared_down"]].contiguous()
            self.w_shared_scale = tensors[t["shared_scale"]].reshape(-1).contiguous()

    def flops_per_token(self) -> float:
        """Multiply-add flops of one token: its ``top`` experts and the shared one."""
        return 2.0 * (3 * self.top * self.ff * self.hidden + 3 * self.shared_ff * self.hidden + (self.hidden if self.shared_ff else 0))

    def forward(self, h, residual, ctx: StepContext):
        rt, T, top = self.runtime, ctx.n_tokens, self.top
        pairs = T * top
        # bfloat16 engine: one tensor-core launch per projection for all experts, whatever the step's size
        tensor_cores = self.interleaved
        small = not tensor_cores and pairs <= self.SMALL_PAIRS_PER_EXPERT * self.n_experts
        large = tensor_cores and pairs >= self.LARGE_PAIRS_PER_EXPERT * self.n_experts
        rows = ops.GROUPED_ROWS_LARGE if large else _ROWS_PER_TILE[small]
        max_tiles = self._max_tiles(pairs, rows)
        order = rt.get_scratch("moe_order", torch.int32).view(-1)
        tiles = rt.get_scratch("moe_tiles", torch.int32).view(-1)
        n_tiles, tiles = tiles[:1], tiles[4:]
        act = rt.get_scratch(self.act_name)[:, : self.ff]
        pair_out = rt.get_scratch("moe_pair_out", torch.float32)[:, : self.hidden]
        ops.moe_route(ctx.token_ids, self.table, self.n_experts, T, rows, order, tiles, n_tiles, ctx.status)
        if tensor_cores:
            ops.grouped_gemm_mma(h, top, self.w_gate_up, act, order, tiles, n_tiles, max_tiles, gated=True, large=large)
            ops.grouped_gemm_mma(act, 1, self.w_down, pair_out, order, tiles, n_tiles, max_tiles, gated=False, large=large)
        else:
            ops.grouped_linear(h, top, self.w_gate_up, act, order, tiles, n_tiles, max_tiles, gated=True, small=small)
            ops.grouped_linear(act, 1, self.w_down, pair_out, order, tiles, n_tiles, max_tiles, gated=False, small=small)
        shared_out = None
        if self.shared_ff:
            sact = rt.get_scratch("moe_shared_act")[:, : self.shared_ff]
            shared_out = rt.get_scratch("moe_shared_out", torch.float32)[:, : self.hidden]
            if self.shared_fused:
                ops.linear_swiglu(h, self.w_shared_gu, sact, T, status=ctx.status)
            else:
                gu = rt.get_scratch("moe_shared_gu")[:, : 2 * self.shared_ff]
                ops.linear(h, self.w_shared_gu, gu, T)
                ops.silu_mul(gu, sact, T)
            ops.linear(sact, self.w_shared_down, shared_out, T, status=ctx.status)
        if ctx.store_output:
            ops.moe_combine(pair_out, top, 1.0 / top, residual, T, shared=shared_out, h=h,
                            gate_weight=self.w_shared_scale if self.shared_ff else None)
        else:
            delta = rt.get_scratch("moe_delta", torch.float32)[:, : self.hidden]
            ops.moe_combine(pair_out, top, 1.0 / top, delta, T, shared=shared_out, h=h,
                            gate_weight=self.w_shared_scale if self.shared_ff else None)
            ops.residual_add(residual, delta, T)




@register_part("feed_forward", "routed_moe")
class RoutedMoE(FeedForward):
    """A mixture of experts chosen per token by a router, with an optional shared expert.

    Router logits z = W_r h are float32 in both engines; the scores s are softmax(z) over all experts (``score``
    "softmax") or sigmoid(z), each expert for itself ("sigmoid").  The ``top`` experts with the largest s + correction are
    chosen (``correction``: one learned number per expert that steers the choice only).  With ``groups`` the experts form
    that many equal groups of neighbours; a group is worth the sum of its two largest s + correction, and only experts
    of the ``keep`` groups worth most can be chosen.  The weights are the chosen experts' scores s times ``route_scale``,
    divided by the sum of the chosen scores (+ 1e-20) first if ``renormalize``.  An expert (``expert``) is "relu2":
    down(relu(up h)^2), or "gated_silu": down(silu(gate h) * (up h)), without biases; a shared expert of the same form
    runs for every token and is added unweighted.

    params: hidden, experts, top, expert_ff, shared_ff (0 or None: no shared expert), correction (bool), score, groups
    (0 or None: none), keep, route_scale (default 1), renormalize (default True), expert (default "relu2").
    tensors: router [experts, hidden], correction [experts]; expert_up / expert_down (and expert_gate): name patterns
    with ``{e}`` for the expert's number; shared_up, shared_down (and shared_gate).  The step's (token, k) pairs are sorted
    by expert on the device and one grouped product per projection serves all experts, as in :class:`TableMoE`."""
    SMALL_PAIRS_PER_EXPERT = TableMoE.SMALL_PAIRS_PER_EXPERT
    LARGE_PAIRS_PER_EXPERT = TableMoE.LARGE_PAIRS_PER_EXPERT

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.n_experts, self.top = int(p["experts"]), int(p["top"])
        self.ff = int(p["expert_ff"])
        self.shared_ff = int(p.get("shared_ff") or 0)
        self.has_correction = bool(p.get("correction", False))
        self.score = p.get("score", "softmax")
        self.groups, self.keep = int(p.get("groups") or 0), int(p.get("keep") or 0)
        self.route_scale = float(p.get("route_scale", 1.0))
        self.renormalize = bool(p.get("renormalize", True))
        self.form = p.get("expert", "relu2")
        if self.score not in ("softmax", "sigmoid"):
            raise ValueError(f"routed_moe: score {self.score!r} (known: 'softmax', 'sigmoid')")
        if self.form not in ("relu2", "gated_silu"):
            raise ValueError(f"routed_moe: expert form {self.form!r} (known: 'relu2', 'gated_silu')")
        self.gated = self.form == "gated_silu"
        if not 1 <= self.top <= self.n_experts <= 1024:
            raise ValueError(f"routed_moe: top {self.top} of {self.n_experts} experts (up to 1024)")
        if self.groups and (self.n_experts % self.groups or not 1 <= self.keep <= self.groups
                            or self.top > self.keep * (self.n_experts // self.groups)):
            raise ValueError(f"routed_moe: {self.groups} groups of {self.n_experts} experts with {self.keep} kept cannot "
                             f"give {self.top} experts")
        rt = runtime
        pairs = rt.max_batch_tokens * self.top
        self.act_name = f"moe_act_{self.ff}"
        rt.scratch(self.act_name, pairs, self.ff)
        rt.scratch("moe_pair_out", pairs, self.hidden, torch.float32)
        rt.scratch("moe_order", 1, pairs, torch.int32)
        rt.scratch("moe_tiles", 1, 3 * self._max_tiles(pairs, min(_ROWS_PER_TILE.values())) + 4, torch.int32)
        rt.scratch("moe_delta", rt.max_batch_tokens, self.hidden, torch.float32)
        rt.scratch("router_logits", rt.max_batch_tokens, self.n_experts, torch.float32)
        rt.scratch("router_choice", 1, pairs, torch.int32)
        rt.scratch("router_weights", 1, pairs, torch.float32)
        if self.shared_ff:
            rt.scratch("moe_shared_act", rt.max_batch_tokens, self.shared_ff)
            rt.scratch("moe_shared_out", rt.max_batch_tokens, self.hidden, torch.float32)
            if self.gated:
                rt.scratch("moe_shared_gu", rt.max_batch_tokens, 2 * self.shared_ff)

    def _max_tiles(self, pairs: int, rows: int) -> int:
        return pairs // rows + min(self.n_experts, pairs)

    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["router"]: TensorNeed((self.n_experts, self.hidden))}
        if self.has_correction:
            needs[t["correction"]] = TensorNeed((self.n_experts,))
        for e in range(self.n_experts):
            if self.gated:
                needs[t["expert_gate"].format(e=e)] = TensorNeed((self.ff, self.hidden))
            needs[t["expert_up"].format(e=e)] = TensorNeed((self.ff, self.hidden))
            needs[t["expert_down"].format(e=e)] = TensorNeed((self.hidden, self.ff))
        if self.shared_ff:
            if self.gated:
                needs[t["shared_gate"]] = TensorNeed((self.shared_ff, self.hidden))
            needs[t["shared_up"]] = TensorNeed((self.shared_ff, self.hidden))
            needs[t["shared_down"]] = TensorNeed((self.hidden, self.shared_ff))
        return needs

    def load(self, tensors):
        t, E = self.spec.tensors, self.n_experts
        self.w_router = tensors[t["router"]].contiguous()
        self.correction = tensors[t["correction"]].to(torch.float32).contiguous() if self.has_correction else None
        u0 = tensors[t["expert_up"].format(e=0)]
        # bfloat16 engine with 16-byte aligned rows: the grouped products run on the tensor cores
        self.tensor_cores = (u0.dtype == torch.bfloat16 and self.runtime.dtype == torch.bfloat16
                             and self.hidden % 8 == 0 and self.ff % 8 == 0)
        if self.gated:
            # on the tensor cores gate and up rows alternate, so that the grouped product finds a gate and its up in
            # neighbouring accumulator columns; else gate rows first, up rows behind them
            join = (lambda g, u: torch.stack([g, u], dim=1).reshape(2 * self.ff, self.hidden)) if self.tensor_cores else \
                (lambda g, u: torch.cat([g, u], dim=0))
            self.w_up = torch.stack([join(tensors[t["expert_gate"].format(e=e)], tensors[t["expert_up"].format(e=e)])
                                     for e in range(E)]).contiguous()
        else:
            self.w_up = torch.stack([tensors[t["expert_up"].format(e=e)] for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[t["expert_down"].format(e=e)] for e in range(E)]).contiguous()
        if self.shared_ff:
            self.w_shared_up = tensors[t["shared_up"]].contiguous()
            self.w_shared_down = tensors[t["shared_down"]].contiguous()
            if self.gated:
                g, u = tensors[t["shared_gate"]], self.w_shared_up
                self.shared_fused = (g.dtype == torch.bfloat16 and self.runtime.dtype == torch.bfloat16 and self.hidden % 8 == 0)
                if self.shared_fused:      # gate and up rows alternate: the product's epilogue applies SiLU(gate) * up
                    self.w_shared_up = torch.stack([g, u], dim=1).reshape(2 * self.shared_ff, self.hidden).contiguous()
                else:
                    self.w_shared_up = torch.cat([g, u], dim=0).contiguous()

    def flops_per_token(self) -> float:
        m = 3 if self.gated else 2
        return 2.0 * (m * self.top * self.ff * self.hidden + m * self.shared_ff * self.hidden + self.n_experts * self.hidden)

    def forward(self, h, residual, ctx: StepContext):
        rt, T, top = self.runtime, ctx.n_tokens, self.top
        pairs = T * top
        tensor_cores = self.tensor_cores
        small = not tensor_cores and pairs <= self.SMALL_PAIRS_PER_EXPERT * self.n_experts
        large = tensor_cores and pairs >= self.LARGE_PAIRS_PER_EXPERT * self.n_experts
        rows = ops.GROUPED_ROWS_LARGE if large else _ROWS_PER_TILE[small]
        max_tiles = self._max_tiles(pairs, rows)
        order = rt.get_scratch("moe_order", torch.int32).view(-1)
        tiles = rt.get_scratch("moe_tiles", torch.int32).view(-1)
        n_tiles, tiles = tiles[:1], tiles[4:]
        act = rt.get_scratch(self.act_name)[:, : self.ff]
        pair_out = rt.get_scratch("moe_pair_out", torch.float32)[:, : self.hidden]
        logits = rt.get_scratch("router_logits", torch.float32)[:, : self.n_experts]
        choice = rt.get_scratch("router_choice", torch.int32).view(-1)[:pairs]
        weights = rt.get_scratch("router_weights", torch.float32).view(-1)[:pairs]
        ops.linear(h, self.w_router, logits, T, status=ctx.status)
        ops.router_topk(logits, self.correction, top, T, choice, weights, ctx.status, sigmoid=self.score == "sigmoid",
                        groups=self.groups, keep=self.keep, scale=self.route_scale, renormalize=self.renormalize)
        ops.moe_route(None, choice.view(T, top), self.n_experts, T, rows, order, tiles, n_tiles, ctx.status)
        if tensor_cores:
            ops.grouped_gemm_mma(h, top, self.w_up, act, order, tiles, n_tiles, max_tiles, gated=self.gated, large=large,
                                 relu2=not self.gated)
            ops.grouped_gemm_mma(act, 1, self.w_down, pair_out, order, tiles, n_tiles, max_tiles, gated=False, large=large)
        else:
            ops.grouped_linear(h, top, self.w_up, act, order, tiles, n_tiles, max_tiles, gated=self.gated, small=small,
                               relu2=not self.gated)
            ops.grouped_linear(act, 1, self.w_down, pair_out, order, tiles, n_tiles, max_tiles, gated=False, small=small)
        shared_out = None
        if self.shared_ff:
            sact = rt.get_scratch("moe_shared_act")[:, : self.shared_ff]
            shared_out = rt.get_scratch("moe_shared_out", torch.float32)[:, : self.hidden]
            if not self.gated:
                ops.linear(h, self.w_shared_up, sact, T, status=ctx.status)
                ops.relu_squared(sact, sact, T)
            elif self.shared_fused:
                ops.linear_swiglu(h, self.w_shared_up, sact, T, status=ctx.status)
            else:
                gu = rt.get_scratch("moe_shared_gu")[:, : 2 * self.shared_ff]
                ops.linear(h, self.w_shared_up, gu, T)
                ops.silu_mul(gu, sact, T)
            ops.linear(sact, self.w_shared_down, shared_out, T, status=ctx.status)
        if ctx.store_output:
            ops.moe_combine(pair_out, top, 1.0, residual, T, shared=shared_out, pair_weights=weights)
        else:
            delta = rt.get_scratch("moe_delta", torch.float32)[:, : self.hidden]
            ops.moe_combine(pair_out, top, 1.0, delta, T, shared=shared_out, pair_weights=weights)
            ops.residual_add(residual, delta, T)
