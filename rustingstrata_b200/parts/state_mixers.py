"""Mixers that keep a matrix of state per head in place of a cache of keys: HGRN2, the gated delta rule with a decay
per key channel, and retention with one fixed decay per head.  All walk a float32 state S [dim, vdim] per (request, head)
token by token and read it out with a query.

``hgrn2`` (gated linear recurrence whose forget gate also decides what is written).  From the mixer's input h:
q = silu(W_q h), v = W_v h, f = l + (1 - l) sigmoid(W_f h + b_f) per head and channel, l a learned lower bound;

    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,        o_t = S_t^T q_t        (no key, no other scale);

each head's o_t is divided by its root mean square over vdim and multiplied by a weight [vdim] shared by the heads,
the heads are joined and W_o maps them back.

``gated_delta`` (delta rule with a decay per head and key channel).  q = W_q h, k = W_k h (qk heads x dim), v = W_v h
(heads x vdim), state head i reading q/k head i // (heads / qk heads); each channel of q, k, v passes a short causal
convolution over time and silu; q and k heads become unit vectors x / sqrt(sum x^2 + unit_eps), q times dim^-1/2;
beta = sigmoid(W_b h) per head; g = exp(-exp(A_h) softplus(W_a2 (W_a1 h) + dt)) per head and key channel;

    S <- diag(g_t) S;    u = beta_t (v_t - S^T k_t);    S <- S + k_t u^T;    o_t = S^T q_t

(the read-out sees the token's own write); each head's o_t divided by its root mean square over vdim, times a weight
[vdim] shared by the heads, times sigmoid(W_g2 (W_g1 h)) laid out heads x vdim; then W_o.

``retention`` (linear attention with a fixed decay per head, no softmax and no denominator).  q = W_q h, k = W_k h
(heads x dim), v = W_v h (heads x vdim), no biases; the layer's position part rotates a prefix of every q and k head;
k times dim^-1/2 after the rotation;

    S_t = decay_h S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t;

each head's o_t is divided by its root mean square over vdim (no weight), the heads are joined, multiplied by
silu(W_g h) coordinate by coordinate, and W_o maps them back.

Per request the state slot holds S for every head (zero at admission) and, for the convolution, the last taps - 1
projected rows.  The projections follow the engine's element type with float32 results; gates, decays, norms, the
state and the recurrence are float32 in both engines.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import CallInfo, Mixer, StepContext
from .registry import register_part
from .spec import StateNeed, TensorNeed


@register_part("mixer", "hgrn2")
class Hgrn2(Mixer):
    """params: hidden, n_heads, dim, vdim, eps (of the read-out norm), f_bias (bool, default True).
    tensors: q_proj, f_proj, f_bias, lower [heads * dim], v_proj, norm [vdim], o_proj."""

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.n_heads = int(p["hidden"]), int(p["n_heads"])
        self.dk, self.dv = int(p["dim"]), int(p["vdim"])
        self.eps = float(p.get("eps", 0.0))
        self.has_f_bias = bool(p.get("f_bias", True))
        self.rows_pad = ops.state_rows_pad(self.dk)
        self.qf_cols, self.v_cols = self.n_heads * self.dk, self.n_heads * self.dv
        self.in_cols = 2 * self.qf_cols + self.v_cols
        rt = runtime
        rt.scratch("state_proj", rt.max_batch_tokens, self.in_cols, torch.float32)
        rt.scratch("state_rows", 1, 3 * rt.max_batch_tokens * self.n_heads * self.rows_pad, torch.float32)
        rt.scratch("state_read", rt.max_batch_tokens, self.v_cols, torch.float32)
        rt.scratch("state_out", rt.max_batch_tokens, self.v_cols)

    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["q_proj"]: TensorNeed((self.qf_cols, self.hidden)), t["f_proj"]: TensorNeed((self.qf_cols, self.hidden)),
                 t["lower"]: TensorNeed((self.qf_cols,)), t["v_proj"]: TensorNeed((self.v_cols, self.hidden)),
                 t["norm"]: TensorNeed((self.dv,), "norm"), t["o_proj"]: TensorNeed((self.hidden, self.v_cols))}
        if self.has_f_bias:
            needs[t["f_bias"]] = TensorNeed((self.qf_cols,))
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        mats = [tensors[t["q_proj"]], tensors[t["f_proj"]], tensors[t["v_proj"]]]
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("hgrn2: the input projections must share an element type")
        self.w_in = torch.cat(mats, dim=0).contiguous()              # [q | f | v]
        self.f_bias = tensors[t["f_bias"]].to(torch.float32).contiguous() if self.has_f_bias else None
        self.lower = tensors[t["lower"]].to(torch.float32).contiguous()
        self.norm_w = tensors[t["norm"]].to(torch.float32).contiguous()
        self.w_o = tensors[t["o_proj"]].contiguous()

    def state_need(self):
        return StateNeed(self.n_heads * self.dv * self.rows_pad, "float32")

    def flops_per_token(self) -> float:
        return 2.0 * self.hidden * (self.in_cols + self.v_cols) + 6.0 * self.n_heads * self.dk * self.dv

    def forward(self, h, residual, ctx: StepContext, call: CallInfo):
        rt, T, H, RP = self.runtime, ctx.n_tokens, self.n_heads, self.rows_pad
        proj = rt.get_scratch("state_proj", torch.float32)[:, : self.in_cols]
        n = rt.max_batch_tokens * H * RP
        rows = rt.get_scratch("state_rows", torch.float32)[0]
        q, g, w = (rows[i * n:(i + 1) * n].view(rt.max_batch_tokens, H * RP) for i in range(3))
        read = rt.get_scratch("state_read", torch.float32)[:, : self.v_cols]
        out = rt.get_scratch("state_out")[:, : self.v_cols]
        ops.linear(h, self.w_in, proj, T, status=ctx.status)
        ops.hgrn2_prep(proj, self.f_bias, self.lower, q, g, w, H, self.dk, RP, T)
        ops.state_recurrence(q, w, g, None, proj[:, 2 * self.qf_cols:], read, call.state, ctx.q_start, ctx.state_slots,
                             ctx.n_seqs, H, 1, RP, self.dv, delta=False)
        ops.head_norm_gate(read, self.norm_w, None, out, H, self.dv, self.eps, T)
        ops.linear(out, self.w_o, residual, T, accumulate=not ctx.store_output, status=ctx.status)


@register_part("mixer", "gated_delta")
class GatedDelta(Mixer):
    """params: hidden, n_heads, n_qk_heads, dim, vdim, taps (0: no convolution), decay_rank, gate_rank, eps (of the
    read-out norm), unit_eps (inside the root of the unit vectors, default 1e-6).
    tensors: q_proj, k_proj, v_proj, q_conv, k_conv, v_conv [channels, taps], b_proj [heads, hidden], a_log [heads],
    a1_proj [decay_rank, hidden], a2_proj [heads * dim, decay_rank], dt_bias [heads * dim], g1_proj [gate_rank, hidden],
    g2_proj [heads * vdim, gate_rank], norm [vdim], o_proj."""

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.n_heads, self.n_qk = int(p["hidden"]), int(p["n_heads"]), int(p["n_qk_heads"])
        self.dk, self.dv = int(p["dim"]), int(p["vdim"])
        self.taps = int(p.get("taps") or 0)
        self.decay_rank, self.gate_rank = int(p["decay_rank"]), int(p["gate_rank"])
        self.eps, self.unit_eps = float(p.get("eps", 0.0)), float(p.get("unit_eps", 1e-6))
        if self.n_heads % self.n_qk:
            raise ValueError(f"gated_delta: {self.n_heads} heads are not a multiple of {self.n_qk} q/k heads")
        if self.taps > 64:
            raise ValueError(f"gated_delta: {self.taps} taps (up to 64 are supported)")
        self.rows_pad = ops.state_rows_pad(self.dk)
        self.qk_cols, self.v_cols = self.n_qk * self.dk, self.n_heads * self.dv
        self.channels = 2 * self.qk_cols + self.v_cols                   # what the convolution runs over
        self.beta_off = self.channels
        self.a1_off = self.beta_off + self.n_heads
        self.g1_off = self.a1_off + self.decay_rank
        self.in_cols = self.g1_off + self.gate_rank
        self.tail = max(0, self.taps - 1) * self.channels
        self.state_cols = self.n_heads * self.dv * self.rows_pad
        rt, mbt = runtime, runtime.max_batch_tokens
        rt.scratch("state_proj", mbt, self.in_cols, torch.float32)
        rt.scratch("state_rows", 1, mbt * (2 * self.n_qk + self.n_heads) * self.rows_pad, torch.float32)
        rt.scratch("delta_step", mbt, self.n_heads * self.dk, torch.float32)
        rt.scratch("delta_gate", mbt, self.v_cols, torch.float32)
        rt.scratch("delta_v", 1, mbt * (self.v_cols + self.n_heads), torch.float32)
        rt.scratch("state_read", mbt, self.v_cols, torch.float32)
        rt.scratch("state_out", mbt, self.v_cols)

    def tensor_needs(self):
        t, D = self.spec.tensors, self.hidden
        needs = {t["q_proj"]: TensorNeed((self.qk_cols, D)), t["k_proj"]: TensorNeed((self.qk_cols, D)),
                 t["v_proj"]: TensorNeed((self.v_cols, D)), t["b_proj"]: TensorNeed((self.n_heads, D)),
                 t["a_log"]: TensorNeed((self.n_heads,)), t["a1_proj"]: TensorNeed((self.decay_rank, D)),
                 t["a2_proj"]: TensorNeed((self.n_heads * self.dk, self.decay_rank)),
                 t["dt_bias"]: TensorNeed((self.n_heads * self.dk,)), t["g1_proj"]: TensorNeed((self.gate_rank, D)),
                 t["g2_proj"]: TensorNeed((self.v_cols, self.gate_rank)), t["norm"]: TensorNeed((self.dv,), "norm"),
                 t["o_proj"]: TensorNeed((D, self.v_cols))}
        if self.taps >= 1:
            needs.update({t["q_conv"]: TensorNeed((self.qk_cols, self.taps)), t["k_conv"]: TensorNeed((self.qk_cols, self.taps)),
                          t["v_conv"]: TensorNeed((self.v_cols, self.taps))})
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        mats = [tensors[t[n]] for n in ("q_proj", "k_proj", "v_proj", "b_proj", "a1_proj", "g1_proj")]
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("gated_delta: the input projections must share an element type")
        self.w_in = torch.cat(mats, dim=0).contiguous()              # [q | k | v | beta | a1 | g1]: h is read by one product
        self.w_a2, self.w_g2 = tensors[t["a2_proj"]].contiguous(), tensors[t["g2_proj"]].contiguous()
        self.w_o = tensors[t["o_proj"]].contiguous()
        f32 = lambda name: tensors[t[name]].to(torch.float32).contiguous()                        # noqa: E731
        self.a_log, self.dt_bias, self.norm_w = f32("a_log"), f32("dt_bias"), f32("norm")
        self.w_conv = None
        if self.taps >= 1:
            conv = torch.cat([tensors[t["q_conv"]], tensors[t["k_conv"]], tensors[t["v_conv"]]], dim=0)
            self.w_conv = conv.to(torch.float32).t().contiguous()    # tap-major, as the kernel reads it

    def state_need(self):
        # the slot's pitch stays a multiple of 16 bytes: the recurrence moves a state's rows in runs of four values
        return StateNeed(self.state_cols + (self.tail + 3) // 4 * 4, "float32")

    def flops_per_token(self) -> float:
        low_rank = self.decay_rank * self.n_heads * self.dk + self.gate_rank * self.v_cols
        return 2.0 * (self.hidden * (self.in_cols + self.v_cols) + low_rank) + 10.0 * self.n_heads * self.dk * self.dv

    def forward(self, h, residual, ctx: StepContext, call: CallInfo):
        rt, T, H, G, RP = self.runtime, ctx.n_tokens, self.n_heads, self.n_qk, self.rows_pad
        mbt = rt.max_batch_tokens
        proj = rt.get_scratch("state_proj", torch.float32)[:, : self.in_cols]
        rows = rt.get_scratch("state_rows", torch.float32)[0]
        q = rows[: mbt * G * RP].view(mbt, G * RP)
        k = rows[mbt * G * RP: 2 * mbt * G * RP].view(mbt, G * RP)
        g = rows[2 * mbt * G * RP: mbt * (2 * G + H) * RP].view(mbt, H * RP)
        step = rt.get_scratch("delta_step", torch.float32)[:, : H * self.dk]
        gate = rt.get_scratch("delta_gate", torch.float32)[:, : self.v_cols]
        vb = rt.get_scratch("delta_v", torch.float32)[0]
        v = vb[: mbt * self.v_cols].view(mbt, self.v_cols)
        beta = vb[mbt * self.v_cols: mbt * (self.v_cols + H)].view(mbt, H)
        read = rt.get_scratch("state_read", torch.float32)[:, : self.v_cols]
        out = rt.get_scratch("state_out")[:, : self.v_cols]
        ops.linear(h, self.w_in, proj, T, status=ctx.status)
        # the second halves of the two low-rank maps: decay steps and output gates, float32 in and out
        ops.linear(proj[:, self.a1_off: self.a1_off + self.decay_rank], self.w_a2, step, T, status=ctx.status)
        ops.linear(proj[:, self.g1_off: self.g1_off + self.gate_rank], self.w_g2, gate, T, status=ctx.status)
        state = call.state
        tail = state[:, self.state_cols:] if self.tail else None
        ops.delta_prep(proj, self.w_conv, tail, step, self.dt_bias, self.a_log, q, k, g, v, beta, ctx.seq_of_token, ctx.q_start,
                       ctx.state_slots, G, H, self.dk, self.dv, RP, self.beta_off, self.unit_eps, float(self.dk) ** -0.5, T,
                       ctx.n_seqs)
        ops.state_recurrence(q, k, g, beta, v, read, state, ctx.q_start, ctx.state_slots, ctx.n_seqs, H, H // G, RP, self.dv,
                             delta=True)
        ops.head_norm_gate(read, self.norm_w, gate, out, H, self.dv, self.eps, T)
        ops.linear(out, self.w_o, residual, T, accumulate=not ctx.store_output, status=ctx.status)


@register_part("mixer", "retention")
class Retention(Mixer):
    """params: hidden, n_heads, dim, vdim, decay (one number per head), eps (of the read-out norm), k_scale (default
    dim^-1/2), gate (bool, default True: the normed heads times silu(g_proj h)).
    tensors: q_proj, k_proj, v_proj, o_proj, and g_proj [heads * vdim, hidden] with a gate.  The layer's position part,
    if it has a rotation, must pair halves (coordinate i with i + n_rot / 2)."""

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.n_heads = int(p["hidden"]), int(p["n_heads"])
        self.dk, self.dv = int(p["dim"]), int(p["vdim"])
        self.decay = [float(d) for d in p["decay"]]
        if len(self.decay) != self.n_heads:
            raise ValueError(f"retention: {len(self.decay)} decays for {self.n_heads} heads")
        self.eps = float(p.get("eps", 0.0))
        self.k_scale = float(p["k_scale"]) if p.get("k_scale") is not None else float(self.dk) ** -0.5
        self.has_gate = bool(p.get("gate", True))
        self.position = position
        self.n_rot = int(getattr(position, "n_rot", 0) or 0)
        if self.n_rot and getattr(position, "pairing", "half") != "half":
            raise ValueError("retention: its kernel pairs the halves of the rotated prefix; the position part pairs otherwise")
        if self.n_rot > self.dk:
            raise ValueError(f"retention: {self.n_rot} rotated coordinates in heads of {self.dk}")
        self.rows_pad = ops.state_rows_pad(self.dk)
        self.qk_cols, self.v_cols = self.n_heads * self.dk, self.n_heads * self.dv
        self.in_cols = 2 * self.qk_cols + self.v_cols * (2 if self.has_gate else 1)
        rt = runtime
        rt.scratch("state_proj", rt.max_batch_tokens, self.in_cols, torch.float32)
        rt.scratch("state_rows", 1, 2 * rt.max_batch_tokens * self.n_heads * self.rows_pad, torch.float32)
        rt.scratch("state_read", rt.max_batch_tokens, self.v_cols, torch.float32)
        rt.scratch("state_out", rt.max_batch_tokens, self.v_cols)
        self.decay_rows = None

    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["q_proj"]: TensorNeed((self.qk_cols, self.hidden)), t["k_proj"]: TensorNeed((self.qk_cols, self.hidden)),
                 t["v_proj"]: TensorNeed((self.v_cols, self.hidden)), t["o_proj"]: TensorNeed((self.hidden, self.v_cols))}
        if self.has_gate:
            needs[t["g_proj"]] = TensorNeed((self.v_cols, self.hidden))
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        mats = [tensors[t[n]] for n in ("q_proj", "k_proj", "v_proj")] + ([tensors[t["g_proj"]]] if self.has_gate else [])
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("retention: the input projections must share an element type")
        self.w_in = torch.cat(mats, dim=0).contiguous()              # [q | k | v | gate]: h is read by one product
        self.w_o = tensors[t["o_proj"]].contiguous()
        # the decay of every row of every head, one row that all tokens read
        d = torch.tensor(self.decay, dtype=torch.float32).view(self.n_heads, 1).expand(self.n_heads, self.rows_pad)
        self.decay_rows = d.reshape(1, -1).contiguous().to(self.w_o.device)

    def state_need(self):
        return StateNeed(self.n_heads * self.dv * self.rows_pad, "float32")

    def flops_per_token(self) -> float:
        return 2.0 * self.hidden * (self.in_cols + self.v_cols) + 6.0 * self.n_heads * self.dk * self.dv

    def forward(self, h, residual, ctx: StepContext, call: CallInfo):
        rt, T, H, RP = self.runtime, ctx.n_tokens, self.n_heads, self.rows_pad
        proj = rt.get_scratch("state_proj", torch.float32)[:, : self.in_cols]
        n = rt.max_batch_tokens * H * RP
        rows = rt.get_scratch("state_rows", torch.float32)[0]
        q, k = (rows[i * n:(i + 1) * n].view(rt.max_batch_tokens, H * RP) for i in range(2))
        read = rt.get_scratch("state_read", torch.float32)[:, : self.v_cols]
        out = rt.get_scratch("state_out")[:, : self.v_cols]
        ops.linear(h, self.w_in, proj, T, status=ctx.status)
        rot = getattr(self.position, "cos_sin", None) if self.n_rot else None
        ops.retention_prep(proj, rot, self.n_rot, ctx.positions, self.k_scale, q, k, H, self.dk, RP, T, ctx.status)
        g = self.decay_rows.expand(T, H * RP)                        # pitch 0: the same decays for every token
        v_off = 2 * self.qk_cols
        ops.state_recurrence(q, k, g, None, proj[:, v_off: v_off + self.v_cols], read, call.state, ctx.q_start,
                             ctx.state_slots, ctx.n_seqs, H, 1, RP, self.dv, delta=False)
        gate = proj[:, v_off + self.v_cols:] if self.has_gate else None
        ops.head_norm_gate(read, None, gate, out, H, self.dv, self.eps, T, gate_silu=True)
        ops.linear(out, self.w_o, residual, T, accumulate=not ctx.store_output, status=ctx.status)
