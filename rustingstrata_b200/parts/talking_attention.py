"""Attention over a paged key/value cache whose scores are mixed across heads before the softmax, with a learned sink
in every head's denominator and a sigmoid gate per head.

Per token, from the mixer's input h:  q = W_q h + b_q (heads x dim), k = W_k h + b_k, v = W_v h + b_v (kv heads x dim /
vdim; query head i reads kv head i // (heads / kv heads)).  Every q and k head is divided by its root mean square and
multiplied by a weight of ``dim`` values shared by the heads (``norm`` "head"), or the whole q row and the whole k row
are each divided by their root mean square and multiplied by a weight per coordinate (``norm`` "row"); the position
encoding then rotates the first ``n_rot`` coordinates of each q and k head, in neighbouring pairs or, for a part that
pairs halves, coordinate i with i + n_rot / 2.  With raw[g, i, j] = (q_gi . k_gj) * scale the score of head h is

    mixed[h, i, j] = sum_g talk[h, g] raw[g, i, j]                      (talk [heads, heads]; None: the raw score)

and the weights of query i over the keys j <= i (within ``window`` if there is one; with ``chunk`` only keys of the
query's own block of that many positions, floor(i / chunk) = floor(j / chunk), blocks counted from position 0) are

    exp(mixed[h, i, j]) / (exp(sink[h]) + sum_j' exp(mixed[h, i, j']))  (sink [heads]; None: no such term).

The sink has no key and no value, is neither scaled nor mixed, and counts once.  Head h's weighted sum of values is
multiplied by sigmoid(w_g[h] . h), and W_o maps the joined heads back to the stream.  Norms, angles, scores, the mix,
weights and gates are float32 in both engines; keys and values are cached in the engine's element type, in rows
padded to a common size.  Each of bias, norm, talk, sink and gate is a parameter of the part and may be left out.
"""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import CallInfo, HostBatch, Mixer, StepContext
from .registry import register_part
from .spec import CacheNeed, TensorNeed


KEY_TILE = 32              # keys per tile of the tensor-core form
MMA_SINGLE_Q = 4           # its query tile in a step of single tokens (the smallest it has: more CTAs fit a multiprocessor)
FILL_CTAS = 148            # one CTA per multiprocessor
MAX_PARTS = 32
MIN_PART_TILES = 4         # a part walks at least this many key tiles
PARTIAL_ROWS = 4096        # (query, part) rows of partial sums the workspace holds


@register_part("mixer", "talking_attention")
class TalkingAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, dim, vdim, scale, eps, window (None: every key), chunk (None: no blocks),
    bias, qk_norm, talk, sink, gate (bools, default True), norm ("head", the default, or "row").  tensors: q_proj, k_proj,
    v_proj, o_proj, and as the params ask q_bias, k_bias, v_bias, q_norm, k_norm ([dim] each; "row": [heads * dim] and
    [kv heads * dim]), talk [heads, heads], sink [heads], g_proj [heads, hidden]."""

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.n_heads, self.n_kv = int(p["n_heads"]), int(p["n_kv_heads"])
        self.dk, self.dv = int(p["dim"]), int(p["vdim"])
        self.scale = float(p["scale"])
        self.eps = float(p.get("eps", 0.0))
        self.window = int(p["window"]) if p.get("window") else 0
        self.chunk = int(p["chunk"]) if p.get("chunk") else 0
        self.row_norm = p.get("norm", "head") == "row"
        if p.get("norm", "head") not in ("head", "row"):
            raise ValueError(f"talking_attention: norm {p.get('norm')!r} (known: 'head', 'row')")
        self.has_bias, self.qk_norm = bool(p.get("bias", True)), bool(p.get("qk_norm", True))
        self.has_talk, self.has_sink, self.has_gate = bool(p.get("talk", True)), bool(p.get("sink", True)), bool(p.get("gate", True))
        self.position = position
        if self.n_heads % self.n_kv:
            raise ValueError(f"talking_attention: {self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        if max(self.dk, self.dv) > 256:
            raise ValueError(f"talking_attention: head sizes {self.dk} / {self.dv} exceed the 256 the kernels take")
        n_rot = int(getattr(position, "n_rot", 0) or 0)
        self.half_pairs = bool(n_rot) and getattr(position, "pairing", "half") != "interleaved"
        if n_rot > self.dk:
            raise ValueError(f"talking_attention: {n_rot} rotated coordinates in heads of {self.dk}")
        self.head_pad = (max(self.dk, self.dv) + 7) // 8 * 8           # cache rows start on 16 bytes in both element types
        self.q_cols, self.k_cols, self.v_cols = self.n_heads * self.dk, self.n_kv * self.dk, self.n_kv * self.dv
        self.g_cols = self.n_heads if self.has_gate else 0
        self.in_cols = self.q_cols + self.k_cols + self.v_cols + self.g_cols
        self.o_in = self.n_heads * self.dv
        self.q_per_cta = None
        self.mma_q = 0
        rt = runtime
        if not rt.precise:
            rt.scratch("talk_partial", PARTIAL_ROWS, self.n_heads * (self.dv + 2), torch.float32)
        rt.scratch("talk_proj", rt.max_batch_tokens, self.in_cols, torch.float32)
        rt.scratch("talk_q", rt.max_batch_tokens, self.q_cols, torch.float32)
        rt.scratch("talk_gate", 1, rt.max_batch_tokens * self.n_heads, torch.float32)      # flat: [T, heads] without a pitch
        rt.scratch("talk_out", rt.max_batch_tokens, self.o_in)

    # ---------------------------------------------------------------- weights
    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["q_proj"]: TensorNeed((self.q_cols, self.hidden)), t["k_proj"]: TensorNeed((self.k_cols, self.hidden)),
                 t["v_proj"]: TensorNeed((self.v_cols, self.hidden)), t["o_proj"]: TensorNeed((self.hidden, self.o_in))}
        if self.has_bias:
            needs.update({t["q_bias"]: TensorNeed((self.q_cols,)), t["k_bias"]: TensorNeed((self.k_cols,)),
                          t["v_bias"]: TensorNeed((self.v_cols,))})
        if self.qk_norm:
            nq, nk = (self.q_cols, self.k_cols) if self.row_norm else (self.dk, self.dk)
            needs.update({t["q_norm"]: TensorNeed((nq,), "norm"), t["k_norm"]: TensorNeed((nk,), "norm")})
        if self.has_talk:
            needs[t["talk"]] = TensorNeed((self.n_heads, self.n_heads), "average")
        if self.has_sink:
            needs[t["sink"]] = TensorNeed((self.n_heads,))
        if self.has_gate:
            needs[t["g_proj"]] = TensorNeed((self.n_heads, self.hidden))
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        mats = [tensors[t["q_proj"]], tensors[t["k_proj"]], tensors[t["v_proj"]]] + ([tensors[t["g_proj"]]] if self.has_gate else [])
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("talking_attention: the input projections must share an element type")
        self.w_in = torch.cat(mats, dim=0).contiguous()              # one [q | k | v | gate] matrix: h is read by one product
        self.w_o = tensors[t["o_proj"]].contiguous()
        f32 = lambda name: tensors[t[name]].to(torch.float32).contiguous()                        # noqa: E731
        self.bias = torch.cat([f32("q_bias"), f32("k_bias"), f32("v_bias")]) if self.has_bias else None
        self.q_norm_w = f32("q_norm") if self.qk_norm else None
        self.k_norm_w = f32("k_norm") if self.qk_norm else None
        self.talk = f32("talk") if self.has_talk else None
        self.sink = f32("sink") if self.has_sink else None

    # ---------------------------------------------------------------- what it keeps
    def cache_need(self):
        # a block of ``chunk`` positions never reaches further back than chunk keys, the query's own included
        reach = [w for w in (self.window, self.chunk) if w]
        return CacheNeed(self.n_kv, self.head_pad, min(reach) if reach else None)

    def flops_per_token(self) -> float:
        return 2.0 * self.hidden * (self.in_cols + self.o_in)

    def mixing_flops(self, q_lens, kv_lens) -> float:
        pairs = 0.0
        for q, kv in zip(np.asarray(q_lens, dtype=np.int64), np.asarray(kv_lens, dtype=np.int64)):
            pos = np.arange(kv - q, kv, dtype=np.float64)
            seen = pos + 1 if not self.window else np.minimum(pos + 1, self.window)
            if self.chunk:
                seen = np.minimum(seen, pos % self.chunk + 1)
            pairs += float(seen.sum())
        mix = 2.0 * self.n_heads * self.n_heads if self.has_talk else 0.0
        return (2.0 * self.n_heads * (self.dk + self.dv) + mix) * pairs

    # ---------------------------------------------------------------- planning
    def _setup(self):
        if self.q_per_cta is None:
            self.q_per_cta = ops.talking_attention_q_per_cta(self.n_heads, self.dk, self.dv)
            # the tensor-core form reads a bfloat16 cache; the 32-bit engine and shapes it does not take use the other
            self.mma_q = 0 if self.runtime.precise else ops.talking_attention_mma_q_per_cta(self.n_heads, self.n_kv, self.dk, self.dv)

    def plan_key(self):
        self._setup()
        return ("talking_attention", self.q_per_cta, self.mma_q, self.window, self.chunk)

    def build_plan(self, batch: HostBatch):
        """Tiles of neighbouring queries of one sequence, the ones with the most keys to walk first.  For the tensor-core
        form a tile's key tiles are dealt out over several CTAs when the step has too few tiles to fill the device."""
        self._setup()
        single = int(batch.q_lens.max()) == 1
        qt = (MMA_SINGLE_Q if single else self.mma_q) if self.mma_q else (1 if single else self.q_per_cta)
        tiles = []
        for s in range(batch.n_seqs):
            offs = np.arange(0, batch.q_lens[s], qt, dtype=np.int32)
            tiles.append(np.stack([np.full_like(offs, s), offs], axis=1))
        work = np.concatenate(tiles, axis=0).astype(np.int32)
        first = batch.kv_lens[work[:, 0]] - batch.q_lens[work[:, 0]] + work[:, 1]        # position of the tile's first query
        if len(work) > 1 and not batch.bucketed:
            order = np.argsort(-first, kind="stable")
            work, first = work[order], first[order]
        if not self.mma_q:
            return {"work": work.reshape(-1), "n_work": int(work.shape[0]), "any_parts": 0, "qt": qt}
        n = work.shape[0]
        nq = np.minimum(qt, batch.q_lens[work[:, 0]] - work[:, 1])
        parts = np.ones(n, dtype=np.int64)
        # single tokens: one wave of CTAs (each is mostly fixed cost); portions: up to two, which also evens out the
        # unequal walks of a causal portion's tiles
        fill = FILL_CTAS if single else 2 * FILL_CTAS
        if n <= fill // 2:
            share = min(MAX_PARTS, fill // n)
            if batch.bucketed:
                parts[:] = share              # a captured step: the launch shape must not follow the lengths
            else:
                begin = np.maximum(0, first - self.window + 1) if self.window else np.zeros(n, dtype=np.int64)
                if self.chunk:
                    begin = np.maximum(begin, first // self.chunk * self.chunk)
                key_tiles = -(-(first + nq) // KEY_TILE) - begin // KEY_TILE
                parts = np.clip(key_tiles // MIN_PART_TILES, 1, share)
            while int((parts * nq)[parts > 1].sum()) > PARTIAL_ROWS:
                parts = np.maximum(1, parts // 2)
        rows = np.where(parts > 1, parts * nq, 0)
        base = np.concatenate([[0], np.cumsum(rows)[:-1]])
        rep = np.repeat(np.arange(n), parts)
        part = np.arange(len(rep)) - np.repeat(np.cumsum(parts) - parts, parts)
        full = np.stack([work[rep, 0], work[rep, 1], part, parts[rep], base[rep]], axis=1).astype(np.int32)
        return {"work": full.reshape(-1), "n_work": int(full.shape[0]), "any_parts": int(bool((parts > 1).any())), "qt": qt}

    # ---------------------------------------------------------------- the step
    def forward(self, h, residual, ctx: StepContext, call: CallInfo):
        rt, T = self.runtime, ctx.n_tokens
        if not call.writes_cache:
            raise RuntimeError("talking_attention: every call owns its cache")
        proj = rt.get_scratch("talk_proj", torch.float32)[:, : self.in_cols]
        q = rt.get_scratch("talk_q", torch.float32)[:, : self.q_cols]
        gate = rt.get_scratch("talk_gate", torch.float32)[0, : rt.max_batch_tokens * self.n_heads] \
            .view(rt.max_batch_tokens, self.n_heads) if self.has_gate else None
        out = rt.get_scratch("talk_out")[:, : self.o_in]
        ops.linear(h, self.w_in, proj, T, status=ctx.status)
        table = ctx.block_tables[call.cache_group]
        pos = self.position
        rot = getattr(pos, "cos_sin", None) if pos is not None else None
        ops.talking_attention_prep(proj, self.bias, self.q_norm_w, self.k_norm_w, self.eps, rot,
                                   int(pos.n_rot) if rot is not None else 0, q, gate, call.cache, table, rt.page_size,
                                   ctx.positions, ctx.seq_of_token, self.n_heads, self.n_kv, self.dk, self.dv, T, True, ctx.status,
                                   row_norm=self.row_norm, half_pairs=self.half_pairs)
        plan = ctx.plans[self.plan_key()]
        if self.mma_q:
            partial = rt.get_scratch("talk_partial", torch.float32) if plan["any_parts"] else None
            ops.talking_attention_mma(q, gate, call.cache, table, rt.page_size, ctx.q_start, ctx.kv_len, plan["work"],
                                      plan["n_work"], bool(plan["any_parts"]), self.talk, self.sink, out, partial, self.n_heads,
                                      self.n_kv, self.dk, self.dv, self.window, plan["qt"], self.scale, ctx.status, chunk=self.chunk)
        else:
            # a step of single tokens: a CTA's shared memory is sized for its one query
            ops.talking_attention(q, gate, call.cache, table, rt.page_size, ctx.q_start, ctx.kv_len, plan["work"],
                                  plan["n_work"], self.talk, self.sink, out, self.n_heads, self.n_kv, self.dk, self.dv,
                                  self.window, plan["qt"], self.scale, ctx.status, chunk=self.chunk)
        ops.linear(out, self.w_o, residual, T, accumulate=not ctx.store_output, status=ctx.status)
