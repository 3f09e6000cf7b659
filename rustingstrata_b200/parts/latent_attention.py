"""Attention whose keys and values are expanded from a cached low-rank latent (multi-head latent attention).

Per token the mixer's input h gives q = W_q h, laid out head by head as [dim unrotated | rot_dim rotated], and
W_dkv h = [latent part (kv_rank) | one rotated key part (rot_dim) shared by all heads].  c = RMSNorm(latent part) is
the latent; head k's key is [W_uk,k c | rotated part], its value W_uv,k c, and a score is
(q_unrotated . k_unrotated + q_rotated . k_rotated) * scale over the causal keys, softmax, W_o on the joined heads.

``rot_dim`` may be 0 (no rotated parts, no position part).  With ``gate`` every head's result is multiplied by
sigmoid(w_g[h] . h), one number per token and head, before W_o.

Only [c | rotated key part] is cached: one row per token (a one-plane cache, one "kv head" that every query head
reads).  The expansion is folded into the query and the result, which gives the same numbers:

    q_unrotated . (W_uk,k c) = (W_uk,k^T q_unrotated) . c         so the query of head k becomes [W_uk,k^T q_unrotated | q_rotated],
    sum_j p_j (W_uv,k c_j)   = W_uv,k (sum_j p_j c_j)             so attention returns latent sums and W_uv,k follows,

i.e. attention with ``heads`` query heads over one shared key/value row of kv_rank + rot_dim values (rounded up to
the kernels' multiple of 16, the padding zero).  The work lists, split form and partial-result workspace are those
of :class:`~rustingstrata_b200.parts.attention.PagedAttention`; the per-head maps are block-diagonal products.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .attention import SPLIT_KEYS, PagedAttention
from .base import CallInfo, StepContext
from .registry import register_part
from .spec import CacheNeed, PartSpec, TensorNeed


@register_part("mixer", "latent_attention")
class LatentAttention(PagedAttention):
    """params: hidden, n_heads, dim (unrotated query/key size per head), rot_dim, vdim, kv_rank, scale, eps (of the
    latent's norm), window (None: every key), gate (bool, default False), weights_bits (16, the default: the tensor-core
    kernel rounds the softmax weights to bfloat16 for the weighted sum; 32: it multiplies them in two bfloat16 terms).  tensors: q_proj, dkv_proj, latent_norm, uk_proj
    [heads * dim, kv_rank], uv_proj [heads * vdim, kv_rank], o_proj, and g_proj [heads, hidden] with a gate.  The layer's position part rotates the first ``n_rot`` <= rot_dim coordinates of the rotated
    parts (pairs (2i, 2i + 1): a part whose ``pairing`` is "interleaved")."""
    chain_safe = False
    one_plane = True
    max_head_dim = 576     # what the CUDA-core attention takes: a 512-wide latent with a 64-wide rotated part

    def __init__(self, spec, runtime, position=None):
        p = spec.params
        self.dim, self.rot_dim, self.vdim = int(p["dim"]), int(p["rot_dim"]), int(p["vdim"])
        self.rank = int(p["kv_rank"])
        self.q_head = self.dim + self.rot_dim
        self.lat = (self.rank + self.rot_dim + 15) // 16 * 16            # width of a cache row and of an absorbed query head
        if self.lat > 576:
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {self.rank + self.rot_dim} exceeds the 576 values "
                             f"the attention kernels take per head")
        inner = PartSpec(spec.kind, {"hidden": p["hidden"], "n_heads": p["n_heads"], "n_kv_heads": 1, "head_dim": self.lat,
                                     "window": p.get("window"), "scale": p["scale"], "qk_norm": False}, spec.tensors)
        super().__init__(inner, runtime, position)
        self.spec = spec
        self._tensor_cores = None
        self.latent_eps = float(p["eps"])
        self.has_gate = bool(p.get("gate", False))
        self.split_weights = int(p.get("weights_bits", 16)) == 32
        self.dkv_cols = self.rank + self.rot_dim + (self.n_heads if self.has_gate else 0)
        if position is not None and getattr(position, "cos_sin", None) is not None:
            if getattr(position, "pairing", "") != "interleaved":
                raise ValueError("latent_attention rotates neighbouring pairs: its position part must be an interleaved rotation")
            if position.n_rot > self.rot_dim:
                raise ValueError(f"latent_attention: {position.n_rot} rotated coordinates exceed rot_dim {self.rot_dim}")
        rt = runtime
        rt.scratch("latent_q", rt.max_batch_tokens, self.n_heads * self.q_head)
        rt.scratch("latent_dkv", rt.max_batch_tokens, self.dkv_cols, torch.float32)
        rt.scratch("latent_o", rt.max_batch_tokens, self.n_heads * self.vdim)

    def tensor_needs(self):
        t, H = self.spec.tensors, self.n_heads
        needs = {t["q_proj"]: TensorNeed((H * self.q_head, self.hidden)),
                 t["dkv_proj"]: TensorNeed((self.rank + self.rot_dim, self.hidden)),
                 t["latent_norm"]: TensorNeed((self.rank,), "norm"),
                 t["uk_proj"]: TensorNeed((H * self.dim, self.rank)),
                 t["uv_proj"]: TensorNeed((H * self.vdim, self.rank)),
                 t["o_proj"]: TensorNeed((self.hidden, H * self.vdim))}
        if self.has_gate:
            needs[t["g_proj"]] = TensorNeed((H, self.hidden))
        return needs

    def load(self, tensors):
        t, H = self.spec.tensors, self.n_heads
        self.w_q = tensors[t["q_proj"]].contiguous()
        self.w_dkv = tensors[t["dkv_proj"]].contiguous()
        if self.has_gate:
            g = tensors[t["g_proj"]]
            if g.dtype != self.w_dkv.dtype:
                raise ValueError("latent_attention: the gate's and the latent's projections must share an element type")
            self.w_dkv = torch.cat([self.w_dkv, g], dim=0).contiguous()      # [latent | rotated key part | gates]: one product
        self.latent_norm = tensors[t["latent_norm"]].contiguous()
        # head k's key expansion transposed: [rank, dim], the map from its unrotated query to the latent's coordinates
        self.w_uk_t = tensors[t["uk_proj"]].reshape(H, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[t["uv_proj"]].reshape(H, self.vdim, self.rank).contiguous()
        self.w_o = tensors[t["o_proj"]].contiguous()

    def cache_need(self):
        return CacheNeed(1, self.lat, self.window or None, planes=1)

    @property
    def tensor_cores(self) -> bool:
        """Whether the tensor-core kernel of latent attention runs (the bfloat16 engine); else the CUDA-core kernel."""
        if self._tensor_cores is None:
            self._tensor_cores = ops.attention_latent_ok(self.runtime.dtype, self.n_heads, self.lat, self.runtime.page_size)
        return self._tensor_cores

    def plan_key(self):
        if self.q_per_cta is None and self.tensor_cores:
            self.q_per_cta = ops.attention_latent_q_per_cta(self.n_heads)
        return super().plan_key()

    def _attend(self, q, ctx: StepContext, call: CallInfo):
        if not self.tensor_cores:
            return super()._attend(q, ctx, call)
        rt = self.runtime
        out = rt.get_scratch("attn_out")[:, : self.q_width]
        plan = ctx.plans[self.plan_key()]
        common = dict(q=q, out=out, cache=call.cache, block_table=ctx.block_tables[call.cache_group], q_start=ctx.q_start,
                      kv_len=ctx.kv_len, n_heads=self.n_heads, lat=self.lat, page_size=rt.page_size, window=self.window,
                      scale=self.scale, status=ctx.status, split_weights=self.split_weights)
        if plan["n_prefill"]:
            ops.attention_latent(work=plan["prefill_work"], n_work=plan["n_prefill"], decode=False, **common)
        if plan["n_decode"]:
            ops.attention_latent(work=plan["decode_work"], n_work=plan["n_decode"], decode=True, split_keys=SPLIT_KEYS,
                                 max_splits=plan["max_splits"], split_start=plan["split_start"],
                                 total_splits=plan["total_splits"], partial=rt.get_scratch("attn_partial", torch.float32),
                                 **common)
        return out

    def flops_per_token(self) -> float:
        """Multiply-add flops of the products one token passes (the folded form the kernels run)."""
        H = self.n_heads
        return 2.0 * (H * self.q_head * self.hidden + self.dkv_cols * self.hidden + H * self.rank * self.dim
                      + H * self.vdim * self.rank + self.hidden * H * self.vdim)

    def forward(self, h, residual, ctx: StepContext, call: CallInfo):
        rt, T, H = self.runtime, ctx.n_tokens, self.n_heads
        if not call.writes_cache:
            raise RuntimeError("latent_attention: every call owns its cache")
        q = rt.get_scratch("latent_q")[:, : H * self.q_head]
        dkv = rt.get_scratch("latent_dkv", torch.float32)[:, : self.dkv_cols]
        q_lat = rt.get_scratch("qkv")[:, : H * self.lat]
        o = rt.get_scratch("latent_o")[:, : H * self.vdim]
        ops.linear(h, self.w_q, q, T, status=ctx.status)
        ops.linear(h, self.w_dkv, dkv, T, status=ctx.status)
        ops.block_linear(q, self.w_uk_t, q_lat, T, self.q_head, self.lat)
        pos = self.position
        rot = getattr(pos, "cos_sin", None) if pos is not None else None
        ops.latent_kv_write(dkv, self.latent_norm, self.latent_eps, q, self.q_head, self.dim, q_lat, rot,
                            pos.n_rot if rot is not None else 0, ctx.positions, ctx.seq_of_token,
                            ctx.block_tables[call.cache_group], rt.page_size, call.cache, self.rank, self.rot_dim, self.lat,
                            H, T, ctx.status)
        out = self._attend(q_lat, ctx, call)
        ops.block_linear(out, self.w_uv, o, T, self.lat, self.vdim)
        if self.has_gate:
            ops.head_sigmoid_gate(o, dkv[:, self.rank + self.rot_dim:], H, self.vdim, T)
        ops.linear(o, self.w_o, residual, T, accumulate=not ctx.store_output, status=ctx.status)
