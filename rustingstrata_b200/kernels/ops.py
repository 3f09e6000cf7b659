"""Python launchers of the CUDA kernels: torch tensors in, raw pointers out.

Every function launches on torch's current CUDA stream, checks what it can on the
host (devices, element types, shapes, contiguity, alignment) and raises on a bad
launch.  There is no CPU path and no library fallback: if the extension cannot be
built or loaded the first call raises :class:`~.build.KernelBuildError`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_long, c_float, c_void_p
from typing import Optional

import torch

from ..dtypes import element_type
from .build import load_library

F32, BF16 = element_type("float32").code, element_type("bfloat16").code

STATUS_BAD_TOKEN = 1
STATUS_BAD_PAGE = 2
STATUS_WAIT_EXPIRED = 4
STATUS_NON_FINITE = 8
STATUS_BAD_PLAN = 16


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"unsupported element type {t.dtype} (float32 and bfloat16 only)")
    return element_type(t.dtype).code


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    """The stream to launch on.  Every launcher asks for it right before its launch, so this is also where a recorded
    chain of decode products (see :func:`begin_chain`) is sent off before any other kernel can overtake it."""
    flush_chain()
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_LAUNCHES = 0


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the decode-path kernels (default on); off gives plain stream order."""
    core().rs_core_set_pdl(1 if on else 0)
    bf16lib().rs_bf16_set_pdl(1 if on else 0)


def launch_count() -> int:
    """Kernels of this package launched so far by this process."""
    return _LAUNCHES


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _LAUNCHES
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    _LAUNCHES += kernels


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel launchers take CUDA tensors only; there is no CPU path")


def _rows_contiguous(t: torch.Tensor, name: str):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-D with unit stride along its last axis, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")


_core = None


def core():
    global _core
    if _core is None:
        lib = load_library("core")
        lib.rs_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.rs_gather_i32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        lib.rs_rmsnorm.argtypes = [c_void_p, c_long, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_long,
                                   c_int, c_int, c_void_p]
        lib.rs_qk_norm_rope_kv.argtypes = [c_void_p, c_int, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                           c_float, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                           c_int, c_int, c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.rs_silu_mul.argtypes = [c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p]
        lib.rs_head_sigmoid_gate.argtypes = [c_void_p, c_int, c_long, c_void_p, c_long, c_int, c_int, c_int, c_void_p]
        lib.rs_residual_add.argtypes = [c_void_p, c_void_p, c_int, c_long, c_void_p]
        lib.rs_linear_simt.argtypes = [c_void_p, c_int, c_long, c_void_p, c_int, c_long, c_void_p, c_int, c_long,
                                       c_int, c_int, c_int, c_int, c_void_p]
        lib.rs_attention_simt.argtypes = [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int,
                                          c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                          c_int, c_int, c_void_p, c_void_p]
        lib.rs_attention_simt_q_per_cta.argtypes = [c_int, c_int]
        lib.rs_attention_simt_partial_floats.argtypes = [c_int, c_int, c_int]
        lib.rs_attention_simt_partial_floats.restype = c_long
        lib.rs_fill_random.argtypes = [c_void_p, c_int, c_long, ctypes.c_ulonglong, c_long, c_void_p, c_float, c_float,
                                       c_void_p]
        lib.rs_sample.argtypes = [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.rs_rmsnorm_add.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_int, c_int, c_float, c_void_p, c_int,
                                       c_int, c_float, c_void_p, c_int, c_long, c_int, c_int, c_void_p]
        lib.rs_concat_embed.argtypes = [c_void_p, c_long, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                        c_long, c_int, c_int, c_void_p, c_void_p]
        lib.rs_short_conv.argtypes = [c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                      c_int, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_int, c_int, c_void_p]
        lib.rs_block_linear.argtypes = [c_void_p, c_int, c_long, c_long, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                        c_long, c_long, c_int, c_int, c_int, c_int, c_void_p]
        lib.rs_gated_linear_recurrence.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_void_p, c_int,
                                                   c_void_p, c_int, c_void_p, c_int, c_long, c_void_p, c_long, c_void_p,
                                                   c_void_p, c_int, c_int, c_float, c_int, c_void_p]
        lib.rs_gated_linear_recurrence_chunked.argtypes = lib.rs_gated_linear_recurrence.argtypes[:-1] + [
            c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.rs_latent_kv_write.argtypes = [c_void_p, c_long, c_void_p, c_int, c_float, c_void_p, c_int, c_long, c_int, c_int,
                                           c_void_p, c_int, c_long, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                                           c_void_p, c_int, c_int, c_void_p, c_int, c_long, c_int, c_int, c_int, c_int,
                                           c_int, c_int, c_void_p, c_void_p]
        lib.rs_relu_squared.argtypes = [c_void_p, c_int, c_long, c_void_p, c_long, c_int, c_int, c_void_p]
        lib.rs_moe_route.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                     c_int, c_void_p, c_void_p]
        lib.rs_grouped_linear_rows_per_tile.argtypes = [c_int]
        lib.rs_grouped_linear.argtypes = [c_void_p, c_int, c_long, c_int, c_void_p, c_int, c_long, c_void_p, c_int, c_long,
                                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.rs_moe_combine.argtypes = [c_void_p, c_long, c_int, c_float, c_void_p, c_void_p, c_int, c_long, c_void_p, c_int, c_long,
                                       c_void_p, c_int, c_void_p, c_long, c_int, c_int, c_void_p]
        _core = lib
    return _core


# ----------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[t] = table[ids[t]] as float32.  ids int32 [T]; out float32 [T, H]."""
    _cuda(table, ids, out, status)
    T, H = out.shape
    if ids.dtype != torch.int32 or out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed: ids must be int32, out contiguous float32, table contiguous")
    if table.shape[1] != H or ids.numel() < T:
        raise KernelError(f"embed: table {tuple(table.shape)} / ids {ids.numel()} do not fit out {tuple(out.shape)}")
    _check(core().rs_embed(_ptr(table), dtype_code(table), _ptr(ids), _ptr(out), T, H, table.shape[0], _ptr(status),
                           _stream()), "embed")


def gather_i32(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor, n: int) -> None:
    """dst[i] = src[idx[i]] for i < n, all int32 on the device (idx must point inside src)."""
    _cuda(dst, src, idx)
    if dst.dtype != torch.int32 or src.dtype != torch.int32 or idx.dtype != torch.int32 or dst.numel() < n or idx.numel() < n:
        raise KernelError("gather_i32: int32 tensors with at least n entries")
    _check(core().rs_gather_i32(_ptr(dst), _ptr(src), _ptr(idx), n, _stream()), "gather_i32")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None, pending=None) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight.  x float32 [*, n].

    ``pending``: a :class:`PendingSum` still owed to ``x``.  If it covers exactly the rows that are normed, one kernel
    adds the partial sums and norms the rows (the same bits as the two kernels in turn); else it is finished first."""
    _cuda(x, weight, out, rows)
    if _ACTIVE_CHAIN is not None and _ACTIVE_CHAIN.ops and pending is None and rows is None:
        nr = n_rows if n_rows is not None else x.shape[0]
        lib = bf16lib()
        if (nr <= lib.rs_decode_chain_max_rows() and x.dtype == torch.float32 and out.dtype == torch.bfloat16
                and x.dim() == 2 and out.dim() == 2 and x.stride(1) == 1 and out.stride(1) == 1
                and x.shape[1] == weight.numel() == out.shape[1] and x.shape[1] % 4 == 0
                and x.shape[1] <= lib.rs_decode_chain_max_norm_width() and x.stride(0) % 4 == 0 and out.stride(0) % 4 == 0
                and x.data_ptr() % 16 == 0 and out.data_ptr() % 8 == 0 and weight.data_ptr() % 16 == 0
                and weight.is_contiguous() and weight.dtype in (torch.float32, torch.bfloat16) and nr <= out.shape[0]):
            _ACTIVE_CHAIN.add_rmsnorm(x, weight, eps, out, nr)
            return
    if pending is not None and not pending.done:
        nr = n_rows if n_rows is not None else (out.shape[0] if rows is not None else x.shape[0])
        lib = bf16lib()
        if (rows is None and pending.out.data_ptr() == x.data_ptr() and pending.out.stride(0) == x.stride(0)
                and pending.n_rows == nr and pending.N == x.shape[1] == weight.numel() == out.shape[1]
                and x.dtype == torch.float32 and out.dtype == torch.bfloat16 and weight.is_contiguous()
                and weight.dtype in (torch.float32, torch.bfloat16) and nr <= out.shape[0] and x.stride(1) == 1 and out.stride(1) == 1
                and lib.rs_skinny_finish_rmsnorm_supported(_ptr(x), x.stride(0), pending.N, _ptr(weight), _ptr(out), out.stride(0))):
            pending.finish_with_rmsnorm(weight, eps, out)
            return
        pending.finish()
    _rows_contiguous(x, "rmsnorm x")
    _rows_contiguous(out, "rmsnorm out")
    n = x.shape[1]
    if x.dtype != torch.float32:
        raise KernelError("rmsnorm reads the float32 residual stream")
    if weight.numel() != n or out.shape[1] != n or not weight.is_contiguous():
        raise KernelError(f"rmsnorm: weight {tuple(weight.shape)} / out {tuple(out.shape)} do not fit width {n}")
    if n_rows is None:
        n_rows = out.shape[0] if rows is not None else x.shape[0]
    if n_rows > out.shape[0] or (rows is None and n_rows > x.shape[0]):
        raise KernelError("rmsnorm: more rows than the buffers hold")
    if rows is not None and (rows.dtype != torch.int32 or rows.numel() < n_rows):
        raise KernelError("rmsnorm: rows must be int32 with n_rows entries")
    _check(core().rs_rmsnorm(_ptr(x), x.stride(0), _ptr(rows), _ptr(weight), dtype_code(weight), float(eps),
                             _ptr(out), dtype_code(out), out.stride(0), n_rows, n, _stream()), "rmsnorm")


def qk_norm_rope_kv(qkv: torch.Tensor, n_tokens: int, n_q: int, n_kv: int, head_dim: int,
                    q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                    cos_sin: Optional[torch.Tensor], n_rot: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                    block_table: torch.Tensor, page_size: int, cache: torch.Tensor, write_kv: bool,
                    status: torch.Tensor, stream: int = 0) -> None:
    """Per-head norm and rotation of q (in place) and k, and the write of k and v into their pages.

    qkv: [T, (n_q + 2 n_kv) * head_dim] (only the q part when ``write_kv`` is false);
    cache: [pages, 2, n_kv, page_size, head_dim] of the same element type.
    positions: [T] or [T, n_streams] int32; column 0 is the token's place in the cache, column ``stream`` the
    position the rotation follows (a row of ``cos_sin``).
    """
    _cuda(qkv, q_weight, k_weight, cos_sin, positions, seq_of_token, block_table, cache, status)
    _rows_contiguous(qkv, "qkv")
    need = (n_q + (2 * n_kv if write_kv else 0)) * head_dim
    if qkv.shape[1] < need or qkv.shape[0] < n_tokens:
        raise KernelError(f"qk_norm_rope_kv: qkv {tuple(qkv.shape)} is smaller than {n_tokens} x {need}")
    if cache.dtype != qkv.dtype or not cache.is_contiguous():
        raise KernelError("qk_norm_rope_kv: cache must be contiguous and of the activations' element type")
    if tuple(cache.shape[1:]) != (2, n_kv, page_size, head_dim):
        raise KernelError(f"qk_norm_rope_kv: cache shape {tuple(cache.shape)} is not [pages, 2, {n_kv}, {page_size}, "
                          f"{head_dim}]")
    w_dt = F32
    for w in (q_weight, k_weight):
        if w is not None:
            if w.numel() != head_dim or not w.is_contiguous():
                raise KernelError("qk_norm_rope_kv: norm weights must hold head_dim values")
            w_dt = dtype_code(w)
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("qk_norm_rope_kv: q and k norm weights must share an element type")
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or cos_sin.shape[1] != n_rot or
                                not cos_sin.is_contiguous()):
        raise KernelError("qk_norm_rope_kv: cos_sin must be contiguous float32 [positions, n_rot]")
    for name, t in (("positions", positions), ("seq_of_token", seq_of_token), ("block_table", block_table)):
        if t.dtype != torch.int32:
            raise KernelError(f"qk_norm_rope_kv: {name} must be int32")
    n_streams = 1 if positions.dim() == 1 else positions.shape[1]
    if positions.dim() > 2 or not positions.is_contiguous() or positions.shape[0] < n_tokens or not 0 <= stream < n_streams:
        raise KernelError(f"qk_norm_rope_kv: positions must be contiguous [tokens] or [tokens, streams] and hold stream "
                          f"{stream}; got shape {tuple(positions.shape)}")
    _check(core().rs_qk_norm_rope_kv(
        _ptr(qkv), dtype_code(qkv), qkv.stride(0), n_q, n_kv, head_dim, _ptr(q_weight), _ptr(k_weight), w_dt,
        float(eps), _ptr(cos_sin), n_rot, 0 if cos_sin is None else cos_sin.shape[0], _ptr(positions), n_streams, stream,
        _ptr(seq_of_token), _ptr(block_table),
        block_table.stride(0), page_size, _ptr(cache), cache.stride(0), cache.shape[0], 1 if write_kv else 0,
        n_tokens, _ptr(status), _stream()), "qk_norm_rope_kv")


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, n_rows: int, activation: str = "silu") -> None:
    """out[r, c] = act(gate_up[r, c]) * gate_up[r, I + c], I = out.shape[1]; act is SiLU or ("gelu_tanh") the tanh
    form of GELU."""
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"silu_mul: unknown activation '{activation}' (known: {', '.join(sorted(GATE_ACTIVATIONS))})")
    _cuda(gate_up, out)
    _rows_contiguous(gate_up, "gate_up")
    _rows_contiguous(out, "out")
    I = out.shape[1]
    if gate_up.shape[1] != 2 * I or gate_up.dtype != out.dtype or n_rows > min(gate_up.shape[0], out.shape[0]):
        raise KernelError(f"silu_mul: gate_up {tuple(gate_up.shape)} does not fit out {tuple(out.shape)}")
    _check(core().rs_silu_mul(_ptr(gate_up), gate_up.stride(0), _ptr(out), out.stride(0), dtype_code(out), n_rows, I,
                              GATE_ACTIVATIONS[activation], _stream()), "silu_mul")


def head_sigmoid_gate(a: torch.Tensor, gate: torch.Tensor, n_heads: int, dv: int, n_tokens: int) -> None:
    """a[t, h * dv + d] *= sigmoid(gate[t, h]) in place; gate float32 [T, >= heads] (pre-activations)."""
    _cuda(a, gate)
    _rows_contiguous(a, "head_sigmoid_gate a")
    if gate.dtype != torch.float32 or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape[1] < n_heads \
            or a.shape[1] < n_heads * dv or n_tokens > min(a.shape[0], gate.shape[0]):
        raise KernelError("head_sigmoid_gate: a [T, heads * dv], gate float32 [T, heads]")
    _check(core().rs_head_sigmoid_gate(_ptr(a), dtype_code(a), a.stride(0), _ptr(gate), gate.stride(0), n_heads, dv, n_tokens,
                                       _stream()), "head_sigmoid_gate")


def residual_add(x: torch.Tensor, delta: torch.Tensor, n_rows: int) -> None:
    """x[:n_rows] += delta[:n_rows] in float32 (both contiguous, same width)."""
    _cuda(x, delta)
    if x.dtype != torch.float32 or not x.is_contiguous() or not delta.is_contiguous() or x.shape[1] != delta.shape[1]:
        raise KernelError("residual_add: x must be contiguous float32 and delta contiguous of the same width")
    _check(core().rs_residual_add(_ptr(x), _ptr(delta), dtype_code(delta), n_rows * x.shape[1], _stream()),
           "residual_add")


def fill_random(out: torch.Tensor, key: int, table: Optional[torch.Tensor], scale: float, shift: float,
                first: int = 0) -> None:
    """out.flatten()[i] = shift + scale * table[z_i >> 48] with z_i the 64-bit hash of (key, first + i): the device
    half of the random-weights generator (weights/random_init.py is the host half and gives the same bits).
    ``out`` float32 or bfloat16; int32 takes the low bit of z_i and needs no table."""
    _cuda(out, table)
    if not out.is_contiguous():
        raise KernelError("fill_random: out must be contiguous")
    if out.dtype == torch.int32:
        code = element_type("int32").code
    else:
        code = dtype_code(out)
        if table is None or table.dtype != torch.float32 or table.numel() != 1 << 16 or not table.is_contiguous():
            raise KernelError("fill_random: table must be the 65,536 float32 normal quantiles")
    _check(core().rs_fill_random(_ptr(out), code, out.numel(), key & 0xFFFFFFFFFFFFFFFF, first, _ptr(table), float(scale),
                                 float(shift), _stream()), "fill_random")


# ----------------------------------------------------------------------------- matrix products
def linear_simt(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False) -> None:
    """out[:n_rows] (=|+=) a[:n_rows] @ weight.T on CUDA cores, float32 accumulation."""
    _cuda(a, weight, out)
    _rows_contiguous(a, "a")
    _rows_contiguous(weight, "weight")
    _rows_contiguous(out, "out")
    N, K = weight.shape
    if a.shape[1] != K or out.shape[1] != N or n_rows > min(a.shape[0], out.shape[0]):
        raise KernelError(f"linear: a {tuple(a.shape)} x weight {tuple(weight.shape)} -> out {tuple(out.shape)} "
                          f"for {n_rows} rows does not fit")
    _check(core().rs_linear_simt(_ptr(a), dtype_code(a), a.stride(0), _ptr(weight), dtype_code(weight),
                                 weight.stride(0), _ptr(out), dtype_code(out), out.stride(0), n_rows, N, K,
                                 1 if accumulate else 0, _stream()), "linear_simt")


_bf16 = None


def bf16lib():
    global _bf16
    if _bf16 is None:
        lib = load_library("bf16")
        lib.rs_gemm_bf16_tc.argtypes = [c_void_p, c_long, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_void_p, c_void_p]
        lib.rs_skinny_gemm_bf16.argtypes = [c_void_p, c_long, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                            c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.rs_skinny_gemm_workspace_floats.restype = c_long
        lib.rs_skinny_finish.argtypes = [c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.rs_skinny_finish_rmsnorm_supported.argtypes = [c_void_p, c_long, c_int, c_void_p, c_void_p, c_long]
        lib.rs_skinny_finish_rmsnorm.argtypes = [c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                                 c_float, c_void_p, c_long, c_void_p]
        lib.rs_decode_chain.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.rs_mid_gemm_bf16.argtypes = [c_void_p, c_long, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                         c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.rs_mid_finish.argtypes = lib.rs_skinny_finish.argtypes
        lib.rs_mid_finish_rmsnorm.argtypes = lib.rs_skinny_finish_rmsnorm.argtypes
        lib.rs_mid_gemm_workspace_floats.restype = c_long
        lib.rs_attention_decode_bf16.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                                 c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                 c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_void_p, c_int, c_void_p, c_void_p]
        lib.rs_attention_decode_build_items.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.rs_attention_decode_bf16_supported.argtypes = [c_int, c_int, c_int, c_int]
        lib.rs_attention_prefill_bf16.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                                  c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                  c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p]
        lib.rs_attention_prefill_tc.argtypes = [c_void_p, c_long, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                                c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                c_int, c_float, c_void_p, c_int, c_void_p, c_void_p]
        lib.rs_attention_prefill_tc_supported.argtypes = [c_int, c_int, c_int, c_int]
        lib.rs_attention_prefill_tc_q_per_cta.argtypes = [c_int, c_int]
        lib.rs_grouped_gemm_mma.argtypes = [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_void_p, c_int, c_long, c_void_p,
                                            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.rs_grouped_gemm_mma_rows_per_tile.argtypes = [c_int]
        lib.rs_block_linear_mma.argtypes = [c_void_p, c_int, c_long, c_long, c_void_p, c_void_p, c_int, c_void_p, c_int, c_long,
                                            c_long, c_int, c_int, c_int, c_int, c_void_p]
        lib.rs_attention_latent_supported.argtypes = [c_int, c_int, c_int]
        lib.rs_attention_latent_q_per_cta.argtypes = [c_int]
        lib.rs_attention_latent_bf16.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_void_p,
                                                 c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                                 c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.rs_attention_prefill_bf16_supported.argtypes = [c_int, c_int, c_int]
        lib.rs_attention_prefill_bf16_q_per_cta.argtypes = [c_int, c_int]
        _bf16 = lib
    return _bf16


EPI_STORE_BF16, EPI_STORE_F32, EPI_ADD_F32, EPI_SWIGLU_BF16, EPI_GEGLU_BF16 = 0, 1, 2, 3, 4


def tensor_core_shape_ok(a: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the bfloat16 tensor-core kernels take this product: both operands bfloat16, every row
    16-byte aligned (K and the row pitches multiples of 8 elements, base pointers multiples of 16)."""
    if a.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return False
    K = weight.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


def _epilogue_code(out: torch.Tensor, accumulate: bool, swiglu) -> int:
    """``swiglu``: False, or which gated epilogue: True or "silu" for SiLU(gate) * up, "gelu_tanh" for the tanh form of GELU."""
    if swiglu:
        if out.dtype != torch.bfloat16 or accumulate:
            raise KernelError("the fused act(gate)*up epilogue writes bfloat16 and does not accumulate")
        return EPI_GEGLU_BF16 if swiglu == "gelu_tanh" else EPI_SWIGLU_BF16
    if out.dtype == torch.bfloat16:
        if accumulate:
            raise KernelError("accumulating products go into the float32 residual stream")
        return EPI_STORE_BF16
    if out.dtype == torch.float32:
        return EPI_ADD_F32 if accumulate else EPI_STORE_F32
    raise KernelError(f"unsupported output element type {out.dtype}")


def _check_product(a, weight, out, n_rows, swiglu):
    _cuda(a, weight, out)
    _rows_contiguous(a, "a")
    _rows_contiguous(weight, "weight")
    _rows_contiguous(out, "out")
    N, K = weight.shape
    n_out = N // 2 if swiglu else N
    if a.shape[1] != K or out.shape[1] != n_out or n_rows > min(a.shape[0], out.shape[0]) or (swiglu and N % 2):
        raise KernelError(f"linear: a {tuple(a.shape)} x weight {tuple(weight.shape)} -> out {tuple(out.shape)} "
                          f"for {n_rows} rows does not fit")
    return N, K


def gemm_bf16_tc(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False,
                 swiglu: bool = False, status: Optional[torch.Tensor] = None, bn: int = 0, max_ctas: int = 0) -> None:
    """out[:n_rows] (=|+=) a[:n_rows] @ weight.T on the tcgen05 tensor cores (csrc/gemm_tcgen05.cu).
    ``swiglu``: weight rows alternate gate, up and out[:, j] = silu(gate_j) * up_j."""
    N, K = _check_product(a, weight, out, n_rows, swiglu)
    if not tensor_core_shape_ok(a, weight):
        raise KernelError(f"gemm_bf16_tc refuses a {tuple(a.shape)} {a.dtype} stride {a.stride(0)} x weight "
                          f"{tuple(weight.shape)} {weight.dtype}: rows must be bfloat16 and 16-byte aligned")
    if status is None:
        status = _default_status(a.device)
    _check(bf16lib().rs_gemm_bf16_tc(_ptr(a), a.stride(0), a.shape[0], _ptr(weight), weight.stride(0), _ptr(out),
                                     out.stride(0), n_rows, N, K, _epilogue_code(out, accumulate, swiglu), bn, max_ctas,
                                     _ptr(status), _stream()), "gemm_bf16_tc")


SKINNY_MAX_ROWS = 64     # what the kernel takes
SKINNY_MAX_WEIGHT = 1 << 28   # weights of this many elements or more (an output head) stream faster through the tcgen05 kernel
SKINNY_ROWS = 8          # up to here the engine prefers it; from 9 rows the stream-K tcgen05 kernel is as fast or faster
_SKINNY_SCRATCH = {}


def _skinny_scratch(device):
    """Workspace of the skinny product (partials of shared row tiles), one per device, made at the first call
    (before any graph capture: the engine runs every shape once eagerly first)."""
    ws = _SKINNY_SCRATCH.get(device)
    if ws is None:
        ws = _SKINNY_SCRATCH[device] = torch.empty(int(bf16lib().rs_skinny_gemm_workspace_floats()), dtype=torch.float32,
                                                   device=device)
    return ws


class PendingSum:
    """A product into the float32 residual stream whose last step is still owed: the partial sums of the weight tiles
    that several CTAs shared lie in the product's workspace and have not been added to ``out`` yet.  Whoever reads
    ``out`` next either takes the object along (``rmsnorm(..., pending=...)`` adds the partials while it reads the
    rows) or calls :meth:`finish` first.  No other product of the same kind may run in between: it would overwrite the
    workspace.  ``kind``: "skinny" (up to 8 rows) or "mid" (the stream-K tcgen05 product, up to 128 rows)."""

    def __init__(self, kind: str, out: torch.Tensor, n_rows: int, N: int, K: int, workspace: torch.Tensor, max_ctas: int):
        self.kind, self.out, self.n_rows, self.N, self.K = kind, out, n_rows, N, K
        self.workspace, self.max_ctas = workspace, max_ctas
        self.done = False

    def finish(self) -> None:
        """out += the partial sums (the small kernel that the product would have launched itself)."""
        if not self.done:
            self.done = True
            fn = bf16lib().rs_skinny_finish if self.kind == "skinny" else bf16lib().rs_mid_finish
            _check(fn(_ptr(self.out), self.out.stride(0), self.n_rows, self.N, self.K, _ptr(self.workspace), self.max_ctas,
                      _stream()), self.kind + "_finish")

    def finish_with_rmsnorm(self, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        """The same and out[r] = RMSNorm(self.out[r]) * weight, in one kernel."""
        self.done = True
        fn = bf16lib().rs_skinny_finish_rmsnorm if self.kind == "skinny" else bf16lib().rs_mid_finish_rmsnorm
        _check(fn(_ptr(self.out), self.out.stride(0), self.n_rows, self.N, self.K, _ptr(self.workspace), self.max_ctas,
                  _ptr(weight), dtype_code(weight), float(eps), _ptr(out), out.stride(0), _stream()),
               self.kind + "_finish_rmsnorm")


SKINNY_DEFER_ROWS = 8    # the deferred form exists for the thread layout of up to 8 rows
DEFER_SUMS = True        # whether linear() lets a product leave its last sum to the next reader when the caller allows it


def skinny_gemm_bf16(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False,
                     swiglu: bool = False, status: Optional[torch.Tensor] = None, max_ctas: int = 0,
                     defer: bool = False) -> Optional[PendingSum]:
    """out[:n_rows] (=|+=) a[:n_rows] @ weight.T for n_rows <= 64: persistent CTAs stream the weight through a
    TMA-fed ring of shared-memory stages (csrc/skinny_gemm_tma.cu).  With ``defer`` (float32 +=, up to 8 rows) the
    kernel that adds up the shared tiles is not launched and a :class:`PendingSum` is returned instead."""
    N, K = _check_product(a, weight, out, n_rows, swiglu)
    if defer and not (accumulate and out.dtype == torch.float32 and n_rows <= SKINNY_DEFER_ROWS):
        raise KernelError("skinny_gemm_bf16 defers only a float32 += of up to 8 rows")
    if n_rows > SKINNY_MAX_ROWS or not tensor_core_shape_ok(a, weight) or N <= 0:
        raise KernelError(f"skinny_gemm_bf16 refuses {n_rows} rows of a {tuple(a.shape)} {a.dtype} x weight "
                          f"{tuple(weight.shape)} {weight.dtype}: at most {SKINNY_MAX_ROWS} rows, bfloat16, 16-byte aligned")
    if status is None:
        status = _default_status(a.device)
    ws = _skinny_scratch(a.device)
    _check(bf16lib().rs_skinny_gemm_bf16(_ptr(a), a.stride(0), a.shape[0], _ptr(weight), weight.stride(0), _ptr(out),
                                         out.stride(0), n_rows, N, K, _epilogue_code(out, accumulate, swiglu), _ptr(ws),
                                         max_ctas, 1 if defer else 0, _ptr(status), _stream()), "skinny_gemm_bf16", 1 if defer else 2)
    return PendingSum("skinny", out, n_rows, N, K, ws, max_ctas) if defer else None


MID_MAX_ROWS = 128       # what the stream-K tcgen05 kernel takes; the engine uses it from SKINNY_ROWS + 1 rows up to here
_MID_SCRATCH = {}


def _mid_scratch(device):
    """Workspace of the stream-K tcgen05 product, one per device, made at the first call."""
    ws = _MID_SCRATCH.get(device)
    if ws is None:
        ws = _MID_SCRATCH[device] = torch.empty(int(bf16lib().rs_mid_gemm_workspace_floats()), dtype=torch.float32,
                                                device=device)
    return ws


def mid_gemm_bf16(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False,
                  swiglu: bool = False, status: Optional[torch.Tensor] = None, max_ctas: int = 0,
                  defer: bool = False) -> Optional[PendingSum]:
    """out[:n_rows] (=|+=) a[:n_rows] @ weight.T for n_rows <= 128 on the tensor cores with the operands swapped
    (rows of the weight fill the 128-row side of the MMA) and the work dealt to the SMs in equal shares of k
    (csrc/mid_gemm_tcgen05.cu).  With ``defer`` (float32 += only) the kernel that adds up the shared tiles is not
    launched and a :class:`PendingSum` is returned instead."""
    N, K = _check_product(a, weight, out, n_rows, swiglu)
    if defer and not (accumulate and out.dtype == torch.float32):
        raise KernelError("mid_gemm_bf16 defers only a float32 +=")
    if n_rows > MID_MAX_ROWS or not tensor_core_shape_ok(a, weight):
        raise KernelError(f"mid_gemm_bf16 refuses {n_rows} rows of a {tuple(a.shape)} {a.dtype} x weight "
                          f"{tuple(weight.shape)} {weight.dtype}: at most {MID_MAX_ROWS} rows, bfloat16, 16-byte aligned")
    if status is None:
        status = _default_status(a.device)
    ws = _mid_scratch(a.device)
    _check(bf16lib().rs_mid_gemm_bf16(_ptr(a), a.stride(0), a.shape[0], _ptr(weight), weight.stride(0), _ptr(out),
                                      out.stride(0), n_rows, N, K, _epilogue_code(out, accumulate, swiglu), _ptr(ws),
                                      max_ctas, 1 if defer else 0, _ptr(status), _stream()), "mid_gemm_bf16",
           1 if defer else 2)
    return PendingSum("mid", out, n_rows, N, K, ws, max_ctas) if defer else None


_STATUS = {}


def _default_status(device) -> torch.Tensor:
    t = _STATUS.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[device] = t
    return t


# ----------------------------------------------------------------------------- a chain of decode products in one kernel
class RsChainOp(ctypes.Structure):
    """One operation of a chain, as csrc/decode_chain.cu takes it."""
    _fields_ = [("type", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("epi", c_int), ("owed", c_int), ("w_dt", c_int),
                ("reserved", c_int), ("lda", c_long), ("a_rows", c_long), ("ldw", c_long), ("ldc", c_long), ("out_stride", c_long),
                ("A", c_void_p), ("W", c_void_p), ("C", c_void_p), ("w", c_void_p), ("out", c_void_p), ("eps", c_float),
                ("reserved2", c_int)]


CHAIN_GEMV, CHAIN_REDUCE, CHAIN_ROWNORM = 0, 1, 2
CHAIN_DECODE = False     # whether the engine chains the products of a decode step of up to 8 tokens (begin_chain); measured
                         # slower than the separate kernels under programmatic dependent launch, so it is off
_CHAIN_BUFFERS = {}


class _Chain:
    """The products of up to 8 rows, and the row norms between them, that have been asked for since the last kernel of
    another kind: they wait here and leave as ONE persistent kernel (csrc/decode_chain.cu) when anything else is about
    to be launched, so that the weights of a whole run of dependent products stream without a kernel boundary."""

    def __init__(self, status: torch.Tensor):
        self.status = status
        self.ops = []            # RsChainOp
        self.keep = []           # the tensors the operations point into
        self.n_products = 0
        self.open_product = None   # the last op, if it is a product whose shared tiles nobody has been told to finish
        self.launches = 0

    def _room(self, n_ops: int, n_products: int = 0) -> None:
        lib = bf16lib()
        if (len(self.ops) + n_ops > lib.rs_decode_chain_max_ops()
                or self.n_products + n_products > lib.rs_decode_chain_max_products()):
            self.flush()

    def _close_product(self) -> None:
        """The product recorded last leaves its shared tiles to a REDUCE operation (nobody else took them)."""
        g = self.open_product
        if g is not None:
            self.open_product = None
            r = RsChainOp.from_buffer_copy(g)
            r.type = CHAIN_REDUCE
            self.ops.append(r)

    def add_product(self, a, weight, out, n_rows, epi) -> None:
        self._close_product()
        self._room(2, 1)
        N, K = weight.shape
        op = RsChainOp(type=CHAIN_GEMV, M=n_rows, N=N, K=K, epi=epi, lda=a.stride(0), a_rows=a.shape[0], ldw=weight.stride(0),
                       ldc=out.stride(0), A=a.data_ptr(), W=weight.data_ptr(), C=out.data_ptr())
        self.ops.append(op)
        self.keep += [a, weight, out]
        self.n_products += 1
        self.open_product = op

    def add_rmsnorm(self, x, weight, eps, out, n_rows) -> None:
        g = self.open_product
        owed = (g is not None and g.epi == EPI_ADD_F32 and g.C == x.data_ptr() and g.ldc == x.stride(0) and g.M == n_rows
                and g.N == x.shape[1])
        if owed:
            self.open_product = None                 # the norm adds the product's partial sums while it reads the rows
        else:
            self._close_product()
        self._room(1)
        self.ops.append(RsChainOp(type=CHAIN_ROWNORM, M=n_rows, N=x.shape[1], K=g.K if owed else 1, owed=1 if owed else 0,
                                  w_dt=dtype_code(weight), ldc=x.stride(0), out_stride=out.stride(0), C=x.data_ptr(),
                                  w=weight.data_ptr(), out=out.data_ptr(), eps=float(eps)))
        self.keep += [x, weight, out]

    def flush(self) -> None:
        if not self.ops:
            return
        self._close_product()
        ops, self.ops, keep, self.keep = self.ops, [], self.keep, []
        self.n_products = 0
        arr = (RsChainOp * len(ops))(*ops)
        dev = self.status.device
        bufs = _CHAIN_BUFFERS.get(dev)
        if bufs is None:
            bufs = _CHAIN_BUFFERS[dev] = torch.zeros(2, dtype=torch.int32, device=dev)
        ws = _skinny_scratch(dev)
        global _FLUSHING
        _FLUSHING = True
        try:
            stream = c_void_p(torch.cuda.current_stream().cuda_stream)
            _check(bf16lib().rs_decode_chain(ctypes.cast(arr, c_void_p), len(ops), _ptr(ws), _ptr(bufs), _ptr(self.status), stream),
                   "decode_chain")
        finally:
            _FLUSHING = False
        self.launches += 1
        del keep


_ACTIVE_CHAIN: Optional[_Chain] = None
_FLUSHING = False


def chain_max_rows() -> int:
    return int(bf16lib().rs_decode_chain_max_rows())


def begin_chain(status: torch.Tensor) -> None:
    """From here to :func:`end_chain`, products of up to 8 bfloat16 rows (``linear``, ``linear_swiglu``) and the row
    norms between them are recorded instead of launched, and leave as one kernel when any other kernel of this module is
    asked for or the chain is ended.  Only for callers that touch the tensors involved through this module alone in
    between (torch operations on them would not see the recorded work)."""
    global _ACTIVE_CHAIN
    if _ACTIVE_CHAIN is not None:
        raise KernelError("a chain of decode products is already being recorded")
    _ACTIVE_CHAIN = _Chain(status)


def end_chain() -> int:
    """Launches what is recorded and stops recording; returns the number of chain kernels launched since begin_chain."""
    global _ACTIVE_CHAIN
    ch, _ACTIVE_CHAIN = _ACTIVE_CHAIN, None
    if ch is None:
        return 0
    ch.flush()
    return ch.launches


def flush_chain() -> None:
    if _ACTIVE_CHAIN is not None and not _FLUSHING:
        _ACTIVE_CHAIN.flush()


def reset_chain_barrier() -> None:
    """After a chain kernel gave up on a wait its arrival counter may be left mid-count: set it back."""
    for t in _CHAIN_BUFFERS.values():
        t.zero_()


def _chain_takes_product(a, weight, out, n_rows, swiglu: bool) -> bool:
    if _ACTIVE_CHAIN is None:            # asked first: the 32-bit engine must not load (or compile) the bfloat16 library
        return False
    if swiglu == "gelu_tanh":            # the chained kernel has the SiLU gate only
        return False
    lib = bf16lib()
    return (n_rows <= lib.rs_decode_chain_max_rows() and tensor_core_shape_ok(a, weight)
            and weight.numel() < SKINNY_MAX_WEIGHT and out.dtype in (torch.bfloat16, torch.float32)
            and a.is_cuda and weight.is_cuda and out.is_cuda)


def linear(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False,
           status: Optional[torch.Tensor] = None, may_defer: bool = False) -> Optional[PendingSum]:
    """The engine's matrix product: the tensor-core kernels for bfloat16 operands whose rows are 16-byte
    aligned (skinny kernel up to 8 rows, stream-K tcgen05 kernel up to 128, tiled tcgen05 kernel above), the
    CUDA-core kernel for everything else
    (the 32-bit engine, float32-stored weights, odd widths).  ``may_defer``: the caller hands a :class:`PendingSum`
    on to the next reader of ``out`` if the kernel that runs can leave one (else None comes back and ``out`` is whole)."""
    if _chain_takes_product(a, weight, out, n_rows, False):
        _check_product(a, weight, out, n_rows, False)
        _ACTIVE_CHAIN.add_product(a, weight, out, n_rows, _epilogue_code(out, accumulate, False))
        return None
    if tensor_core_shape_ok(a, weight) and out.dtype in (torch.bfloat16, torch.float32):
        if n_rows <= SKINNY_ROWS and weight.numel() < SKINNY_MAX_WEIGHT:
            defer = may_defer and DEFER_SUMS and accumulate and out.dtype == torch.float32 and n_rows <= SKINNY_DEFER_ROWS
            return skinny_gemm_bf16(a, weight, out, n_rows, accumulate, status=status, defer=defer)
        elif n_rows <= MID_MAX_ROWS:
            return mid_gemm_bf16(a, weight, out, n_rows, accumulate, status=status,
                                 defer=may_defer and DEFER_SUMS and accumulate and out.dtype == torch.float32)
        else:
            gemm_bf16_tc(a, weight, out, n_rows, accumulate, status=status)
    else:
        linear_simt(a, weight, out, n_rows, accumulate)


def linear_swiglu(a: torch.Tensor, weight_interleaved: torch.Tensor, out: torch.Tensor, n_rows: int,
                  status: Optional[torch.Tensor] = None, activation: str = "silu") -> None:
    """out[:, j] = act(a @ w[2j]) * (a @ w[2j+1]) in one kernel, act SiLU or ("gelu_tanh") the tanh form of GELU; only for
    shapes ``tensor_core_shape_ok`` takes."""
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"linear_swiglu: unknown activation '{activation}' (known: {', '.join(sorted(GATE_ACTIVATIONS))})")
    if _chain_takes_product(a, weight_interleaved, out, n_rows, activation):
        _check_product(a, weight_interleaved, out, n_rows, True)
        _ACTIVE_CHAIN.add_product(a, weight_interleaved, out, n_rows, _epilogue_code(out, False, True))
        return
    if n_rows <= SKINNY_ROWS:
        skinny_gemm_bf16(a, weight_interleaved, out, n_rows, swiglu=activation, status=status)
    elif n_rows <= MID_MAX_ROWS:
        mid_gemm_bf16(a, weight_interleaved, out, n_rows, swiglu=activation, status=status)
    else:
        gemm_bf16_tc(a, weight_interleaved, out, n_rows, swiglu=activation, status=status)


# ----------------------------------------------------------------------------- attention
def attention_q_per_cta(n_q: int, n_kv: int) -> int:
    return int(core().rs_attention_simt_q_per_cta(n_q, n_kv))


def attention_partial_floats(total_splits: int, n_q: int, head_dim: int) -> int:
    return int(core().rs_attention_simt_partial_floats(total_splits, n_q, head_dim))


def attention_simt(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                   q_start: torch.Tensor, kv_len: torch.Tensor, work: torch.Tensor, n_work: int, n_q: int, n_kv: int,
                   head_dim: int, page_size: int, window: int, scale: float, decode: bool, status: torch.Tensor,
                   split_keys: int = 128, max_splits: int = 1, split_start: Optional[torch.Tensor] = None,
                   total_splits: int = 0, partial: Optional[torch.Tensor] = None,
                   slopes: Optional[torch.Tensor] = None, one_plane: bool = False,
                   dist_bias: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention (see csrc/attention_simt.cu).  q/out: [T, >= n_q*head_dim] views.

    ``one_plane``: the cache is [pages, 1, n_kv, page_size, head_dim] and a row is key and value at once (a latent
    shared by both); else [pages, 2, ...] with keys in plane 0 and values in plane 1.

    ``slopes``: float32 [n_q] or None: slopes[h] * (key position - query position) is added to every scaled score of
    head h (a position encoding that biases scores by distance instead of rotating q and k).

    ``dist_bias``: float32 [n_dist, n_q] or None: row min(query position - key position, n_dist - 1) is added to the
    scaled scores, one value per head (a bias tabulated by distance; the last row serves every longer distance).

    Decode form: ``partial`` is the workspace of un-normalised partial results, one slot of n_q * (head_dim + 2)
    float32 values per (sequence, split); ``split_start[w]`` is the first slot of sequence w and ``total_splits`` the
    slots the caller knows the step uses (0 when it cannot say, as for a captured step whose lengths change from
    replay to replay).  The kernels are told how many slots the workspace holds and flag a slot beyond it
    (STATUS_BAD_PLAN) instead of writing there."""
    _cuda(q, out, cache, block_table, q_start, kv_len, work, status, partial, split_start)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and cache must share an element type")
    planes = 1 if one_plane else 2
    if tuple(cache.shape[1:]) != (planes, n_kv, page_size, head_dim) or not cache.is_contiguous():
        raise KernelError(f"attention: cache shape {tuple(cache.shape)} is not [pages, {planes}, {n_kv}, {page_size}, {head_dim}]")
    if head_dim % 16 or head_dim > 576:
        raise KernelError(f"attention: head size {head_dim} is not a multiple of 16 up to 576")
    if n_q % n_kv:
        raise KernelError(f"attention: {n_q} query heads are not a multiple of {n_kv} key/value heads")
    for name, t in (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len), ("work", work)):
        if t.dtype != torch.int32:
            raise KernelError(f"attention: {name} must be int32")
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.numel() != n_q or not slopes.is_contiguous() or not slopes.is_cuda):
        raise KernelError(f"attention: slopes must be contiguous float32 [{n_q}] on the device")
    if dist_bias is not None and (dist_bias.dtype != torch.float32 or dist_bias.dim() != 2 or dist_bias.shape[1] != n_q
                                  or dist_bias.shape[0] < 1 or not dist_bias.is_contiguous() or not dist_bias.is_cuda):
        raise KernelError(f"attention: dist_bias must be contiguous float32 [distances, {n_q}] on the device")
    slots = 0
    if decode:
        if split_start is None or split_start.dtype != torch.int32:
            raise KernelError("attention: the decode form needs int32 split_start")
        slots = _partial_slots(partial, total_splits, n_q, head_dim, "attention")
    _check(core().rs_attention_simt(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), dtype_code(q), _ptr(cache), cache.stride(0), cache.shape[0],
        page_size, _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, n_q,
        n_kv, head_dim, int(window), float(scale), 1 if decode else 0, split_keys, max_splits, _ptr(split_start),
        _ptr(partial), slots, _ptr(slopes), _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0],
        1 if one_plane else 0, _ptr(status), _stream()), "attention_simt", 2 if decode else 1)


def _partial_slots(partial: Optional[torch.Tensor], total_splits: int, n_q: int, head_dim: int, who: str) -> int:
    """Slots of partial results the workspace holds; raises if the step is known to need more."""
    if partial is None or partial.dtype != torch.float32 or not partial.is_contiguous():
        raise KernelError(f"{who}: the decode form needs a contiguous float32 workspace of partial results")
    slots = min(partial.numel() // (n_q * (head_dim + 2)), 0x7FFFFFFF)
    if slots < max(1, total_splits):
        raise KernelError(f"{who}: the step's {max(1, total_splits)} (sequence, split) pairs need "
                          f"{attention_partial_floats(max(1, total_splits), n_q, head_dim)} float32 values of partial "
                          f"workspace, {partial.numel()} were given")
    return int(slots)


def attention_prefill_kernel(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int, page_size: int, force: str = "") -> str:
    """Which kernel ``attention_prefill`` runs for this shape: "tc" (tcgen05, head 64/128, page size a power of
    two from 8 to 128), "mma" (mma.sync, head 32/64/96/128) or "simt" (everything else, and float32).  ``force``
    names one; "biased" asks for the fastest kernel that adds a bias tabulated by distance (all three do; "biased_mma"
    leaves the tcgen05 kernel out)."""
    if force in ("biased", "biased_mma"):
        if dtype == torch.bfloat16:
            if force == "biased" and bf16lib().rs_attention_prefill_tc_supported(n_q, n_kv, head_dim, page_size):
                return "tc"
            if bf16lib().rs_attention_prefill_bf16_supported(n_q, n_kv, head_dim):
                return "mma"
        return "simt"
    if force:
        return force
    if dtype == torch.bfloat16:
        if bf16lib().rs_attention_prefill_tc_supported(n_q, n_kv, head_dim, page_size):
            return "tc"
        if bf16lib().rs_attention_prefill_bf16_supported(n_q, n_kv, head_dim):
            return "mma"
    return "simt"


def attention_prefill_fast_ok(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int) -> bool:
    """Whether a tensor-core portion kernel takes this shape (bfloat16, head size 32/64/96/128)."""
    return dtype == torch.bfloat16 and bool(bf16lib().rs_attention_prefill_bf16_supported(n_q, n_kv, head_dim))


def attention_prefill_q_per_cta(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int, page_size: int = 16,
                                force: str = "") -> int:
    """Query tokens per work item of the portion form, for the kernel ``attention_prefill`` will pick."""
    kind = attention_prefill_kernel(dtype, n_q, n_kv, head_dim, page_size, force)
    if kind == "tc":
        return int(bf16lib().rs_attention_prefill_tc_q_per_cta(n_q, n_kv))
    if kind == "mma":
        return int(bf16lib().rs_attention_prefill_bf16_q_per_cta(n_q, n_kv))
    return attention_q_per_cta(n_q, n_kv)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      q_start: torch.Tensor, kv_len: torch.Tensor, work: torch.Tensor, n_work: int, n_q: int, n_kv: int,
                      head_dim: int, page_size: int, window: int, scale: float, status: torch.Tensor,
                      force: str = "", slopes: Optional[torch.Tensor] = None, one_plane: bool = False,
                      dist_bias: Optional[torch.Tensor] = None, dist_bias_by_head: Optional[torch.Tensor] = None) -> None:
    """Attention of prompt portions; ``work`` lists (sequence, first query) tiles of ``attention_prefill_q_per_cta``
    tokens.  tcgen05 kernel (csrc/attention_prefill_tc.cu), mma.sync kernel (csrc/attention_prefill_mma.cu) or
    CUDA cores, whichever takes the shape; ``force`` names one.  Score slopes are the CUDA-core kernel's; a bias
    tabulated by distance (``dist_bias`` [distances, heads], see :func:`attention_simt`) is added by all three, the
    tcgen05 kernel reading its transpose ``dist_bias_by_head`` [heads, distances] (and wanting a positive scale)."""
    kind = attention_prefill_kernel(q.dtype, n_q, n_kv, head_dim, page_size, force)
    if (slopes is not None or one_plane) and kind != "simt":
        raise KernelError("attention_prefill: only the CUDA-core kernel (force='simt') adds score slopes or reads a "
                          "one-plane cache")
    if dist_bias is not None and kind == "tc":
        if dist_bias_by_head is None or dist_bias_by_head.dtype != torch.float32 or not dist_bias_by_head.is_contiguous() \
                or tuple(dist_bias_by_head.shape) != (n_q, dist_bias.shape[0]) or not dist_bias_by_head.is_cuda or scale <= 0:
            raise KernelError(f"attention_prefill: the tcgen05 kernel reads the bias as contiguous float32 [{n_q}, distances] "
                              f"and wants a positive scale")
    if kind == "simt":
        attention_simt(q, out, cache, block_table, q_start, kv_len, work, n_work, n_q, n_kv, head_dim, page_size, window,
                       scale, False, status, slopes=slopes, one_plane=one_plane, dist_bias=dist_bias)
        return
    _cuda(q, out, cache, block_table, q_start, kv_len, work, status)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or q.dtype != torch.bfloat16 or not cache.is_contiguous():
        raise KernelError("attention_prefill: q, out and cache must be bfloat16 and the cache contiguous")
    if tuple(cache.shape[1:]) != (2, n_kv, page_size, head_dim):
        raise KernelError(f"attention_prefill: cache shape {tuple(cache.shape)} is not [pages, 2, {n_kv}, {page_size}, {head_dim}]")
    for name, t in (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len), ("work", work)):
        if t.dtype != torch.int32:
            raise KernelError(f"attention_prefill: {name} must be int32")
    if kind == "tc":
        fn = bf16lib().rs_attention_prefill_tc
        _check(fn(
            _ptr(q), q.stride(0), min(q.shape[0], out.shape[0]), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), cache.shape[0],
            page_size, _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, n_q, n_kv,
            head_dim, int(window), float(scale), _ptr(dist_bias_by_head if dist_bias is not None else None),
            0 if dist_bias is None else dist_bias.shape[0], _ptr(status), _stream()), "attention_prefill_" + kind)
        return
    _check(bf16lib().rs_attention_prefill_bf16(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), cache.shape[0], page_size,
        _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, n_q, n_kv, head_dim,
        int(window), float(scale), _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0], _ptr(status), _stream()),
        "attention_prefill_bf16")


def attention_decode_fast_ok(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int, page_size: int = 16) -> bool:
    """Whether the tensor-core decode kernel takes this shape (bfloat16, head size 64 or 128, group <= 16, pages of
    8 to 128 tokens, a power of two)."""
    return dtype == torch.bfloat16 and bool(
        bf16lib().rs_attention_decode_bf16_supported(n_q, n_kv, head_dim, page_size))


def attention_decode_loads_per_page() -> int:
    """TMA loads the tensor-core decode kernel issued per page of an item in its most recent launch: 1 when the
    driver took the 5-d map of the cache, else one per K/V and 64-wide half of the head."""
    return int(bf16lib().rs_attention_decode_bf16_loads_per_page())


def attention_decode(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     q_start: torch.Tensor, kv_len: torch.Tensor, work: torch.Tensor, n_work: int, n_q: int, n_kv: int,
                     head_dim: int, page_size: int, window: int, scale: float, status: torch.Tensor, split_keys: int,
                     max_splits: int, split_start: torch.Tensor, total_splits: int, partial: torch.Tensor,
                     force_simt: bool = False, slopes: Optional[torch.Tensor] = None,
                     items: Optional[torch.Tensor] = None, one_plane: bool = False,
                     dist_bias: Optional[torch.Tensor] = None) -> None:
    """Attention of sequences with one query token each: the tensor-core kernel (csrc/attention_decode_mma.cu)
    where it takes the shape, else the CUDA-core kernel's split form (always, when score biases are given).  Same
    partial-workspace layout.  ``items``: the step's list of live (sequence, kv head, split) items from
    :func:`attention_decode_items`, which a caller with several layers builds once per step; built here if not given."""
    if (force_simt or slopes is not None or one_plane
            or not attention_decode_fast_ok(q.dtype, n_q, n_kv, head_dim, page_size)):
        attention_simt(q, out, cache, block_table, q_start, kv_len, work, n_work, n_q, n_kv, head_dim, page_size, window,
                       scale, True, status, split_keys=split_keys, max_splits=max_splits, split_start=split_start,
                       total_splits=total_splits, partial=partial, slopes=slopes, one_plane=one_plane, dist_bias=dist_bias)
        return
    _cuda(q, out, cache, block_table, q_start, kv_len, work, status, partial, split_start)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or not cache.is_contiguous():
        raise KernelError("attention_decode: q, out and cache must be bfloat16 and the cache contiguous")
    if tuple(cache.shape[1:]) != (2, n_kv, page_size, head_dim):
        raise KernelError(f"attention_decode: cache shape {tuple(cache.shape)} is not [pages, 2, {n_kv}, {page_size}, {head_dim}]")
    for name, t in (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len), ("work", work),
                    ("split_start", split_start)):
        if t.dtype != torch.int32:
            raise KernelError(f"attention_decode: {name} must be int32")
    slots = _partial_slots(partial, total_splits, n_q, head_dim, "attention_decode")
    if items is None:
        items = torch.empty(n_work * n_kv * max_splits, dtype=torch.int32, device=q.device)
        attention_decode_items(split_start, n_work, n_kv, max_splits, items)
    elif items.dtype != torch.int32 or not items.is_cuda or not items.is_contiguous():
        raise KernelError("attention_decode: items must be a contiguous int32 device tensor")
    _check(bf16lib().rs_attention_decode_bf16(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), cache.shape[0], page_size,
        _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, n_q, n_kv, head_dim,
        int(window), float(scale), split_keys, max_splits, _ptr(split_start), _ptr(items), _ptr(partial), slots,
        _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0], _ptr(status), _stream()), "attention_decode_bf16", 2)


def attention_latent_ok(dtype: torch.dtype, n_heads: int, lat: int, page_size: int) -> bool:
    """Whether the tensor-core kernel of latent attention takes this shape (bfloat16, rows a multiple of 16 up to 576)."""
    return dtype == torch.bfloat16 and bool(bf16lib().rs_attention_latent_supported(n_heads, lat, page_size))


def attention_latent_q_per_cta(n_heads: int) -> int:
    """Query tokens per work item of the portion form of :func:`attention_latent`."""
    return int(bf16lib().rs_attention_latent_q_per_cta(n_heads))


def attention_latent(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     q_start: torch.Tensor, kv_len: torch.Tensor, work: torch.Tensor, n_work: int, n_heads: int, lat: int,
                     page_size: int, window: int, scale: float, decode: bool, status: torch.Tensor, split_keys: int = 128,
                     max_splits: int = 1, split_start: Optional[torch.Tensor] = None, total_splits: int = 0,
                     partial: Optional[torch.Tensor] = None, split_weights: bool = False) -> None:
    """Attention of ``n_heads`` query heads over a one-plane cache [pages, 1, 1, page_size, lat] whose rows are key and
    value at once, on the tensor cores (csrc/attention_latent_mma.cu).  ``work``: (sequence, first query) tiles of
    :func:`attention_latent_q_per_cta` tokens, or with ``decode`` one sequence per entry, the keys cut into splits whose
    partial results (layout of :func:`attention_simt`) are merged by a second kernel.  ``split_weights``: the softmax weights
    enter the weighted sum in two bfloat16 terms (the float32 weight to 2^-17) instead of rounded to bfloat16."""
    _cuda(q, out, cache, block_table, q_start, kv_len, work, status, partial, split_start)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or not cache.is_contiguous():
        raise KernelError("attention_latent: q, out and cache must be bfloat16 and the cache contiguous")
    if tuple(cache.shape[1:]) != (1, 1, page_size, lat):
        raise KernelError(f"attention_latent: cache shape {tuple(cache.shape)} is not [pages, 1, 1, {page_size}, {lat}]")
    if q.shape[1] < n_heads * lat or out.shape[1] < n_heads * lat:
        raise KernelError("attention_latent: q and out must hold heads * lat columns")
    for name, t in (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len), ("work", work)):
        if t.dtype != torch.int32:
            raise KernelError(f"attention_latent: {name} must be int32")
    slots = 0
    if decode:
        if split_start is None or split_start.dtype != torch.int32:
            raise KernelError("attention_latent: the split form needs int32 split_start")
        slots = _partial_slots(partial, total_splits, n_heads, lat, "attention_latent")
    _check(bf16lib().rs_attention_latent_bf16(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), cache.shape[0], page_size,
        _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, n_heads, lat, int(window),
        float(scale), 1 if decode else 0, split_keys, max_splits, _ptr(split_start), _ptr(partial), slots,
        1 if split_weights else 0, _ptr(status), _stream()), "attention_latent", 2 if decode else 1)


def attention_decode_items(split_start: torch.Tensor, n_work: int, n_kv: int, max_splits: int, items: torch.Tensor) -> None:
    """items[id] for every live (sequence, kv head, split) of a step of single tokens, id as the tensor-core decode
    kernel counts them; ``items`` int32 with room for split_start[n_work] * n_kv entries (n_work * n_kv * max_splits
    always suffices).  One small kernel; its result serves every layer of the step."""
    _cuda(split_start, items)
    if split_start.dtype != torch.int32 or items.dtype != torch.int32 or not items.is_contiguous() or split_start.numel() < n_work + 1:
        raise KernelError("attention_decode_items: int32 tensors, split_start with n_work + 1 entries")
    _check(bf16lib().rs_attention_decode_build_items(_ptr(split_start), n_work, n_kv, max_splits, _ptr(items), _stream()),
           "attention_decode_items")


# ----------------------------------------------------------------------------- the bounded-wait probe
def wait_probe(status: torch.Tensor) -> dict:
    """Runs the probe kernel of csrc/wait_probe.cu (a wait nobody satisfies, limit 2 ms) with ``status`` as its status
    word and returns {"satisfied": bool, "waited_us": int, "limit_us": int} once it has ended.  For tests."""
    lib = load_library("probe")
    lib.rs_wait_probe.argtypes = [c_void_p, c_void_p, c_void_p]
    lib.rs_wait_probe_limit_ns.restype = ctypes.c_ulonglong
    _cuda(status)
    outcome = torch.full((2,), -1, dtype=torch.int32, device=status.device)
    _check(lib.rs_wait_probe(_ptr(status), _ptr(outcome), _stream()), "wait_probe")
    got = outcome.cpu().tolist()
    return {"satisfied": got[0] == 1, "waited_us": got[1], "limit_us": int(lib.rs_wait_probe_limit_ns() // 1000)}


# ----------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, n_rows: int, out: torch.Tensor, status: torch.Tensor,
           temps: Optional[torch.Tensor] = None, uniforms: Optional[torch.Tensor] = None) -> None:
    """out[r] = argmax of row r when temps is None or temps[r] <= 0, else a draw at temperature temps[r]."""
    _cuda(logits, out, status, temps, uniforms)
    _rows_contiguous(logits, "logits")
    if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() < n_rows:
        raise KernelError("sample: logits float32, out int32 with n_rows entries")
    if temps is not None and (uniforms is None or temps.dtype != torch.float32 or uniforms.dtype != torch.float32):
        raise KernelError("sample: temps and uniforms must both be float32")
    _check(core().rs_sample(_ptr(logits), logits.stride(0), n_rows, logits.shape[1], _ptr(temps), _ptr(uniforms),
                            _ptr(out), _ptr(status), _stream()), "sample")


# ----------------------------------------------------------------------------- parts with state, sandwich norms, experts
def _any_code(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else dtype_code(t)


def rmsnorm_add(x: torch.Tensor, delta: torch.Tensor, gain: torch.Tensor, eps: float, n_rows: int,
                then_weight: Optional[torch.Tensor] = None, then_eps: float = 0.0,
                out: Optional[torch.Tensor] = None) -> None:
    """x[r] += delta[r] * rsqrt(mean(delta[r]^2) + eps) * gain  (gain: one number or [n]); with ``out``, also
    out[r] = x[r] * rsqrt(mean(x[r]^2) + then_eps) * then_weight, the norm of the stream's next reader, in the same
    kernel.  x and delta float32 [*, n]."""
    _cuda(x, delta, gain, then_weight, out)
    _rows_contiguous(x, "rmsnorm_add x")
    _rows_contiguous(delta, "rmsnorm_add delta")
    n = x.shape[1]
    if x.dtype != torch.float32 or delta.dtype != torch.float32 or delta.shape[1] != n:
        raise KernelError("rmsnorm_add: the stream and the sublayer's output are float32 of one width")
    if gain.numel() not in (1, n) or not gain.is_contiguous():
        raise KernelError(f"rmsnorm_add: gain holds {gain.numel()} values, neither 1 nor {n}")
    if n_rows > min(x.shape[0], delta.shape[0]):
        raise KernelError("rmsnorm_add: more rows than the buffers hold")
    if out is not None:
        _rows_contiguous(out, "rmsnorm_add out")
        if then_weight is None or then_weight.numel() not in (1, n) or not then_weight.is_contiguous() or out.shape[1] != n \
                or n_rows > out.shape[0]:
            raise KernelError("rmsnorm_add: the following norm needs a weight of 1 or n values and an output of n columns")
    _check(core().rs_rmsnorm_add(_ptr(x), x.stride(0), _ptr(delta), delta.stride(0), _ptr(gain), dtype_code(gain),
                                 gain.numel(), float(eps), _ptr(then_weight if out is not None else None),
                                 _any_code(then_weight), 0 if then_weight is None else then_weight.numel(), float(then_eps),
                                 _ptr(out), _any_code(out), 0 if out is None else out.stride(0), n_rows, n, _stream()),
           "rmsnorm_add")


def concat_embed(x: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, row: Optional[torch.Tensor], cat: torch.Tensor,
                 n_tokens: int, status: torch.Tensor) -> None:
    """cat[t] = [x[t] | table[ids[t]]] in cat's element type, then x[t] = row (zeros when row is None)."""
    _cuda(x, table, ids, row, cat, status)
    _rows_contiguous(x, "concat_embed x")
    _rows_contiguous(cat, "concat_embed cat")
    n = x.shape[1]
    if x.dtype != torch.float32 or ids.dtype != torch.int32 or table.shape[1] != n or cat.shape[1] != 2 * n \
            or not table.is_contiguous() or n_tokens > min(x.shape[0], cat.shape[0], ids.numel()):
        raise KernelError("concat_embed: x float32 [T, n], table [V, n], cat [T, 2n], ids int32 [T]")
    if row is not None and (row.numel() != n or not row.is_contiguous()):
        raise KernelError("concat_embed: row must hold n values")
    _check(core().rs_concat_embed(_ptr(x), x.stride(0), _ptr(table), dtype_code(table), _ptr(ids), table.shape[0], _ptr(row),
                                  _any_code(row), _ptr(cat), dtype_code(cat), cat.stride(0), n_tokens, n, _ptr(status),
                                  _stream()), "concat_embed")


def short_conv(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, state: torch.Tensor, seq_of_token: torch.Tensor,
               q_start: torch.Tensor, slots: torch.Tensor, n_tokens: int, n_seqs: int, in_bias: Optional[torch.Tensor] = None,
               bias: Optional[torch.Tensor] = None, add_input: bool = False) -> None:
    """Causal convolution over time on each channel for the step's packed sequences (csrc/sequence_parts.cu).

    x [T, C]; weight [taps, C] (tap-major; the last row multiplies the current token); out [T, C], not x itself;
    state: float32 [slots, >= (taps - 1) * C] view whose rows hold each request's last taps - 1 inputs (updated)."""
    _cuda(x, weight, out, state, seq_of_token, q_start, slots, in_bias, bias)
    _rows_contiguous(x, "short_conv x")
    _rows_contiguous(out, "short_conv out")
    taps, C = weight.shape
    if x.shape[1] < C or out.shape[1] < C or not weight.is_contiguous() or n_tokens > min(x.shape[0], out.shape[0]):
        raise KernelError(f"short_conv: x {tuple(x.shape)} / out {tuple(out.shape)} do not fit {C} channels")
    if x.data_ptr() == out.data_ptr():
        raise KernelError("short_conv: out must not be x (later tokens read earlier inputs)")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < (taps - 1) * C:
        raise KernelError("short_conv: state must be float32 [slots, >= (taps - 1) * channels]")
    for name, t in (("seq_of_token", seq_of_token), ("q_start", q_start), ("slots", slots)):
        if t.dtype != torch.int32:
            raise KernelError(f"short_conv: {name} must be int32")
    for name, t in (("in_bias", in_bias), ("bias", bias)):
        if t is not None and (t.numel() != C or not t.is_contiguous()):
            raise KernelError(f"short_conv: {name} must hold one value per channel")
    _check(core().rs_short_conv(_ptr(x), dtype_code(x), x.stride(0), _ptr(in_bias), _any_code(in_bias), _ptr(weight),
                                dtype_code(weight), _ptr(bias), _any_code(bias), _ptr(out), dtype_code(out), out.stride(0),
                                _ptr(state), state.stride(0), _ptr(seq_of_token), _ptr(q_start), _ptr(slots), C, taps,
                                1 if add_input else 0, n_tokens, n_seqs, _stream()), "short_conv",
           2 if taps > 1 and n_tokens != n_seqs else 1)


BLOCK_LINEAR_ROWS_FORM = 8     # up to this many rows the CUDA-core kernel's row-streaming form runs (float32 inputs stay exact)


def block_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, in_block_stride: int,
                 out_block_stride: int, bias: Optional[torch.Tensor] = None) -> None:
    """out[t, b * out_block_stride + o] = bias[b, o] + sum_i weight[b, o, i] * x[t, b * in_block_stride + i]: one small
    matrix per block of channels (a block-diagonal product), float32 accumulation.  weight [B, O, I] contiguous."""
    _cuda(x, weight, out, bias)
    _rows_contiguous(x, "block_linear x")
    _rows_contiguous(out, "block_linear out")
    if weight.dim() != 3 or not weight.is_contiguous():
        raise KernelError("block_linear: weight must be contiguous [blocks, out, in]")
    B, O, I = weight.shape
    if (B - 1) * in_block_stride + I > x.shape[1] or (B - 1) * out_block_stride + O > out.shape[1] \
            or n_rows > min(x.shape[0], out.shape[0]):
        raise KernelError(f"block_linear: x {tuple(x.shape)} -> out {tuple(out.shape)} does not hold {B} blocks of "
                          f"{I} -> {O} at strides {in_block_stride}, {out_block_stride}")
    if bias is not None and (bias.numel() != B * O or not bias.is_contiguous()):
        raise KernelError("block_linear: bias must hold blocks * out values")
    per16 = 4 if x.dtype == torch.float32 else 8
    if (n_rows > BLOCK_LINEAR_ROWS_FORM and weight.dtype == torch.bfloat16 and x.dtype in (torch.bfloat16, torch.float32)
            and out.dtype in (torch.bfloat16, torch.float32) and I % 8 == 0 and in_block_stride % per16 == 0
            and x.stride(0) % per16 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0):
        # more than a few rows, bfloat16 weights: the tensor-core kernel of the grouped product, a block as an "expert"
        # that takes every row (float32 inputs are rounded to bfloat16 as they enter the product)
        _check(bf16lib().rs_block_linear_mma(_ptr(x), dtype_code(x), x.stride(0), in_block_stride, _ptr(weight), _ptr(bias),
                                             _any_code(bias), _ptr(out), dtype_code(out), out.stride(0), out_block_stride,
                                             n_rows, B, O, I, _stream()), "block_linear_mma")
        return
    _check(core().rs_block_linear(_ptr(x), dtype_code(x), x.stride(0), in_block_stride, _ptr(weight), dtype_code(weight),
                                  _ptr(bias), _any_code(bias), _ptr(out), dtype_code(out), out.stride(0), out_block_stride,
                                  n_rows, B, O, I, _stream()), "block_linear")


def gated_linear_recurrence(gates: torch.Tensor, u: torch.Tensor, y: torch.Tensor, y_bias: Optional[torch.Tensor],
                            lam: torch.Tensor, out: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor,
                            slots: torch.Tensor, n_seqs: int, decay: float, chunks: Optional[dict] = None,
                            block_width: int = 0) -> None:
    """The real-gated linear recurrence of csrc/sequence_parts.cu over the step's packed sequences.

    gates float32 [T, 2W]: per block of ``block_width`` channels the pre-activations of the block's recurrence gate, then
    of its input gate (0: one block, all recurrence gates, then all input gates); u float32 [T, W], y float32
    [T, W] view (pre-activation of the GELU branch), lam [W]; out [T, W]; state float32 [slots, >= W] view (updated).

    ``chunks``: for long portions, the step's tokens cut into chunks that run side by side (three kernels instead of one
    thread per channel walking the whole portion): int32 device arrays ``chunk_seq``, ``chunk_start``, ``seq_first_chunk``,
    ints ``n_chunks`` and ``chunk_len``, and ``work``, float32 with room for 3 * n_chunks * W values."""
    _cuda(gates, u, y, y_bias, lam, out, state, q_start, slots)
    W = lam.numel()
    for name, t in (("gates", gates), ("u", u), ("y", y)):
        _rows_contiguous(t, "gated_linear_recurrence " + name)
        if t.dtype != torch.float32:
            raise KernelError(f"gated_linear_recurrence: {name} must be float32")
    _rows_contiguous(out, "gated_linear_recurrence out")
    if gates.shape[1] < 2 * W or u.shape[1] < W or y.shape[1] < W or out.shape[1] < W or not lam.is_contiguous():
        raise KernelError("gated_linear_recurrence: buffers narrower than the recurrence")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < W:
        raise KernelError("gated_linear_recurrence: state must be float32 [slots, >= width]")
    if q_start.dtype != torch.int32 or slots.dtype != torch.int32:
        raise KernelError("gated_linear_recurrence: q_start and slots must be int32")
    if y_bias is not None and (y_bias.numel() != W or not y_bias.is_contiguous()):
        raise KernelError("gated_linear_recurrence: y_bias must hold one value per channel")
    args = (_ptr(gates), gates.stride(0), _ptr(u), u.stride(0), _ptr(y), y.stride(0), _ptr(y_bias), _any_code(y_bias), _ptr(lam),
            dtype_code(lam), _ptr(out), dtype_code(out), out.stride(0), _ptr(state), state.stride(0), _ptr(q_start), _ptr(slots),
            W, n_seqs, float(decay), int(block_width))
    if chunks is not None and chunks["n_chunks"] > 0:
        work = chunks["work"]
        if work.dtype != torch.float32 or work.numel() < 3 * chunks["n_chunks"] * W or not work.is_contiguous():
            raise KernelError("gated_linear_recurrence: the chunks' workspace is too small")
        for k in ("chunk_seq", "chunk_start", "seq_first_chunk"):
            if chunks[k].dtype != torch.int32:
                raise KernelError(f"gated_linear_recurrence: {k} must be int32")
        _check(core().rs_gated_linear_recurrence_chunked(*args, _ptr(chunks["chunk_seq"]), _ptr(chunks["chunk_start"]),
                                                         _ptr(chunks["seq_first_chunk"]), chunks["n_chunks"],
                                                         chunks["chunk_len"], _ptr(work), _stream()),
               "gated_linear_recurrence_chunked", 3)
        return
    _check(core().rs_gated_linear_recurrence(*args, _stream()), "gated_linear_recurrence")


def latent_kv_write(dkv: torch.Tensor, norm_weight: torch.Tensor, eps: float, q: torch.Tensor, q_head: int, q_nope: int,
                    q_lat: torch.Tensor, cos_sin: Optional[torch.Tensor], n_rot: int, positions: torch.Tensor,
                    seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int, cache: Optional[torch.Tensor],
                    rank: int, rot: int, lat: int, heads: int, n_tokens: int, status: torch.Tensor) -> None:
    """Latent norm + interleaved rotation + write of [latent | rotated key part | 0...] into a one-plane cache
    [pages, 1, 1, page_size, lat], and the rotated parts of the queries into q_lat[t, h * lat + rank : ...]."""
    _cuda(dkv, norm_weight, q, q_lat, cos_sin, positions, seq_of_token, block_table, cache, status)
    _rows_contiguous(dkv, "latent_kv_write dkv")
    _rows_contiguous(q, "latent_kv_write q")
    _rows_contiguous(q_lat, "latent_kv_write q_lat")
    if dkv.dtype != torch.float32 or dkv.shape[1] < rank + rot or norm_weight.numel() != rank or not norm_weight.is_contiguous():
        raise KernelError("latent_kv_write: dkv must be float32 [T, >= rank + rot] and the norm weight [rank]")
    if q.shape[1] < heads * q_head or q_lat.shape[1] < heads * lat or q_nope + rot > q_head or rank + rot > lat:
        raise KernelError("latent_kv_write: query buffers do not hold the heads")
    if cache is not None and (tuple(cache.shape[1:]) != (1, 1, page_size, lat) or not cache.is_contiguous()):
        raise KernelError(f"latent_kv_write: cache shape {tuple(cache.shape)} is not [pages, 1, 1, {page_size}, {lat}]")
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or cos_sin.shape[1] != n_rot or not cos_sin.is_contiguous()):
        raise KernelError("latent_kv_write: cos_sin must be contiguous float32 [positions, n_rot]")
    for name, t in (("positions", positions), ("seq_of_token", seq_of_token), ("block_table", block_table)):
        if t.dtype != torch.int32:
            raise KernelError(f"latent_kv_write: {name} must be int32")
    pos_stride = 1 if positions.dim() == 1 else positions.shape[1]
    _check(core().rs_latent_kv_write(
        _ptr(dkv), dkv.stride(0), _ptr(norm_weight), dtype_code(norm_weight), float(eps), _ptr(q), dtype_code(q), q.stride(0),
        q_head, q_nope, _ptr(q_lat), dtype_code(q_lat), q_lat.stride(0), _ptr(cos_sin), n_rot if cos_sin is not None else 0,
        0 if cos_sin is None else cos_sin.shape[0], _ptr(positions), pos_stride, _ptr(seq_of_token), _ptr(block_table),
        block_table.stride(0), page_size, _ptr(cache), _any_code(cache), 0 if cache is None else cache.stride(0),
        0 if cache is None else cache.shape[0], rank, rot, lat, heads, n_tokens, _ptr(status), _stream()), "latent_kv_write")


def relu_squared(x: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    """out[r, c] = max(x[r, c], 0)^2 (same element type; in place allowed)."""
    _cuda(x, out)
    _rows_contiguous(x, "relu_squared x")
    _rows_contiguous(out, "relu_squared out")
    if x.dtype != out.dtype or x.shape[1] != out.shape[1] or n_rows > min(x.shape[0], out.shape[0]):
        raise KernelError("relu_squared: x and out must share type and width")
    _check(core().rs_relu_squared(_ptr(x), dtype_code(x), x.stride(0), _ptr(out), out.stride(0), n_rows, x.shape[1],
                                  _stream()), "relu_squared")


GROUPED_ROWS_SMALL, GROUPED_ROWS_TILED = 8, 64     # rows of one expert per CTA of the grouped product's two forms
_GROUPED_ROWS_CHECKED = False


def grouped_rows_per_tile(small: bool) -> int:
    """Rows of one expert that a CTA of the grouped product takes (its row-streaming or its tiled form)."""
    global _GROUPED_ROWS_CHECKED
    if not _GROUPED_ROWS_CHECKED:
        if (int(core().rs_grouped_linear_rows_per_tile(1)), int(core().rs_grouped_linear_rows_per_tile(0))) != \
                (GROUPED_ROWS_SMALL, GROUPED_ROWS_TILED):
            raise KernelError("grouped_linear: the compiled kernels' tile sizes differ from the launcher's")
        _GROUPED_ROWS_CHECKED = True
    return GROUPED_ROWS_SMALL if small else GROUPED_ROWS_TILED


def moe_route(ids: Optional[torch.Tensor], table: torch.Tensor, n_experts: int, n_tokens: int, rows_per_tile: int,
              order: torch.Tensor, tiles: torch.Tensor, n_tiles: torch.Tensor, status: torch.Tensor) -> None:
    """Sorts the step's (token, k) pairs by the expert that ``table[ids[t], k]`` names: ``order`` [T * top] pair ids
    grouped by expert, ``tiles`` [max_tiles, 3] (expert, first row in order, rows), ``n_tiles`` [1].  Without ``ids``
    the table has one row per token of the step (the choice a router made): pair (t, k) goes to ``table[t, k]``."""
    _cuda(ids, table, order, tiles, n_tiles, status)
    V, top = table.shape
    for name, t in (("ids", ids), ("table", table), ("order", order), ("tiles", tiles), ("n_tiles", n_tiles)):
        if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
            raise KernelError(f"moe_route: {name} must be contiguous int32")
    if order.numel() < n_tokens * top or (ids.numel() if ids is not None else V) < n_tokens:
        raise KernelError("moe_route: order must hold tokens * top entries")
    if rows_per_tile not in (grouped_rows_per_tile(True), grouped_rows_per_tile(False), GROUPED_ROWS_LARGE):
        raise KernelError("moe_route: rows_per_tile must be a tile size of the grouped product")
    _check(core().rs_moe_route(_ptr(ids), _ptr(table), V, top, n_experts, n_tokens, rows_per_tile, _ptr(order), _ptr(tiles),
                               _ptr(n_tiles), tiles.numel() // 3, _ptr(status), _stream()), "moe_route")


def grouped_linear(a: torch.Tensor, a_div: int, weight: torch.Tensor, out: torch.Tensor, order: torch.Tensor,
                   tiles: torch.Tensor, n_tiles: torch.Tensor, max_tiles: int, gated: bool, small: bool,
                   interleaved: bool = False, relu2: bool = False) -> None:
    """One product per expert over the rows ``moe_route`` dealt to it.  Pair p reads row p // a_div of ``a`` and writes
    row p of ``out``.  weight [E, N, K], or [E, 2N, K] when ``gated``: out = SiLU(a Wg.T) * (a Wu.T) with the gate rows
    first and the up rows behind them, or alternating (gate 2n, up 2n + 1) when ``interleaved``.  ``relu2`` (plain
    products only): out = max(a W.T, 0)^2."""
    _cuda(a, weight, out, order, tiles, n_tiles)
    if gated and relu2:
        raise KernelError("grouped_linear: the squared ReLU follows a plain product, not a gated one")
    _rows_contiguous(a, "grouped_linear a")
    _rows_contiguous(out, "grouped_linear out")
    if weight.dim() != 3 or not weight.is_contiguous():
        raise KernelError("grouped_linear: weight must be contiguous [experts, rows, k]")
    E, rows, K = weight.shape
    N = rows // 2 if gated else rows
    if a.shape[1] != K or out.shape[1] != N or (gated and rows % 2) or max_tiles * 3 > tiles.numel():
        raise KernelError(f"grouped_linear: a {tuple(a.shape)} x weight {tuple(weight.shape)} -> out {tuple(out.shape)} "
                          f"does not fit")
    _check(core().rs_grouped_linear(_ptr(a), dtype_code(a), a.stride(0), a_div, _ptr(weight), dtype_code(weight),
                                    weight.stride(0), _ptr(out), dtype_code(out), out.stride(0), _ptr(order), _ptr(tiles),
                                    _ptr(n_tiles), max_tiles, N, K, (2 if interleaved else 1) if gated else 0,
                                    1 if small else 0, 1 if relu2 else 0, _stream()), "grouped_linear")


def grouped_gemm_mma_ok(a: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the tensor-core grouped product takes these operands: bfloat16, k a multiple of 8, rows 16-byte aligned."""
    return (a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 3 and weight.is_contiguous()
            and weight.shape[2] % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1 and a.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


GROUPED_ROWS_LARGE = 128      # row tile of the tensor-core grouped product's form for prompt portions


def grouped_gemm_mma(a: torch.Tensor, a_div: int, weight: torch.Tensor, out: torch.Tensor, order: torch.Tensor,
                     tiles: torch.Tensor, n_tiles: torch.Tensor, max_tiles: int, gated: bool, large: bool = False,
                     relu2: bool = False) -> None:
    """The grouped product of :func:`grouped_linear` on the tensor cores (csrc/grouped_gemm_mma.cu), for the row tiles
    that ``moe_route`` lists: of ``GROUPED_ROWS_TILED`` rows (64 x 64 tiles, for few rows per expert), or with ``large`` of
    ``GROUPED_ROWS_LARGE`` (128 x 128 tiles, for prompt portions).  ``gated``: the rows of every expert's matrix alternate
    gate, up and out = SiLU(gate) * up has half as many columns as the matrix has rows.  ``relu2`` (plain products only):
    out = max(a W.T, 0)^2."""
    _cuda(a, weight, out, order, tiles, n_tiles)
    if gated and relu2:
        raise KernelError("grouped_gemm_mma: the squared ReLU follows a plain product, not a gated one")
    _rows_contiguous(out, "grouped_gemm_mma out")
    if not grouped_gemm_mma_ok(a, weight):
        raise KernelError("grouped_gemm_mma: bfloat16 operands with 16-byte aligned rows and k a multiple of 8")
    E, rows, K = weight.shape
    if a.shape[1] != K or out.shape[1] != (rows // 2 if gated else rows) or (gated and rows % 2) or max_tiles * 3 > tiles.numel():
        raise KernelError(f"grouped_gemm_mma: a {tuple(a.shape)} x weight {tuple(weight.shape)} -> out {tuple(out.shape)} "
                          f"does not fit")
    if (int(bf16lib().rs_grouped_gemm_mma_rows_per_tile(0)), int(bf16lib().rs_grouped_gemm_mma_rows_per_tile(1))) != \
            (GROUPED_ROWS_TILED, GROUPED_ROWS_LARGE):
        raise KernelError("grouped_gemm_mma: the compiled kernel's row tiles differ from the launcher's")
    _check(bf16lib().rs_grouped_gemm_mma(_ptr(a), a.stride(0), a_div, _ptr(weight), weight.stride(0), rows, _ptr(out),
                                         dtype_code(out), out.stride(0), _ptr(order), _ptr(tiles), _ptr(n_tiles), max_tiles,
                                         K, 1 if gated else (2 if relu2 else 0), 1 if large else 0, _stream()), "grouped_gemm_mma")


def moe_combine(pair_out: torch.Tensor, top: int, weight: float, out: torch.Tensor, n_tokens: int,
                shared: Optional[torch.Tensor] = None, h: Optional[torch.Tensor] = None,
                gate_weight: Optional[torch.Tensor] = None, pair_weights: Optional[torch.Tensor] = None) -> None:
    """out[t] = weight * sum_k pair_out[t * top + k] + sigmoid(h[t] . gate_weight) * shared[t]  (float32 out; the
    second term only with ``shared``, its factor 1 without ``gate_weight``).  ``pair_weights`` float32 [T * top]:
    every pair is multiplied by its own weight in the sum."""
    _cuda(pair_out, out, shared, h, gate_weight, pair_weights)
    if pair_weights is not None and (pair_weights.dtype != torch.float32 or not pair_weights.is_contiguous()
                                     or pair_weights.numel() < n_tokens * top):
        raise KernelError("moe_combine: pair_weights must be contiguous float32 [T * top]")
    _rows_contiguous(pair_out, "moe_combine pair_out")
    _rows_contiguous(out, "moe_combine out")
    n = out.shape[1]
    if pair_out.dtype != torch.float32 or out.dtype != torch.float32 or pair_out.shape[1] != n \
            or pair_out.shape[0] < n_tokens * top or out.shape[0] < n_tokens:
        raise KernelError("moe_combine: pair_out float32 [T * top, n], out float32 [T, n]")
    if shared is not None:
        _rows_contiguous(shared, "moe_combine shared")
        if shared.shape[1] != n or shared.shape[0] < n_tokens:
            raise KernelError("moe_combine: shared must be [T, n]")
        if gate_weight is not None:
            _rows_contiguous(h, "moe_combine h")
            if gate_weight.numel() != n or not gate_weight.is_contiguous() or h.shape[1] != n:
                raise KernelError("moe_combine: the gate reads h [T, n] with a weight of n values")
    _check(core().rs_moe_combine(_ptr(pair_out), pair_out.stride(0), top, float(weight), _ptr(pair_weights), _ptr(shared),
                                 _any_code(shared),
                                 0 if shared is None else shared.stride(0), _ptr(h if gate_weight is not None else None),
                                 _any_code(h), 0 if h is None else h.stride(0), _ptr(gate_weight), _any_code(gate_weight),
                                 _ptr(out), out.stride(0), n_tokens, n, _stream()), "moe_combine")


# ----------------------------------------------------------------------------- several residual streams, summed embeddings
_streamlib = None


def streamlib():
    global _streamlib
    if _streamlib is None:
        lib = load_library("stream")
        lib.rs_embed_sum.argtypes = [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_long, c_long, c_void_p, c_int, c_int,
                                     c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_long,
                                     c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
        lib.rs_stream_layernorm.argtypes = [c_void_p, c_long, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                            c_float, c_void_p, c_int, c_long, c_int, c_int, c_int, c_void_p]
        lib.rs_stream_update.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                         c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_int, c_long, c_int, c_int, c_int,
                                         c_void_p]
        lib.rs_router_topk.argtypes = [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                       c_void_p, c_void_p, c_void_p, c_void_p]
        lib.rs_conv_norm_kv_write.argtypes = [c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_long, c_int, c_int, c_int,
                                              c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_long, c_void_p, c_long,
                                              c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.rs_sigmoid_gate.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int,
                                        c_void_p]
        _streamlib = lib
    return _streamlib


MAX_STREAMS = 16           # residual streams the stream kernels take
MAX_STREAM_WIDTH = 12288   # widest row they hold in shared memory


def _i32(name: str, *ts) -> None:
    for t in ts:
        if t is not None and (t.dtype != torch.int32 or not t.is_cuda):
            raise KernelError(f"{name}: index tensors must be int32 on the device")


def embed_sum(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, n_tokens: int, n_seqs: int, copies: int,
              positions: torch.Tensor, seq_of_token: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor,
              status: torch.Tensor, bigram: Optional[torch.Tensor] = None, mul_prev: int = 0, mul_cur: int = 0,
              prev_state: Optional[torch.Tensor] = None, position_table: Optional[torch.Tensor] = None,
              scale: float = 1.0) -> None:
    """out[t, c * D : (c + 1) * D] = scale * table[ids[t]] + bigram[row(t)] + position_table[place(t)] for every copy c < copies
    (float32).  ``bigram`` [buckets + 1, D]: row (previous token * mul_prev + token * mul_cur) mod buckets, the last
    row for a sequence's first token; the previous token of a portion's first token is read from ``prev_state``
    (int32 [slots, >= 1]), which then takes each sequence's last token.  ``positions`` [T, streams]: column 0 is the
    token's place in its sequence.  Either table may be left out."""
    _cuda(table, ids, out, positions, seq_of_token, q_start, slots, status, bigram, prev_state, position_table)
    _i32("embed_sum", ids, positions, seq_of_token, q_start, slots, prev_state)
    _rows_contiguous(out, "embed_sum out")
    V, D = table.shape
    if out.dtype != torch.float32 or out.shape[1] < copies * D or out.shape[0] < n_tokens or not table.is_contiguous():
        raise KernelError(f"embed_sum: out {tuple(out.shape)} must be float32 with {copies} x {D} columns")
    for name, t in (("bigram", bigram), ("position_table", position_table)):
        if t is not None and (t.dim() != 2 or t.shape[1] != D or not t.is_contiguous()):
            raise KernelError(f"embed_sum: {name} must be contiguous [rows, {D}]")
    if bigram is not None and (prev_state is None or prev_state.dim() != 2 or bigram.shape[0] < 2):
        raise KernelError("embed_sum: a bigram table needs the previous-token state [slots, >= 1] and at least two rows")
    _check(streamlib().rs_embed_sum(
        _ptr(table), dtype_code(table), V, _ptr(bigram), _any_code(bigram), 0 if bigram is None else bigram.shape[0] - 1,
        int(mul_prev), int(mul_cur), _ptr(position_table), _any_code(position_table),
        0 if position_table is None else position_table.shape[0], _ptr(ids), _ptr(positions), positions.stride(0),
        _ptr(seq_of_token), _ptr(q_start), _ptr(slots), _ptr(prev_state), 0 if prev_state is None else prev_state.stride(0),
        _ptr(out), out.stride(0), copies, D, n_tokens, n_seqs, float(scale), _ptr(status), _stream()), "embed_sum",
        2 if bigram is not None else 1)


def _check_streams(who: str, x: torch.Tensor, S: int, D: int):
    _rows_contiguous(x, f"{who} x")
    if x.dtype != torch.float32 or x.shape[1] < S * D:
        raise KernelError(f"{who}: x must be float32 with {S} x {D} columns")
    if not 1 <= S <= MAX_STREAMS or not 1 <= D <= MAX_STREAM_WIDTH:
        raise KernelError(f"{who}: {S} streams of width {D} (up to {MAX_STREAMS} streams, width up to {MAX_STREAM_WIDTH})")


def stream_layernorm(x: torch.Tensor, n_streams: int, coef: Optional[torch.Tensor], weight: torch.Tensor,
                     bias: Optional[torch.Tensor], eps: float, out: torch.Tensor, n_rows: int,
                     rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = layer_norm(sum_s coef[s] * x[src(r), s * D : (s + 1) * D]) * weight + bias, src(r) = rows[r] or r.
    x float32 [T, S * D]; coef [S] (None: every stream counts once); mean and variance (of the deviations) float32."""
    _cuda(x, coef, weight, bias, out, rows)
    D = weight.numel()
    _check_streams("stream_layernorm", x, n_streams, D)
    _rows_contiguous(out, "stream_layernorm out")
    if out.shape[1] < D or out.shape[0] < n_rows or (coef is not None and coef.numel() != n_streams):
        raise KernelError("stream_layernorm: out must hold n_rows x D values and coef one value per stream")
    _i32("stream_layernorm", rows)
    _check(streamlib().rs_stream_layernorm(_ptr(x), x.stride(0), _ptr(rows), _ptr(coef), _any_code(coef), _ptr(weight),
                                           dtype_code(weight), _ptr(bias), _any_code(bias), float(eps), _ptr(out),
                                           dtype_code(out), out.stride(0), n_streams, D, n_rows, _stream()),
           "stream_layernorm")


def stream_update(x: torch.Tensor, n_streams: int, y: torch.Tensor, mix: torch.Tensor, out_coef: torch.Tensor, n_rows: int,
                  next_coef: Optional[torch.Tensor] = None, next_weight: Optional[torch.Tensor] = None,
                  next_bias: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                  next_out: Optional[torch.Tensor] = None) -> None:
    """All streams of a token at once from the old ones: x_t <- sum_s mix[s, t] * x_s + out_coef[t] * y  (x float32
    [T, S * D] in place, y float32 [T, D], mix [S, S] indexed [from, to]).  With ``next_out`` also
    next_out = layer_norm(sum_t next_coef[t] * x_t) * next_weight + next_bias of the new streams, in the same pass."""
    _cuda(x, y, mix, out_coef, next_coef, next_weight, next_bias, next_out)
    D = y.shape[1]
    _check_streams("stream_update", x, n_streams, D)
    _rows_contiguous(y, "stream_update y")
    if y.dtype != torch.float32 or mix.numel() != n_streams * n_streams or out_coef.numel() != n_streams \
            or not mix.is_contiguous() or min(x.shape[0], y.shape[0]) < n_rows:
        raise KernelError("stream_update: y float32 [T, D], mix [S, S] contiguous, out_coef [S]")
    if next_out is not None:
        _rows_contiguous(next_out, "stream_update next_out")
        if next_weight is None or next_weight.numel() != D or next_out.shape[1] < D or next_out.shape[0] < n_rows:
            raise KernelError("stream_update: the next norm needs a weight of D values and an out of n_rows x D")
    _check(streamlib().rs_stream_update(
        _ptr(x), x.stride(0), _ptr(y), y.stride(0), _ptr(mix), dtype_code(mix), _ptr(out_coef), dtype_code(out_coef),
        _ptr(next_coef), _any_code(next_coef), _ptr(next_weight), _any_code(next_weight), _ptr(next_bias),
        _any_code(next_bias), float(next_eps), _ptr(next_out), _any_code(next_out),
        0 if next_out is None else next_out.stride(0), n_streams, D, n_rows, _stream()), "stream_update")


def router_topk(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, n_tokens: int, choice: torch.Tensor,
                weights: torch.Tensor, status: torch.Tensor, sigmoid: bool = False, groups: int = 0, keep: int = 0,
                scale: float = 1.0, renormalize: bool = True) -> None:
    """scores = softmax(logits[t]) (float32 [T, E]; ``sigmoid``: the sigmoid of every logit); choice[t] = the ``top``
    experts with the largest score + correction (int32 [T, top], the lower index on a tie); with ``groups`` > 0 only
    experts of the ``keep`` best of that many equal groups of neighbours (a group is worth its two largest scores +
    correction added); weights[t] = their scores times ``scale``, over (the sum of their scores + 1e-20) first if
    ``renormalize``."""
    _cuda(logits, correction, choice, weights, status)
    _rows_contiguous(logits, "router_topk logits")
    E = logits.shape[1]
    if logits.dtype != torch.float32 or choice.dtype != torch.int32 or weights.dtype != torch.float32 \
            or not choice.is_contiguous() or not weights.is_contiguous() or min(choice.numel(), weights.numel()) < n_tokens * top:
        raise KernelError("router_topk: logits float32 [T, E], choice int32 and weights float32 [T * top] contiguous")
    if not 1 <= top <= E <= 1024 or (correction is not None and correction.numel() != E):
        raise KernelError(f"router_topk: top {top} of {E} experts (up to 1024), one correction per expert")
    if groups and (E % groups or not 1 <= keep <= groups or top > keep * (E // groups)):
        raise KernelError(f"router_topk: {groups} groups of {E} experts, {keep} kept, top {top}")
    _check(streamlib().rs_router_topk(_ptr(logits), logits.stride(0), _ptr(correction), _any_code(correction), E, top,
                                      n_tokens, 1 if sigmoid else 0, int(groups), int(keep), float(scale),
                                      1 if renormalize else 0, _ptr(choice), _ptr(weights), _ptr(status), _stream()),
           "router_topk")


def conv_norm_kv_write(proj: torch.Tensor, conv_weight: Optional[torch.Tensor], tails: Optional[torch.Tensor], n_q: int,
                       n_kv: int, dk: int, dv: int, head_pad: int, unit_norm: bool, eps: float, q_out: torch.Tensor,
                       cache: Optional[torch.Tensor], block_table: torch.Tensor, page_size: int, positions: torch.Tensor,
                       seq_of_token: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, n_tokens: int, n_seqs: int,
                       write_kv: bool, status: torch.Tensor) -> None:
    """The projected rows ``proj`` [T, q heads * dk | kv heads * dk | kv heads * dv] (the key and value parts only with
    ``write_kv``) pass a causal convolution over time per channel (``conv_weight`` [taps, C] tap-major, None: none;
    ``tails`` float32 [slots, >= (taps - 1) * C] holds each request's last taps - 1 projected rows and is updated);
    with ``unit_norm`` every q and k head is divided by sqrt(mean square + eps); q goes to ``q_out`` [T, n_q * head_pad],
    k and v into the cache [pages, 2, n_kv, page_size, head_pad] at the tokens' places; padding is zero."""
    _cuda(proj, conv_weight, tails, q_out, cache, block_table, positions, seq_of_token, q_start, slots, status)
    _rows_contiguous(proj, "conv_norm_kv_write proj")
    _rows_contiguous(q_out, "conv_norm_kv_write q_out")
    _i32("conv_norm_kv_write", block_table, positions, seq_of_token, q_start, slots)
    C = n_q * dk + (n_kv * (dk + dv) if write_kv else 0)
    taps = 0 if conv_weight is None else conv_weight.shape[0]
    if proj.shape[1] < C or q_out.shape[1] < n_q * head_pad or q_out.dtype != proj.dtype or min(proj.shape[0], q_out.shape[0]) < n_tokens:
        raise KernelError(f"conv_norm_kv_write: proj {tuple(proj.shape)} / q_out {tuple(q_out.shape)} do not fit {C} channels")
    if head_pad % 16 or head_pad > 256 or max(dk, dv) > head_pad:
        raise KernelError(f"conv_norm_kv_write: head sizes {dk}/{dv} in rows of {head_pad} (a multiple of 16 up to 256)")
    if conv_weight is not None and (tuple(conv_weight.shape) != (taps, C) or not conv_weight.is_contiguous()):
        raise KernelError(f"conv_norm_kv_write: the convolution's weight must be contiguous [taps, {C}]")
    if taps > 1 and (tails is None or tails.dtype != torch.float32 or tails.dim() != 2 or tails.stride(1) != 1
                     or tails.shape[1] < (taps - 1) * C):
        raise KernelError("conv_norm_kv_write: tails must be float32 [slots, >= (taps - 1) * channels]")
    if write_kv and (cache is None or cache.dtype != proj.dtype or not cache.is_contiguous()
                     or tuple(cache.shape[1:]) != (2, n_kv, page_size, head_pad)):
        raise KernelError(f"conv_norm_kv_write: the cache must be [pages, 2, {n_kv}, {page_size}, {head_pad}] of the rows' type")
    _check(streamlib().rs_conv_norm_kv_write(
        _ptr(proj), dtype_code(proj), proj.stride(0), _ptr(conv_weight), _any_code(conv_weight), _ptr(tails),
        0 if tails is None else tails.stride(0), C, taps, n_q, n_kv, dk, dv, head_pad, 1 if unit_norm else 0, float(eps),
        _ptr(q_out), q_out.stride(0), _ptr(cache), 0 if cache is None else cache.stride(0),
        0 if cache is None else cache.shape[0], page_size, 1 if write_kv else 0, _ptr(block_table), block_table.stride(0),
        _ptr(positions), positions.stride(0), _ptr(seq_of_token), _ptr(q_start), _ptr(slots), n_tokens, n_seqs, _ptr(status),
        _stream()), "conv_norm_kv_write", 2 if taps > 1 else 1)


def sigmoid_gate(a: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, n_heads: int, dv: int, head_pad: int,
                 n_tokens: int) -> None:
    """out[t, h * dv + d] = a[t, h * head_pad + d] * sigmoid(gate[t, h * dv + d]) (None: times 1), sigmoid in float32."""
    _cuda(a, gate, out)
    _rows_contiguous(a, "sigmoid_gate a")
    _rows_contiguous(out, "sigmoid_gate out")
    if gate is not None:
        _rows_contiguous(gate, "sigmoid_gate gate")
    if a.shape[1] < n_heads * head_pad or out.shape[1] < n_heads * dv or (gate is not None and (gate.shape[1] < n_heads * dv
                                                                                               or gate.dtype != a.dtype)) \
            or out.dtype != a.dtype:
        raise KernelError("sigmoid_gate: a [T, heads * head_pad], gate and out [T, heads * dv], one element type")
    _check(streamlib().rs_sigmoid_gate(_ptr(a), a.stride(0), _ptr(gate), 0 if gate is None else gate.stride(0), _ptr(out),
                                       out.stride(0), dtype_code(a), n_heads, dv, head_pad, n_tokens, _stream()), "sigmoid_gate")


# ----------------------------------------------------------------------------- state-matrix mixers, talking-heads attention
_mixerslib = None

ACT_XIELU, ACT_GELU_TANH = 0, 1
ACTIVATIONS = {"xielu": ACT_XIELU, "gelu_tanh": ACT_GELU_TANH}


def mixerslib():
    global _mixerslib
    if _mixerslib is None:
        lib = load_library("mixers")
        lib.rs_state_recurrence_rows_pad.argtypes = [c_int]
        lib.rs_state_recurrence.argtypes = [c_void_p, c_long] * 7 + [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                                     c_void_p]
        lib.rs_hgrn2_prep.argtypes = [c_void_p, c_long, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                      c_int, c_int, c_void_p]
        lib.rs_delta_prep.argtypes = [c_void_p, c_long, c_void_p, c_int, c_void_p, c_long, c_void_p, c_long, c_void_p, c_int, c_void_p,
                                      c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p]
        lib.rs_head_norm_gate.argtypes = [c_void_p, c_long, c_void_p, c_int, c_void_p, c_long, c_void_p, c_int, c_long, c_int, c_int,
                                          c_float, c_int, c_int, c_void_p]
        lib.rs_retention_prep.argtypes = [c_void_p, c_long, c_void_p, c_int, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.rs_activation.argtypes = [c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.rs_scale_rows.argtypes = [c_void_p, c_long, c_int, c_int, c_float, c_void_p]
        lib.rs_talking_attention_q_per_cta.argtypes = [c_int, c_int, c_int]
        lib.rs_talking_attention_prep.argtypes = [c_void_p, c_long, c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p,
                                                  c_int, c_int, c_int, c_void_p, c_long, c_void_p, c_void_p, c_int, c_long, c_int, c_int, c_int,
                                                  c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                  c_void_p, c_void_p]
        lib.rs_talking_attention.argtypes = [c_void_p, c_long, c_void_p, c_void_p, c_int, c_long, c_int, c_int, c_int, c_void_p, c_int,
                                             c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_long, c_int,
                                             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
        lib.rs_talking_attention_mma_q_per_cta.argtypes = [c_int, c_int, c_int, c_int]
        lib.rs_talking_attention_mma.argtypes = [c_void_p, c_long, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_int,
                                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                 c_void_p, c_void_p]
        _mixerslib = lib
    return _mixerslib


def _f32_rows(who: str, **ts) -> None:
    for name, t in ts.items():
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"{who}: {name} must be float32 [rows, width] on the device with unit stride along its last axis")


def state_rows_pad(rows: int) -> int:
    """Rows a head of the state-matrix recurrence is padded to (its per-row inputs are laid out with this pitch)."""
    if rows <= 32:
        return 32
    n = 32
    while n < rows:
        n *= 2
    if n > 256:
        raise KernelError(f"state recurrence: {rows} rows per head (up to 256 are supported)")
    return n


def state_recurrence(q: torch.Tensor, k: torch.Tensor, g: torch.Tensor, beta: Optional[torch.Tensor], v: torch.Tensor,
                     out: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, n_seqs: int, heads: int,
                     group: int, rows_pad: int, columns: int, delta: bool) -> None:
    """Per (sequence, head) a float32 state S [rows, columns] walked over the step's tokens (csrc/state_mixers.cu).

    ``delta`` False: S = diag(g) S + k v^T, out = S^T q, with q, k, g [T, heads * rows_pad].
    ``delta`` True:  S = diag(g) S; u = beta (v - S^T k); S += k u^T; out = S^T q, with q and k [T, (heads / group) *
    rows_pad] (state head h reads q/k head h // group), g [T, heads * rows_pad], beta [T, heads].
    v, out [T, heads * columns]; state [slots, >= heads * columns * rows_pad], each head stored column by column."""
    _cuda(q, k, g, beta, v, out, state, q_start, slots)
    _f32_rows("state_recurrence", q=q, k=k, g=g, beta=beta, v=v, out=out, state=state)
    _i32("state_recurrence", q_start, slots)
    if delta and beta is None:
        raise KernelError("state_recurrence: the delta rule needs a write strength per head")
    qk_heads = heads // group if delta else heads
    if q.shape[1] < qk_heads * rows_pad or k.shape[1] < qk_heads * rows_pad or g.shape[1] < heads * rows_pad \
            or v.shape[1] < heads * columns or out.shape[1] < heads * columns or state.shape[1] < heads * columns * rows_pad:
        raise KernelError("state_recurrence: an operand is narrower than heads x rows / columns ask for")
    for name, t in (("q", q), ("k", k), ("g", g), ("state", state)):
        if t.stride(0) % 4 or t.data_ptr() % 16:
            raise KernelError(f"state_recurrence: {name} must start on 16 bytes with a row pitch that is a multiple of 4")
    _check(mixerslib().rs_state_recurrence(
        _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(g), g.stride(0), _ptr(beta), 0 if beta is None else beta.stride(0),
        _ptr(v), v.stride(0), _ptr(out), out.stride(0), _ptr(state), state.stride(0), _ptr(q_start), _ptr(slots), n_seqs, heads,
        group, rows_pad, columns, 1 if delta else 0, _stream()), "state_recurrence")


def hgrn2_prep(proj: torch.Tensor, f_bias: Optional[torch.Tensor], lower: torch.Tensor, q: torch.Tensor, g: torch.Tensor,
               w: torch.Tensor, heads: int, dim: int, rows_pad: int, n_tokens: int) -> None:
    """From proj [T, q | f | ...] (float32): q = silu(.), g = lower + (1 - lower) sigmoid(f + bias), w = 1 - g, each
    [T, heads * rows_pad] contiguous, padding zero."""
    _cuda(proj, f_bias, lower, q, g, w)
    _f32_rows("hgrn2_prep", proj=proj, q=q, g=g, w=w)
    if proj.shape[1] < 2 * heads * dim or any(t.shape[1] != heads * rows_pad or not t.is_contiguous() for t in (q, g, w)) \
            or lower.numel() != heads * dim or (f_bias is not None and f_bias.numel() != heads * dim):
        raise KernelError("hgrn2_prep: shapes do not fit heads x dim")
    _check(mixerslib().rs_hgrn2_prep(_ptr(proj), proj.stride(0), _ptr(f_bias), _any_code(f_bias), _ptr(lower), dtype_code(lower),
                                     _ptr(q), _ptr(g), _ptr(w), heads, dim, rows_pad, n_tokens, _stream()), "hgrn2_prep")


def delta_prep(proj: torch.Tensor, conv: Optional[torch.Tensor], tail: Optional[torch.Tensor], step: torch.Tensor,
               dt_bias: torch.Tensor, a_log: torch.Tensor, q: torch.Tensor, k: torch.Tensor, g: torch.Tensor, v: torch.Tensor,
               beta: torch.Tensor, seq_of_token: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, qk_heads: int,
               heads: int, dim: int, vdim: int, rows_pad: int, beta_off: int, unit_eps: float, q_scale: float, n_tokens: int,
               n_seqs: int) -> None:
    """Inputs of the delta-rule recurrence from proj [T, q | k | v | ... beta at ``beta_off``] (float32): a causal
    convolution over time per channel of q, k, v (``conv`` [taps, C] tap-major; ``tail`` [slots, >= (taps - 1) * C] holds
    every request's last projected rows and is updated), silu, q and k heads to unit length (q times ``q_scale``), the
    decay g = exp(-exp(a_log[h]) softplus(step + dt_bias)) per head and key channel, beta = sigmoid(.)."""
    _cuda(proj, conv, tail, step, dt_bias, a_log, q, k, g, v, beta, seq_of_token, q_start, slots)
    _f32_rows("delta_prep", proj=proj, step=step, q=q, k=k, g=g, v=v, beta=beta, tail=tail)
    _i32("delta_prep", seq_of_token, q_start, slots)
    C = 2 * qk_heads * dim + heads * vdim
    taps = 0 if conv is None else conv.shape[0]
    if conv is not None and (tuple(conv.shape) != (taps, C) or not conv.is_contiguous()):
        raise KernelError(f"delta_prep: the convolution's weight must be contiguous [taps, {C}]")
    if taps > 1 and (tail is None or tail.shape[1] < (taps - 1) * C):
        raise KernelError("delta_prep: tail must hold (taps - 1) * channels values per slot")
    if proj.shape[1] < max(C, beta_off + heads) or step.shape[1] < heads * dim or dt_bias.numel() != heads * dim \
            or a_log.numel() != heads or not all(t.is_contiguous() for t in (q, k, g, v, beta)) \
            or q.shape[1] != qk_heads * rows_pad or k.shape[1] != qk_heads * rows_pad or g.shape[1] != heads * rows_pad \
            or v.shape[1] != heads * vdim or beta.shape[1] != heads:
        raise KernelError("delta_prep: shapes do not fit the head counts and sizes")
    _check(mixerslib().rs_delta_prep(
        _ptr(proj), proj.stride(0), _ptr(conv), _any_code(conv), _ptr(tail), 0 if tail is None else tail.stride(0), _ptr(step),
        step.stride(0), _ptr(dt_bias), dtype_code(dt_bias), _ptr(a_log), dtype_code(a_log), _ptr(q), _ptr(k), _ptr(g), _ptr(v),
        _ptr(beta), _ptr(seq_of_token), _ptr(q_start), _ptr(slots), taps, qk_heads, heads, dim, vdim, rows_pad, beta_off,
        float(unit_eps), float(q_scale), n_tokens, n_seqs, _stream()), "delta_prep", 2 if taps > 1 else 1)


def retention_prep(proj: torch.Tensor, cos_sin: Optional[torch.Tensor], n_rot: int, positions: torch.Tensor, k_scale: float,
                   q: torch.Tensor, k: torch.Tensor, heads: int, dim: int, rows_pad: int, n_tokens: int,
                   status: torch.Tensor) -> None:
    """From proj [T, q | k | ...] (float32): every q and k head with its first ``n_rot`` coordinates turned by the token's
    position (coordinate i with i + n_rot / 2, ``cos_sin`` [positions, cos | sin]), k times ``k_scale`` afterwards; q and k
    [T, heads * rows_pad] contiguous, padding zero."""
    _cuda(proj, cos_sin, positions, q, k, status)
    _f32_rows("retention_prep", proj=proj, q=q, k=k, cos_sin=cos_sin)
    _i32("retention_prep", positions)
    if proj.shape[1] < 2 * heads * dim or any(t.shape[1] != heads * rows_pad or not t.is_contiguous() for t in (q, k)) \
            or rows_pad < dim:
        raise KernelError("retention_prep: shapes do not fit heads x dim")
    if n_rot and (cos_sin is None or cos_sin.shape[1] != n_rot or not cos_sin.is_contiguous() or n_rot > dim or n_rot % 2):
        raise KernelError("retention_prep: the rotation table must be contiguous [positions, n_rot] with n_rot even and <= dim")
    _check(mixerslib().rs_retention_prep(_ptr(proj), proj.stride(0), _ptr(cos_sin), n_rot if cos_sin is not None else 0,
                                         0 if cos_sin is None else cos_sin.shape[0], _ptr(positions), positions.stride(0),
                                         float(k_scale), _ptr(q), _ptr(k), heads, dim, rows_pad, n_tokens, _ptr(status),
                                         _stream()), "retention_prep")


def head_norm_gate(o: torch.Tensor, weight: Optional[torch.Tensor], gate: Optional[torch.Tensor], out: torch.Tensor, heads: int,
                   vdim: int, eps: float, n_tokens: int, gate_silu: bool = False) -> None:
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * sigmoid(gate[t, h, :]) (``gate_silu``: times
    silu(gate) instead); o and gate float32."""
    _cuda(o, weight, gate, out)
    _f32_rows("head_norm_gate", o=o, gate=gate)
    _rows_contiguous(out, "head_norm_gate out")
    if o.shape[1] < heads * vdim or out.shape[1] < heads * vdim or (gate is not None and gate.shape[1] < heads * vdim) \
            or (weight is not None and weight.numel() != vdim):
        raise KernelError("head_norm_gate: shapes do not fit heads x vdim")
    _check(mixerslib().rs_head_norm_gate(_ptr(o), o.stride(0), _ptr(weight), _any_code(weight), _ptr(gate),
                                         0 if gate is None else gate.stride(0), _ptr(out), dtype_code(out), out.stride(0), heads,
                                         vdim, float(eps), n_tokens, 1 if gate_silu else 0, _stream()), "head_norm_gate")


def activation(x: torch.Tensor, out: torch.Tensor, n_rows: int, kind: str, params: Optional[torch.Tensor] = None) -> None:
    """Elementwise activation of the first n_rows rows (float32 arithmetic): "xielu" with ``params`` = (p, q):
    z > 0: softplus(p) z^2 + z/2, else (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2;  "gelu_tanh"."""
    _cuda(x, out, params)
    _rows_contiguous(x, "activation x")
    _rows_contiguous(out, "activation out")
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation: unknown kind '{kind}' (known: {', '.join(sorted(ACTIVATIONS))})")
    if x.dtype != out.dtype or x.shape[1] != out.shape[1] or n_rows > min(x.shape[0], out.shape[0]):
        raise KernelError("activation: x and out must share element type and width")
    if kind == "xielu" and (params is None or params.numel() != 2):
        raise KernelError("activation: xielu takes two numbers")
    _check(mixerslib().rs_activation(_ptr(x), x.stride(0), _ptr(out), out.stride(0), dtype_code(x), x.shape[1], n_rows,
                                     ACTIVATIONS[kind], _ptr(params), _any_code(params), _stream()), "activation")


def scale_rows(x: torch.Tensor, n_rows: int, scale: float) -> None:
    """x[:n_rows] *= scale for float32 rows."""
    _cuda(x)
    _f32_rows("scale_rows", x=x)
    _check(mixerslib().rs_scale_rows(_ptr(x), x.stride(0), x.shape[1], n_rows, float(scale), _stream()), "scale_rows")


def talking_attention_q_per_cta(n_heads: int, dk: int, dv: int) -> int:
    n = int(mixerslib().rs_talking_attention_q_per_cta(n_heads, dk, dv))
    if n < 1:
        raise KernelError(f"talking attention: {n_heads} heads of {dk}/{dv} do not fit a CTA's shared memory")
    return n


def talking_attention_prep(proj: torch.Tensor, bias: Optional[torch.Tensor], q_norm: Optional[torch.Tensor],
                           k_norm: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor], n_rot: int,
                           q_out: torch.Tensor, gate_out: Optional[torch.Tensor], cache: torch.Tensor, block_table: torch.Tensor,
                           page_size: int, positions: torch.Tensor, seq_of_token: torch.Tensor, n_heads: int, n_kv: int, dk: int,
                           dv: int, n_tokens: int, write_kv: bool, status: torch.Tensor, row_norm: bool = False,
                           half_pairs: bool = False) -> None:
    """proj [T, q | k | v | gate] float32 (+ bias): RMS norm of q and k heads (weights [dk], None: none; ``row_norm``: one
    norm over the whole q row and one over the whole k row, weights [heads * dk] and [n_kv * dk]), rotation of
    the first ``n_rot`` coordinates by ``cos_sin`` [positions, cos | sin] in neighbouring pairs (``half_pairs``: coordinate
    i with i + n_rot / 2), q to ``q_out`` float32
    [T, heads * dk], k and v into ``cache`` [pages, 2, n_kv, page_size, head_pad] (padding zero), sigmoid of the gates
    to ``gate_out`` float32 [T, heads]."""
    _cuda(proj, bias, q_norm, k_norm, cos_sin, q_out, gate_out, cache, block_table, positions, seq_of_token, status)
    _f32_rows("talking_attention_prep", proj=proj, q_out=q_out, gate_out=gate_out, cos_sin=cos_sin)
    _i32("talking_attention_prep", block_table, positions, seq_of_token)
    hdp = cache.shape[-1]
    width = n_heads * dk + n_kv * (dk + dv)
    if proj.shape[1] < width + (n_heads if gate_out is not None else 0) or q_out.shape[1] < n_heads * dk \
            or (bias is not None and bias.numel() != width) or not cache.is_contiguous() \
            or tuple(cache.shape[1:]) != (2, n_kv, page_size, hdp) or hdp < max(dk, dv) \
            or (gate_out is not None and (gate_out.shape[1] != n_heads or not gate_out.is_contiguous())):
        raise KernelError("talking_attention_prep: shapes do not fit the head counts and sizes")
    nq_w, nk_w = (n_heads * dk, n_kv * dk) if row_norm else (dk, dk)
    if (q_norm is None) != (k_norm is None) or (q_norm is not None and (q_norm.numel() != nq_w or k_norm.numel() != nk_w
                                                                        or q_norm.dtype != k_norm.dtype)):
        raise KernelError(f"talking_attention_prep: q and k norm weights come together, [{nq_w}] and [{nk_w}], one element type")
    if n_rot and (cos_sin is None or cos_sin.shape[1] != n_rot or not cos_sin.is_contiguous()):
        raise KernelError("talking_attention_prep: the rotation table must be contiguous [positions, n_rot]")
    _check(mixerslib().rs_talking_attention_prep(
        _ptr(proj), proj.stride(0), _ptr(bias), _any_code(bias), _ptr(q_norm), _ptr(k_norm), _any_code(q_norm), float(eps),
        1 if row_norm else 0, _ptr(cos_sin), n_rot if cos_sin is not None else 0, 0 if cos_sin is None else cos_sin.shape[0],
        1 if half_pairs else 0, _ptr(q_out),
        q_out.stride(0), _ptr(gate_out), _ptr(cache), dtype_code(cache), cache.stride(0), cache.shape[0], page_size, hdp,
        _ptr(block_table), block_table.stride(0), _ptr(positions), positions.stride(0), _ptr(seq_of_token), n_heads, n_kv, dk, dv,
        n_tokens, 1 if write_kv else 0, _ptr(status), _stream()), "talking_attention_prep")


def talking_attention(q: torch.Tensor, gate: Optional[torch.Tensor], cache: torch.Tensor, block_table: torch.Tensor,
                      page_size: int, q_start: torch.Tensor, kv_len: torch.Tensor, work: torch.Tensor, n_work: int,
                      talk: Optional[torch.Tensor], sink: Optional[torch.Tensor], out: torch.Tensor, n_heads: int, n_kv: int,
                      dk: int, dv: int, window: int, q_per_cta: int, scale: float, status: torch.Tensor, chunk: int = 0) -> None:
    """Causal attention of the step's queries over the paged cache (within ``window`` keys if positive, within the query's
    own block of ``chunk`` positions if positive) with scores mixed across heads (``talk`` float32
    [heads, heads]: mixed[h] = sum_g talk[h, g] raw[g]) before a softmax whose denominator also holds exp(sink[h]);
    every head's output times ``gate`` [T, heads].  ``work``: (sequence, first query) per tile of ``q_per_cta`` queries."""
    _cuda(q, gate, cache, block_table, q_start, kv_len, work, talk, sink, out, status)
    _f32_rows("talking_attention", q=q, gate=gate)
    _rows_contiguous(out, "talking_attention out")
    _i32("talking_attention", block_table, q_start, kv_len, work)
    for name, t, n in (("talk", talk, n_heads * n_heads), ("sink", sink, n_heads)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError(f"talking_attention: {name} must be contiguous float32 with {n} values")
    if q.shape[1] < n_heads * dk or out.shape[1] < n_heads * dv or work.numel() < 2 * n_work or not cache.is_contiguous() \
            or (gate is not None and (gate.shape[1] != n_heads or not gate.is_contiguous())):
        raise KernelError("talking_attention: shapes do not fit the head counts and sizes")
    _check(mixerslib().rs_talking_attention(
        _ptr(q), q.stride(0), _ptr(gate), _ptr(cache), dtype_code(cache), cache.stride(0), cache.shape[0], page_size,
        cache.shape[-1], _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, _ptr(talk),
        _ptr(sink), _ptr(out), dtype_code(out), out.stride(0), n_heads, n_kv, dk, dv, window, int(chunk), q_per_cta,
        float(scale), _ptr(status), _stream()), "talking_attention")


def talking_attention_mma_q_per_cta(n_heads: int, n_kv: int, dk: int, dv: int) -> int:
    """Queries a CTA of the tensor-core form takes for these sizes; 0 when the shape is not one of its shapes (head sizes
    that are no multiple of 16, more than 32 heads, values wider than 128 or than 64 with more than 16 heads)."""
    return int(mixerslib().rs_talking_attention_mma_q_per_cta(n_heads, n_kv, dk, dv))


TALKING_WORK_COLS = 5          # sequence, first query, part, parts, first row of the tile's partial sums


def talking_attention_mma(q: torch.Tensor, gate: Optional[torch.Tensor], cache: torch.Tensor, block_table: torch.Tensor,
                          page_size: int, q_start: torch.Tensor, kv_len: torch.Tensor, work: torch.Tensor, n_work: int,
                          any_parts: bool, talk: Optional[torch.Tensor], sink: Optional[torch.Tensor], out: torch.Tensor,
                          partial: Optional[torch.Tensor], n_heads: int, n_kv: int, dk: int, dv: int, window: int, q_per_cta: int,
                          scale: float, status: torch.Tensor, chunk: int = 0) -> None:
    """``talking_attention`` for a bfloat16 cache on the tensor cores (csrc/talking_attention_mma.cu).  ``work`` rows are
    (sequence, first query, part, parts, first partial row): a tile's key tiles are dealt out over ``parts`` CTAs, whose
    sums meet in ``partial`` float32 [rows, >= heads * (dv + 2)] (part p of a tile of n queries uses rows first + p * n ..)."""
    _cuda(q, gate, cache, block_table, q_start, kv_len, work, talk, sink, out, partial, status)
    _f32_rows("talking_attention_mma", q=q, gate=gate, partial=partial)
    _rows_contiguous(out, "talking_attention_mma out")
    _i32("talking_attention_mma", block_table, q_start, kv_len, work)
    if cache.dtype != torch.bfloat16:
        raise KernelError("talking_attention_mma: the cache must be bfloat16")
    for name, t, n in (("talk", talk, n_heads * n_heads), ("sink", sink, n_heads)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError(f"talking_attention_mma: {name} must be contiguous float32 with {n} values")
    if q.shape[1] < n_heads * dk or out.shape[1] < n_heads * dv or work.numel() < TALKING_WORK_COLS * n_work \
            or not cache.is_contiguous() or (gate is not None and (gate.shape[1] != n_heads or not gate.is_contiguous())) \
            or out.stride(0) % 2 or out.data_ptr() % 8:
        raise KernelError("talking_attention_mma: shapes do not fit the head counts and sizes")
    rows = 0
    if partial is not None:
        if not partial.is_contiguous() or partial.shape[1] < n_heads * (dv + 2):
            raise KernelError("talking_attention_mma: the partial sums need contiguous rows of heads * (dv + 2) values")
        rows = partial.numel() // (n_heads * (dv + 2))
    _check(mixerslib().rs_talking_attention_mma(
        _ptr(q), q.stride(0), _ptr(gate), _ptr(cache), cache.stride(0), cache.shape[0], page_size, cache.shape[-1],
        _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, 1 if any_parts else 0,
        _ptr(talk), _ptr(sink), _ptr(out), dtype_code(out), out.stride(0), _ptr(partial), rows, n_heads, n_kv, dk, dv, window,
        int(chunk), q_per_cta, float(scale), _ptr(status), _stream()), "talking_attention_mma")
