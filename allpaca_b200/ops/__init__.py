"""Python faces of the CUDA kernels: argument checks, then one C call each.

Every function works on CUDA tensors in place or into a given output; none has
a CPU branch.  Partial sums: a matrix product that was split along K hands its
consumer a 32-bit tensor ``[S, T, N]``; consumers add the S slices in order.
"""
from __future__ import annotations

import functools
import os
from typing import Optional, Sequence

import torch

from . import library
from .library import KernelError, call, core, stream_handle

AP_F32, AP_BF16 = 0, 1


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return AP_F32
    if dt == torch.bfloat16:
        return AP_BF16
    raise KernelError(f"dtype {dt} is not one the kernels take (float32, bfloat16)")


def _check(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, has shape {tuple(t.shape)}")


def _partials(t: torch.Tensor, name: str):
    """(pointer, dtype code, S, stride between slices, T, N) of ``[S,T,N]`` or ``[T,N]``."""
    _check(t, name)
    if t.dim() == 3:
        if t.dtype != torch.float32:
            raise KernelError(f"{name}: partial sums must be float32")
        return t.data_ptr(), AP_F32, t.shape[0], t.shape[1] * t.shape[2], t.shape[1], t.shape[2]
    if t.dim() == 2:
        return t.data_ptr(), dtype_code(t.dtype), 1, t.numel(), t.shape[0], t.shape[1]
    raise KernelError(f"{name} must be [T,N] or [S,T,N], has shape {tuple(t.shape)}")


def embed_gather(tokens: torch.Tensor, table: torch.Tensor, x: torch.Tensor, scale: float = 1.0) -> None:
    """``x[t] = table[tokens[t]] * scale`` into the 32-bit residual stream ``x [T,H]``."""
    _check(tokens, "tokens", torch.int32, 1)
    _check(table, "table", dims=2)
    _check(x, "x", torch.float32, 2)
    T, H = x.shape
    if tokens.shape[0] != T or table.shape[1] != H:
        raise KernelError(f"embed_gather: shapes disagree: tokens {tuple(tokens.shape)}, "
                          f"table {tuple(table.shape)}, x {tuple(x.shape)}")
    call(core(), "ap_embed_gather", tokens.data_ptr(), table.data_ptr(), dtype_code(table.dtype),
         x.data_ptr(), T, H, table.shape[0], float(scale), stream_handle())


def bias_add(out: torch.Tensor, bias: torch.Tensor) -> None:
    """``out[t, n] += bias[n]`` for ``out [T, N]`` (or ``[1, T, N]``) in float32 or bfloat16."""
    _check(out, "out")
    _check(bias, "bias", dims=1)
    N = bias.shape[0]
    if out.dim() not in (2, 3) or out.shape[-1] != N or (out.dim() == 3 and out.shape[0] != 1):
        raise KernelError(f"bias_add: out {tuple(out.shape)} does not end in the bias's {N} columns")
    call(core(), "ap_bias_add", out.data_ptr(), dtype_code(out.dtype), bias.data_ptr(), dtype_code(bias.dtype),
         out.numel() // N, N, stream_handle())


def logit_transform(logits: torch.Tensor, bias: Optional[torch.Tensor] = None, scale: float = 1.0,
                    softcap: float = 0.0) -> None:
    """In place on 32-bit ``logits [R, V]``: ``z = (logit + bias) * scale``, then
    ``cap * tanh(z / cap)`` when ``softcap`` is positive."""
    _check(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    if bias is not None:
        _check(bias, "bias", dims=1)
        if bias.shape[0] != V:
            raise KernelError("logit_transform: the bias must have one entry per column")
    call(core(), "ap_logit_transform", logits.data_ptr(), bias.data_ptr() if bias is not None else 0,
         dtype_code(bias.dtype) if bias is not None else AP_F32, R, V, float(scale), float(softcap or 0.0),
         stream_handle())


def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """``v = x + sum(delta); out = rmsnorm(v) * weight``.

    Without ``rows`` every row is normed and ``x`` is overwritten with ``v``.  With
    ``rows`` (int32 indices) only those rows are normed into ``out[r]`` and ``x`` stays.
    """
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", dims=1)
    _check(out, "out", dims=2)
    T, H = x.shape
    if weight.shape[0] != H or out.shape[1] != H:
        raise KernelError("add_rmsnorm: widths disagree")
    S, dptr, dstride = 0, 0, 0
    if delta is not None:
        dptr, code, S, dstride, dT, dN = _partials(delta, "delta")
        if code != AP_F32 or dT != T or dN != H:
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} {delta.dtype} does not match x {tuple(x.shape)}")
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        R = rows.shape[0]
    else:
        R = T
    if out.shape[0] < R:
        raise KernelError("add_rmsnorm: out has too few rows")
    call(core(), "ap_add_rmsnorm", x.data_ptr(), dptr, S, dstride, weight.data_ptr(),
         dtype_code(weight.dtype), float(eps), out.data_ptr(), dtype_code(out.dtype),
         rows.data_ptr() if rows is not None else 0, R, H, stream_handle())


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    """``x += sum(delta)`` in 32-bit."""
    _check(x, "x", torch.float32, 2)
    dptr, code, S, dstride, dT, dN = _partials(delta, "delta")
    if code != AP_F32 or (dT, dN) != tuple(x.shape):
        raise KernelError("residual_add: delta does not match x")
    call(core(), "ap_residual_add", x.data_ptr(), dptr, S, dstride, x.numel(), stream_handle())


def rope_kv_store(qkv: torch.Tensor, q_out: torch.Tensor, cache_layer: Optional[torch.Tensor],
                  positions: torch.Tensor, token_seq: Optional[torch.Tensor],
                  block_table: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                  pairing: int, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Rotate Q and K of ``qkv [T, (nh+2nkv)*hd]`` and store K, V into cache pages.

    ``cache_layer`` is one layer's pages ``[pages, 2, nkv, P, hd]``; a row's page is
    ``block_table[token_seq[t], pos // P]`` and its slot ``pos % P``.  ``cos_sin`` is the
    ``[T, hd/2, 2]`` table of :func:`rope_table`; None: no rotation.  With ``cache_layer`` None nothing is stored; with ``num_kv_heads`` 0 the input
    holds queries only.
    """
    ptr, code, S, stride, T, N = _partials(qkv, "qkv")
    if N != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"rope_kv_store: qkv width {N} is not (heads + 2 kv_heads) * head_dim")
    _check(q_out, "q_out", dims=2)
    if q_out.shape[0] < T or q_out.shape[1] != num_heads * head_dim:
        raise KernelError("rope_kv_store: q_out shape does not match")
    _check(positions, "positions", torch.int32, 1)
    P, page_stride, cptr, tsptr, btptr, maxb = 1, 0, 0, 0, 0, 0
    if cache_layer is not None:
        _check(cache_layer, "cache_layer", q_out.dtype, 5)
        _, two, nkv, P, hd = cache_layer.shape
        if two != 2 or nkv != num_kv_heads or hd != head_dim:
            raise KernelError(f"rope_kv_store: cache layer {tuple(cache_layer.shape)} does not match the heads")
        page_stride = cache_layer.stride(0)
        cptr = cache_layer.data_ptr()
        if token_seq is None or block_table is None:
            raise KernelError("rope_kv_store: storing needs token_seq and block_table")
        _check(token_seq, "token_seq", torch.int32, 1)
        _check(block_table, "block_table", torch.int32, 2)
        tsptr, btptr, maxb = token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1]
    if cos_sin is not None:
        _check(cos_sin, "cos_sin", torch.float32, 3)
        if cos_sin.shape[0] < T or tuple(cos_sin.shape[1:]) != (head_dim // 2, 2):
            raise KernelError("rope_kv_store: cos_sin must be [T, head_dim/2, 2]")
    call(core(), "ap_rope_kv_store", ptr, code, S, stride, q_out.data_ptr(), cptr,
         dtype_code(q_out.dtype), positions.data_ptr(), tsptr, btptr, maxb,
         cos_sin.data_ptr() if cos_sin is not None else 0, int(pairing), T, num_heads,
         num_kv_heads, head_dim, P, page_stride, stream_handle())


def clear_page_tails(pages: torch.Tensor, page_size_dim: int, positions: torch.Tensor, token_seq: torch.Tensor,
                     block_table: torch.Tensor, context_lens: torch.Tensor) -> None:
    """For every row of the step that lands in slot 0 of a page: clear, in all runs of the cache
    group ``pages [runs, num_pages, *outer, P, *inner]`` (``page_size_dim`` is the index of the
    ``P`` dimension), the slots of that page behind the sequence's last token of this step.  A page
    taken over from another request then holds nothing of it that a kernel could read."""
    _check(pages, "pages")
    for t, n in ((positions, "positions"), (token_seq, "token_seq"), (context_lens, "context_lens")):
        _check(t, n, torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    if not (2 <= page_size_dim < pages.dim()):
        raise KernelError("clear_page_tails: pages must be [runs, num_pages, ..., P, ...]")
    outer = 1
    for d in pages.shape[2:page_size_dim]:
        outer *= d
    inner = 1
    for d in pages.shape[page_size_dim + 1:]:
        inner *= d
    call(core(), "ap_clear_page_tails", pages.data_ptr(), pages.element_size(), pages.stride(0), pages.stride(1),
         pages.shape[0], outer, pages.shape[page_size_dim], inner, positions.data_ptr(), token_seq.data_ptr(),
         block_table.data_ptr(), block_table.shape[1], context_lens.data_ptr(), positions.shape[0], stream_handle())


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, table: torch.Tensor) -> None:
    """``table[t, i] = (cos, sin)(positions[t] * inv_freq[i])`` with a 32-bit angle."""
    _check(positions, "positions", torch.int32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    _check(table, "table", torch.float32, 3)
    T, half = positions.shape[0], inv_freq.shape[0]
    if tuple(table.shape) != (T, half, 2):
        raise KernelError("rope_table: table must be [T, head_dim/2, 2]")
    call(core(), "ap_rope_table", positions.data_ptr(), inv_freq.data_ptr(), table.data_ptr(), T, half,
         stream_handle())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, pairs: bool = False) -> None:
    """``out[t, j] = silu(gate_up[t, j]) * gate_up[t, I + j]``; with ``pairs`` the gate and up
    columns alternate: ``silu(gate_up[t, 2j]) * gate_up[t, 2j + 1]``."""
    ptr, code, S, stride, T, N = _partials(gate_up, "gate_up")
    _check(out, "out", dims=2)
    if N != 2 * out.shape[1] or out.shape[0] != T:
        raise KernelError("swiglu: out must be [T, I] for gate_up [T, 2I]")
    call(core(), "ap_swiglu", ptr, code, S, stride, out.data_ptr(), dtype_code(out.dtype), T,
         out.shape[1], 1 if pairs else 0, stream_handle())


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out[M,N] = a[M,K] @ w[N,K]^T`` on the CUDA cores with 32-bit accumulation."""
    _check(a, "a", dims=2)
    _check(w, "w", dims=2)
    _check(out, "out", dims=2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    call(core(), "ap_gemm_simt", a.data_ptr(), dtype_code(a.dtype), w.data_ptr(), dtype_code(w.dtype),
         out.data_ptr(),
         dtype_code(out.dtype), M, N, K, K, K, N, stream_handle())


def tensor_core_gemm_available() -> bool:
    return hasattr(core(), "ap_gemm_tc")


class RowScale:
    """Partial sums of squares ``ss [rows, parts]`` (float32) of the rows a product's input was
    rounded from, with the rows' width and the norm's eps: the product's result row ``m`` is
    multiplied by ``1/sqrt(sum(ss[m]) / width + eps)``.  With the norm's weight multiplied into
    the product's weight beforehand, that is the RMSNorm of the input, applied afterwards."""

    __slots__ = ("ss", "parts", "width", "eps")

    def __init__(self, ss: torch.Tensor, parts: int, width: int, eps: float):
        self.ss, self.parts, self.width, self.eps = ss, int(parts), int(width), float(eps)


def _scale_args(scale: Optional[RowScale], M: int):
    if scale is None:
        return 0, 0, 0.0, 0.0
    _check(scale.ss, "scale.ss", torch.float32, 2)
    if scale.ss.shape[0] < M or scale.ss.shape[1] != scale.parts:
        raise KernelError(f"gemm_tc: the sums of squares {tuple(scale.ss.shape)} do not cover {M} rows of "
                          f"{scale.parts} parts")
    return scale.ss.data_ptr(), scale.parts, 1.0 / scale.width, scale.eps


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, nsplit: int = 1,
            reduce: bool = False, pairs: bool = False, scale: Optional[RowScale] = None) -> None:
    """bfloat16 ``a[M,K] @ w[N,K]^T`` on the tcgen05 tensor cores.

    ``nsplit`` K slices run as separate CTAs.  With ``reduce`` they add up inside a
    thread-block cluster (at most 8 slices, at most 256 rows) and ``out`` is the finished
    ``[M,N]`` in bfloat16 or float32; without it ``out`` is float32 ``[nsplit, M, N]`` partial
    sums (``[M,N]`` for ``nsplit == 1``).  ``pairs`` (at most 256 rows, finished sums, bfloat16
    out): the rows of ``w`` alternate gate and up, and ``out[M,N/2] = silu(gate) * up``.
    ``scale`` (finished sums only): see :class:`RowScale`.
    """
    _check(a, "a", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    _check(out, "out")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError("gemm_tc: inner sizes disagree")
    if pairs:
        if tuple(out.shape) != (M, N // 2) or N % 2:
            raise KernelError("gemm_tc: out must be [M,N/2] for alternating gate and up rows")
        stride = 0
    elif nsplit == 1 or reduce:
        if tuple(out.shape) != (M, N):
            raise KernelError("gemm_tc: out must be [M,N]")
        stride = 0
    else:
        if tuple(out.shape) != (nsplit, M, N) or out.dtype != torch.float32:
            raise KernelError("gemm_tc: partial sums must be float32 [nsplit,M,N]")
        stride = M * N
    ss, parts, inv_width, eps = _scale_args(scale, M)
    call(core(), "ap_gemm_tc", a.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
         M, N, K, K, K, N // 2 if pairs else N, nsplit, stride, 1 if reduce else 0, 1 if pairs else 0,
         ss, parts, inv_width, eps, 0, 0, 0, 0, stream_handle())


def gemm_tc_residual_parts(N: int, nsplit: int) -> int:
    """Parts of sums of squares per row that :func:`gemm_tc_residual` writes."""
    return int(core().ap_gemm_tc_residual_parts(int(N), int(nsplit)))


def gemm_tc_residual(a: torch.Tensor, w: torch.Tensor, x: torch.Tensor, xb: torch.Tensor, ss: torch.Tensor,
                     nsplit: int = 1) -> int:
    """``x[M,N] += a[M,K] @ w[N,K]^T`` into the 32-bit residual (at most 256 rows; 1, 2, 4 or 8 K
    slices added in a cluster), with the updated rows copied to ``xb`` in bfloat16 and partial sums of
    their squares written to ``ss [M, parts]``; returns ``parts``."""
    _check(a, "a", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    _check(x, "x", torch.float32, 2)
    _check(xb, "xb", torch.bfloat16, 2)
    _check(ss, "ss", torch.float32, 2)
    M, K = a.shape
    N = w.shape[0]
    parts = gemm_tc_residual_parts(N, nsplit)
    if w.shape[1] != K or tuple(x.shape) != (M, N) or tuple(xb.shape) != (M, N) or ss.shape[0] < M \
            or ss.shape[1] != parts:
        raise KernelError(f"gemm_tc_residual: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, x {tuple(x.shape)}, "
                          f"xb {tuple(xb.shape)}, ss {tuple(ss.shape)} (parts {parts})")
    call(core(), "ap_gemm_tc", a.data_ptr(), w.data_ptr(), x.data_ptr(), AP_F32, M, N, K, K, K, N, nsplit, 0,
         1 if nsplit > 1 else 0, 2, 0, 0, 0.0, 0.0, xb.data_ptr(), N, ss.data_ptr(), parts, stream_handle())
    return parts


def gemm_tc_rope(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cache_layer: Optional[torch.Tensor],
                 positions: torch.Tensor, token_seq: Optional[torch.Tensor], block_table: Optional[torch.Tensor],
                 cos_sin: Optional[torch.Tensor], pairing: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 nsplit: int = 1, scale: Optional[RowScale] = None) -> None:
    """The stacked Q, K, V projection of at most 256 rows ``a [M,K]`` with :func:`rope_kv_store` in
    its epilogue: Q rotated into ``q_out [M, nh*hd]``, K rotated and V into the pages of
    ``cache_layer`` (None: not stored).  ``pairing`` 0: the rows of every Q and K head of ``w`` are
    interleaved (row 2j: element j, row 2j+1: element j + hd/2) and the results go back to their
    places; 1: neighbouring elements pair.  ``scale``: see :class:`RowScale`."""
    _check(a, "a", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    _check(q_out, "q_out", torch.bfloat16, 2)
    _check(positions, "positions", torch.int32, 1)
    M, K = a.shape
    if w.shape != ((num_heads + 2 * num_kv_heads) * head_dim, K) or q_out.shape[0] < M \
            or q_out.shape[1] != num_heads * head_dim or positions.shape[0] < M:
        raise KernelError(f"gemm_tc_rope: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, q_out {tuple(q_out.shape)}")
    P, page_stride, cptr, tsptr, btptr, maxb = 1, 0, 0, 0, 0, 0
    if cache_layer is not None:
        _check(cache_layer, "cache_layer", torch.bfloat16, 5)
        _, two, nkv, P, hd = cache_layer.shape
        if two != 2 or nkv != num_kv_heads or hd != head_dim or token_seq is None or block_table is None:
            raise KernelError("gemm_tc_rope: the cache layer does not match the heads, or its block table is missing")
        _check(token_seq, "token_seq", torch.int32, 1)
        _check(block_table, "block_table", torch.int32, 2)
        page_stride, cptr = cache_layer.stride(0), cache_layer.data_ptr()
        tsptr, btptr, maxb = token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1]
    if cos_sin is not None:
        _check(cos_sin, "cos_sin", torch.float32, 3)
        if cos_sin.shape[0] < M or tuple(cos_sin.shape[1:]) != (head_dim // 2, 2):
            raise KernelError("gemm_tc_rope: cos_sin must be [M, head_dim/2, 2]")
    ss, parts, inv_width, eps = _scale_args(scale, M)
    call(core(), "ap_gemm_tc_rope", a.data_ptr(), w.data_ptr(), M, K, K, K, nsplit, ss, parts, inv_width, eps,
         q_out.data_ptr(), cptr, positions.data_ptr(), tsptr, btptr, maxb,
         cos_sin.data_ptr() if cos_sin is not None else 0, int(pairing), num_heads, num_kv_heads, head_dim, P,
         page_stride, stream_handle())


def gemm_tc_dual(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """The tensor-core product with two weight tiles per CTA, for more than 64 rows:
    ``out[M,N] = a[M,K] @ w[N,K]^T``."""
    _check(a, "a", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    _check(out, "out", dims=2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_tc_dual: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    call(core(), "ap_gemm_tc_dual", a.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
         M, N, K, K, K, N, stream_handle())


def gemm_tc_pair(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, pairs: bool = False,
                 share_tiles: bool = True) -> None:
    """The tensor-core product on pairs of SMs (``tcgen05.mma.cta_group::2``), for many rows: two
    CTAs share a tile of 256 weight rows x up to 256 rows of ``a``, each loading half of either.
    With ``share_tiles`` a product of fewer tiles than half the pairs splits every tile's K among
    up to four pairs.

    ``pairs`` False: ``out[M,N] = a[M,K] @ w[N,K]^T``.  True: the rows of ``w [N,K]`` alternate
    gate, up, gate, up ... and ``out[M,N/2] = silu(gate) * up``.
    """
    _check(a, "a", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    _check(out, "out", dims=2)
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if pairs else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or (pairs and N % 2):
        raise KernelError(f"gemm_tc_pair: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    scratch = _scratch_for_persistent(a.device) if share_tiles else None
    call(core(), "ap_gemm_tc_pair", a.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
         M, N, K, K, K, n_out, 1 if pairs else 0, scratch.data_ptr() if scratch is not None else 0,
         scratch.numel() if scratch is not None else 0, stream_handle())


_persistent_scratch = {}


def _scratch_for_persistent(device: torch.device) -> torch.Tensor:
    """The buffer through which CTAs of the persistent product that share a tile hand partial
    sums to one another: one per (device, stream), zero when made; the kernel leaves its
    flags zero again."""
    key = (device.index, stream_handle())
    buf = _persistent_scratch.get(key)
    if buf is None:
        nbytes = int(core().ap_gemm_tc_persistent_scratch_bytes())
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _persistent_scratch[key] = buf
    return buf


def gemm_tc_persistent(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, pairs: bool = False,
                       share_tiles: bool = True) -> None:
    """The persistent tensor-core product for more than 64 rows: one CTA per SM walks the
    output tiles, and a tile is written out while the next one is being computed.  With
    ``share_tiles`` a product of fewer tiles than half the SMs splits every tile's K among
    several CTAs.

    ``pairs`` False: ``out[M,N] = a[M,K] @ w[N,K]^T``.  True: the rows of ``w [N,K]`` alternate
    gate, up, gate, up ... and ``out[M,N/2] = silu(gate) * up``.
    """
    _check(a, "a", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    _check(out, "out", dims=2)
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if pairs else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or (pairs and N % 2):
        raise KernelError(f"gemm_tc_persistent: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, "
                          f"out {tuple(out.shape)}")
    scratch = _scratch_for_persistent(a.device) if share_tiles else None
    call(core(), "ap_gemm_tc_persistent", a.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
         M, N, K, K, K, n_out, 1 if pairs else 0, scratch.data_ptr() if scratch is not None else 0,
         scratch.numel() if scratch is not None else 0, stream_handle())


def _decode_attention(lib, q, out, cache_layer, block_table, positions, rows, num_heads, num_kv_heads, head_dim, P,
                      scale, window, max_context, scratch, use_tma, mean_context=0) -> None:
    """The first ``rows`` rows of the batch, one per sequence: the split kernels."""
    tma = (use_tma and hasattr(lib, "ap_attention_decode_tma")
           and bool(lib.ap_attention_decode_tma_supports(num_heads, num_kv_heads, head_dim, P))
           and cache_layer.stride(0) == 2 * num_kv_heads * P * head_dim)
    sizes = ()
    if tma:
        # 16 slices (a cluster size the kernel has to opt into) where the exchange buffer holds them
        sizes = (2, 4, 8, 16) if lib.ap_attention_decode_tma_in_cluster(num_heads, num_kv_heads, 16) else (2, 4, 8)
    # CTAs the GPU holds at once: of the TMA-fed kernel two per SM at head size 128, four at 64
    slots = 444
    if tma:
        slots = int(lib.ap_attention_decode_tma_slots()) if hasattr(lib, "ap_attention_decode_tma_slots") else 296
    nsplit = decode_splits(rows, num_heads, num_kv_heads, max_context, window, slots=slots, cluster_sizes=sizes,
                           mean_context=mean_context)
    po = pm = 0
    needs_scratch = nsplit > 1 and not (tma and lib.ap_attention_decode_tma_in_cluster(num_heads, num_kv_heads, nsplit))
    if needs_scratch:
        if scratch is None:
            raise KernelError("attention: key slices need a scratch provider")
        po = scratch("attn.part_o", (nsplit, rows, num_heads, head_dim), torch.float32).data_ptr()
        pm = scratch("attn.part_ml", (nsplit, rows, num_heads, 2), torch.float32).data_ptr()
    if tma:
        # fed by TMA: a ring of tiles in flight, two CTAs per SM; 2, 4, 8 or 16 slices are combined
        # inside a thread-block cluster and need no scratch
        call(lib, "ap_attention_decode_tma", q.data_ptr(), out.data_ptr(), cache_layer.data_ptr(),
             cache_layer.shape[0], block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), rows,
             num_heads, num_kv_heads, head_dim, P, cache_layer.stride(0), float(scale), int(window or 0),
             nsplit, po, pm, stream_handle())
        return
    call(lib, "ap_attention_tc", q.data_ptr(), out.data_ptr(), cache_layer.data_ptr(),
         block_table.data_ptr(), block_table.shape[1], 0, positions.data_ptr(),
         rows, rows, num_heads, num_kv_heads, head_dim, P, cache_layer.stride(0), float(scale),
         int(window or 0), 1, 0, nsplit, po, pm, stream_handle())


# CTAs of the tcgen05 attention with two query tiles from which it is preferred to the kernel
# with one: below, the narrow kernel's twice as many CTAs fill the SMs better
WIDE_ATTENTION_MIN_CTAS = int(os.environ.get("ALLPACA_WIDE_ATTENTION_MIN_CTAS", "148"))


def _prompt_attention(lib, q, out, cache_layer, block_table, seq_start, positions, first_seq, query_lens, T,
                      num_heads, num_kv_heads, head_dim, P, scale, window, use_tcgen05, wide=None) -> None:
    """The sequences from ``first_seq`` on (their rows follow those of the sequences before):
    the tcgen05 kernels for 64 rows or more of a shape they take, else the mma.sync tile kernel.
    Of the two tcgen05 kernels the one with two query tiles to a CTA runs when ``wide`` says so,
    or (``wide=None``) when the portions are long enough to fill the GPU with such CTAs.
    Rows are addressed through ``seq_start``, so only it and the block table are offset."""
    nseq = len(query_lens)
    table_ptr = block_table.data_ptr() + first_seq * block_table.shape[1] * 4
    start_ptr = seq_start.data_ptr() + first_seq * 4
    if (use_tcgen05 and wide is not False and sum(query_lens) >= 64 and hasattr(lib, "ap_attention_tcgen05_wide")
            and lib.ap_attention_tcgen05_wide_supports(num_heads, num_kv_heads, head_dim, P)
            and cache_layer.stride(0) == 2 * num_kv_heads * P * head_dim):
        per_cta = int(lib.ap_attention_tcgen05_wide_tokens_per_cta(num_heads, num_kv_heads))
        ctas = sum(-(-n // per_cta) for n in query_lens)
        if wide or ctas * num_kv_heads >= WIDE_ATTENTION_MIN_CTAS:
            call(lib, "ap_attention_tcgen05_wide", q.data_ptr(), out.data_ptr(), cache_layer.data_ptr(),
                 cache_layer.shape[0], table_ptr, block_table.shape[1], start_ptr,
                 positions.data_ptr(), nseq, T, num_heads, num_kv_heads, head_dim, P, cache_layer.stride(0),
                 float(scale), int(window or 0), ctas, stream_handle())
            return
    if (use_tcgen05 and sum(query_lens) >= 64 and hasattr(lib, "ap_attention_tcgen05")
            and lib.ap_attention_tcgen05_supports(num_heads, num_kv_heads, head_dim, P)
            and cache_layer.stride(0) == 2 * num_kv_heads * P * head_dim):
        tpt = int(lib.ap_attention_tcgen05_tokens_per_tile(num_heads, num_kv_heads))
        tiles = sum(-(-n // tpt) for n in query_lens)
        call(lib, "ap_attention_tcgen05", q.data_ptr(), out.data_ptr(), cache_layer.data_ptr(),
             cache_layer.shape[0], table_ptr, block_table.shape[1], start_ptr,
             positions.data_ptr(), nseq, T, num_heads, num_kv_heads, head_dim, P, cache_layer.stride(0),
             float(scale), int(window or 0), tiles, stream_handle())
        return
    tpt = int(lib.ap_attention_tc_tokens_per_tile(num_heads, num_kv_heads))
    tiles = sum(-(-n // tpt) for n in query_lens)
    call(lib, "ap_attention_tc", q.data_ptr(), out.data_ptr(), cache_layer.data_ptr(),
         table_ptr, block_table.shape[1], start_ptr, positions.data_ptr(),
         nseq, T, num_heads, num_kv_heads, head_dim, P, cache_layer.stride(0), float(scale),
         int(window or 0), 0, tiles, 1, 0, 0, stream_handle())


def attention(q: torch.Tensor, out: torch.Tensor, cache_layer: torch.Tensor,
              block_table: torch.Tensor, token_seq: torch.Tensor, positions: torch.Tensor,
              num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
              window: int = 0, seq_start: Optional[torch.Tensor] = None,
              query_lens: Optional[Sequence[int]] = None, max_context: int = 0,
              scratch=None, use_tcgen05: bool = True, use_tma: bool = True,
              wide: Optional[bool] = None, mean_context: int = 0) -> None:
    """Causal attention of every row of ``q [T, nh*hd]`` over its sequence's cached keys.

    float32 runs the general CUDA-core kernel (the true 32-bit path).  bfloat16 runs on the
    tensor cores when ``seq_start`` (device, ``[nseq+1]``) and ``query_lens`` (host) are
    given: the split kernel when every sequence brings one row; else, for 64 rows or more and
    the shapes it takes, a tcgen05 kernel (``use_tcgen05``; ``wide`` picks the one with two query
    tiles to a CTA, ``None`` by the number of CTAs), and otherwise the tile kernel.
    ``scratch(name, shape, dtype)`` supplies the partial-result buffers of the split kernel
    where its key slices are not combined inside a thread-block cluster.  ``max_context`` and
    ``mean_context`` (0: all alike) are bounds on the longest and the average number of keys of
    the one-row sequences, from which the number of key slices is planned.
    """
    _check(q, "q", dims=2)
    _check(out, "out", q.dtype, 2)
    _check(cache_layer, "cache_layer", q.dtype, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(token_seq, "token_seq", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    T = token_seq.shape[0]
    if q.shape[0] < T or q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q/out shape does not match the heads")
    _, two, nkv, P, hd = cache_layer.shape
    if two != 2 or nkv != num_kv_heads or hd != head_dim:
        raise KernelError("attention: cache layer does not match the heads")
    lib = library.attention(head_dim)
    if q.dtype == torch.bfloat16 and seq_start is not None and query_lens is not None \
            and hasattr(lib, "ap_attention_tc"):
        _check(seq_start, "seq_start", torch.int32, 1)
        nseq = len(query_lens)
        if seq_start.shape[0] != nseq + 1 or sum(query_lens) != T:
            raise KernelError("attention: seq_start/query_lens do not describe the rows")
        # Sequences that bring one row each (decoding) go to the split kernel, prompt portions to
        # the tile kernels.  A mixed batch whose one-row sequences come first (the scheduler's
        # order) is two launches over disjoint rows; one-row sequences further back ride along
        # with the portions.
        nd = 0
        while nd < nseq and query_lens[nd] == 1:
            nd += 1
        if nd > 0:
            _decode_attention(lib, q, out, cache_layer, block_table, positions, nd, num_heads, num_kv_heads,
                              head_dim, P, scale, window, max_context, scratch, use_tma, mean_context)
        if nd < nseq:
            _prompt_attention(lib, q, out, cache_layer, block_table, seq_start, positions, nd, query_lens[nd:], T,
                              num_heads, num_kv_heads, head_dim, P, scale, window, use_tcgen05, wide)
        return
    call(lib, "ap_attention_rows", q.data_ptr(), out.data_ptr(), cache_layer.data_ptr(),
         dtype_code(q.dtype), block_table.data_ptr(), block_table.shape[1], token_seq.data_ptr(),
         positions.data_ptr(), T, num_heads, num_kv_heads, head_dim, P, cache_layer.stride(0),
         float(scale), int(window or 0), stream_handle())


def decode_splits(rows: int, num_heads: int, num_kv_heads: int, max_context: int, window: int = 0,
                  slots: int = 444, cluster_sizes: Sequence[int] = (), mean_context: int = 0) -> int:
    """Key slices for the split kernels (see :func:`_decode_splits`; results are remembered)."""
    mean = int(mean_context or 0)
    if mean <= 0 or mean > max_context:
        mean = int(max_context)
    return _decode_splits(int(rows), int(num_heads), int(num_kv_heads), int(max_context), int(window or 0),
                          int(slots), tuple(cluster_sizes), mean)


@functools.lru_cache(maxsize=4096)
def _decode_splits(rows: int, num_heads: int, num_kv_heads: int, max_context: int, window: int,
                   slots: int, cluster_sizes: tuple, mean_context: int = 0) -> int:
    """Key slices for the split kernels.

    The cp.async kernel runs three CTAs per SM (``slots`` 444), the one fed by TMA two (296).
    A slice walks ``tiles / slices`` 64-key tiles plus a fixed set-up and merge worth about
    four tiles, and every slice adds a little to the combining pass.  Slice counts in
    ``cluster_sizes`` are combined inside the kernel; the others pay for a second kernel and a
    round trip of the partial results, counted as ten tiles.  The count with the smallest
    ``waves * (tiles per slice + 4) + 0.15 * slices (+ 10)`` is taken.  Clusters of 16 find room
    only a few at a time (one or two to a GPC): they are considered for up to 8 of them, at the
    price of three tiles (one sequence of 32768 keys: 48 -> 33 us; two such sequences are slower
    with 16 slices than with 8).

    Sequences of unequal length (``mean_context`` below three quarters of ``max_context``): a
    row's keys are cut into the slices whatever their number, so the longest row sets the time
    of the slowest CTA, ``longest tiles / slices + 4``, while all CTAs together have
    ``CTAs * (mean tiles + 4 * slices)`` to walk; the larger of the two (the second spread over
    the slots) is minimised instead.  One sequence of 32768 keys among 31 short ones is then cut
    into 8 or 16 slices instead of being walked by one CTA per KV head.
    """
    reps = num_heads // num_kv_heads
    chunks = -(-reps // min(reps, 16))
    ctas = max(1, rows * num_kv_heads * chunks)
    keys = max_context if not window else min(max_context, window)
    tiles = max(1, -(-max(keys, 1) // 64))
    mean_keys = mean_context if mean_context > 0 else max_context
    if window:
        mean_keys = min(mean_keys, window)
    if mean_keys * 4 < keys * 3:
        mean_tiles = max(1.0, mean_keys / 64.0)
        best, best_cost = 1, None
        for ns in ([1] + [n for n in (cluster_sizes or (2, 4, 8)) if n <= tiles]):
            cost = max(-(-tiles // ns) + 4, ctas * (mean_tiles + 4 * ns) / slots) + 0.15 * ns
            if ns > 8:
                cost += 3
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = ns, cost
        return best
    if ctas >= 2 * slots:
        # several rounds of CTAs even without slices: they follow one another without gaps, which
        # the whole waves of the rule below do not know (batch 128 at 2048 keys: 165 us whole, 188 in two)
        return 1
    best, best_cost = 1, None
    for ns in range(1, min(64, tiles) + 1):
        waves = max(1, -(-int(ctas * ns / 1.02) // slots))
        cost = waves * (-(-tiles // ns) + 4) + 0.15 * ns
        if cluster_sizes and ns > 1 and ns not in cluster_sizes:
            cost += 10
        elif ns > 8 and ns in cluster_sizes:
            if ctas > 8:
                continue
            cost += 3
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = ns, cost
    return best


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """First maximum of every row of 32-bit ``logits [R,V]`` into int32 ``out [R]``."""
    _check(logits, "logits", torch.float32, 2)
    _check(out, "out", torch.int32, 1)
    R, V = logits.shape
    call(core(), "ap_argmax", logits.data_ptr(), V, R, V, out.data_ptr(), stream_handle())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor, method: str = "auto") -> None:
    """One token per row: greedy where temperature <= 1e-5, else temperature/top-k/top-p.

    ``method``: "cluster" (eight CTAs hold a row in registers; vocabularies of up to 262144
    entries), "rows" (one CTA per row, any vocabulary) or "auto" (the first where it fits)."""
    _check(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    for t, n, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                     (top_p, "top_p", torch.float32), (uniform, "uniform", torch.float32),
                     (out, "out", torch.int32)):
        _check(t, n, dt, 1)
        if t.shape[0] < R:
            raise KernelError(f"sample: {n} has fewer than {R} entries")
    entry = {"auto": "ap_sample", "cluster": "ap_sample_cluster", "rows": "ap_sample_rows"}.get(method)
    if entry is None:
        raise KernelError(f"sample: unknown method {method!r}")
    call(core(), entry, logits.data_ptr(), V, R, V, temperature.data_ptr(), top_k.data_ptr(),
         top_p.data_ptr(), uniform.data_ptr(), out.data_ptr(), stream_handle())


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """How many K-slices the tensor-core kernel wants for this shape (1: no split)."""
    lib = core()
    if not hasattr(lib, "ap_gemm_tc_plan"):
        return 1
    return max(1, int(lib.ap_gemm_tc_plan(int(M), int(N), int(K))))


def gemm_tc_prefers_dual(M: int, N: int, K: int) -> bool:
    """Whether the kernel with two weight tiles per CTA is the faster one for this shape."""
    lib = core()
    return hasattr(lib, "ap_gemm_tc_prefers_dual") and bool(lib.ap_gemm_tc_prefers_dual(int(M), int(N), int(K)))


def gemm_tc_prefers_pair(M: int, N: int, K: int) -> bool:
    """Whether the kernel that pairs two SMs on a tile is the faster one for this shape (more than 128 rows)."""
    lib = core()
    return hasattr(lib, "ap_gemm_tc_prefers_pair") and bool(lib.ap_gemm_tc_prefers_pair(int(M), int(N), int(K)))


def gemm_tc_prefers_persistent(M: int, N: int, K: int) -> bool:
    """Whether the persistent kernel is the faster one for this shape (more than 64 rows)."""
    lib = core()
    return hasattr(lib, "ap_gemm_tc_prefers_persistent") and \
        bool(lib.ap_gemm_tc_prefers_persistent(int(M), int(N), int(K)))


def gemm_tc_status() -> int:
    """0 while every tensor-core product ran to its end; else the code of the pipeline wait
    that expired.  Synchronises the device."""
    lib = core()
    return int(lib.ap_gemm_tc_status()) if hasattr(lib, "ap_gemm_tc_status") else 0


def check_kernel_status() -> None:
    """Raise if a kernel reported that it gave up (a bounded wait inside it expired)."""
    for hd, lib in list(library._attn.items()):
        if hasattr(lib, "ap_attention_tcgen05_wide_status") and int(lib.ap_attention_tcgen05_wide_status()) > 0:
            raise KernelError(f"the tcgen05 attention kernel with two query tiles (head size {hd}) gave up "
                              "waiting on its pipeline; its results are not valid")
        if hasattr(lib, "ap_attention_tcgen05_status") and int(lib.ap_attention_tcgen05_status()) != 0:
            raise KernelError(f"the tcgen05 attention kernel (head size {hd}) gave up waiting on its pipeline; "
                              f"its results are void")
        if hasattr(lib, "ap_attention_decode_tma_status") and int(lib.ap_attention_decode_tma_status()) != 0:
            raise KernelError(f"the TMA-fed decode attention kernel (head size {hd}) gave up waiting on its "
                              f"pipeline; its results are void")
    lib = core()
    if hasattr(lib, "ap_gemm_tc_pair_status") and int(lib.ap_gemm_tc_pair_status()) != 0:
        raise KernelError(f"the tensor-core matrix product on pairs of SMs gave up waiting (code "
                          f"{int(lib.ap_gemm_tc_pair_status())}: 1 free stage, 2 operands, 3 accumulator, 4 the two "
                          f"CTAs' tensor memory differs); its results are void")
    code = gemm_tc_status()
    if code != 0:
        raise KernelError(f"the tensor-core matrix product gave up waiting (code {code}: "
                          f"1 free stage, 2 operands, 3 accumulator); its results are void")
