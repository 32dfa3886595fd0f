"""Softmax attention whose keys and values may differ in width (`csrc/attention_kv.cu`): the step between the
projections and the scores (per-head rms norm, rotation of interleaved pairs, query temperature, cache store), and the
attention itself with an optional sigmoid gate on its output.

Pages hold the keys of all kv heads and then the values: [NKV, page, DK] + [NKV, page, DV] elements, which for equal
widths is the layout [2, NKV, page, D] of the other attention kernels, so a mixer with DK == DV may prepare here and
attend there.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build, ops
from .build import KernelError

MAX_WIDTH = 256

ops.register_signatures("attention_kv.cu", {
    "mlb_qk_prepare": [c_void_p, c_longlong, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_longlong, c_int, c_longlong,
                       c_void_p, c_void_p, c_float, c_int, c_void_p, c_int, c_float, c_float, c_int, c_void_p, c_void_p, c_void_p,
                       c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "mlb_gate_heads": [c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "mlb_row_norm_columns": [c_void_p, c_longlong, c_int, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_float,
                             c_void_p, c_void_p],
    "mlb_paged_attention_kv": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_longlong, c_int, c_longlong, c_int,
                               c_int, c_void_p, c_float, c_void_p, c_void_p],
})


def sources():
    return [("attention_kv.cu", {})]


def check_widths(dk: int, dv: int) -> None:
    if not (0 < dk <= MAX_WIDTH and 0 < dv <= MAX_WIDTH):
        raise KernelError(f"key width {dk} / value width {dv}: both must be in 1..{MAX_WIDTH}")


def _columns(t: torch.Tensor, name: str):
    """(first plane, row pitch, planes, plane stride) of fp32 rows or their [S, T, N] partial results."""
    ops._need(t, name, torch.float32)
    if t.dim() == 3:
        return t, t.shape[2], t.shape[0], t.shape[1] * t.shape[2]
    if t.dim() != 2:
        raise KernelError(f"{name} must be [T, N] or [S, T, N]")
    return t, t.shape[1], 1, 0


def page_elements(num_kv_heads: int, page_size: int, dk: int, dv: int) -> int:
    return num_kv_heads * page_size * (dk + dv)


def qk_prepare(src: torch.Tensor, q_col: int, k_col: int, v_col: int, *, kv_src: Optional[torch.Tensor] = None,
               q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float, freq: Optional[torch.Tensor],
               rot_dims: int, magnitude: float, q_temp, positions: torch.Tensor, token_seq: torch.Tensor,
               block_table: Optional[torch.Tensor], pages: Optional[torch.Tensor], page_size: int, q_out: torch.Tensor,
               heads: int, kv_heads: int, dk: int, dv: int, error_flag: Optional[torch.Tensor], stored: Optional[int] = None,
               norm: Optional[str] = None, bias: Optional[torch.Tensor] = None) -> None:
    """`norm`: None (rms norm of q and k in front of the rotation when their weights are given, else none), "before" or
    "after" the rotation (a missing weight then means the plain quotient x / rms(x)).
    q, k, v are column blocks (first columns q_col, k_col, v_col) of `src`; k and v of `kv_src` when that is given.
    `q_temp`: None or (coef, every).  `pages` None: only the queries are made.  `stored`: the width every query, key and
    value row is stored with (zeros behind its own elements), for an attention kernel that wants one width for all.
    `bias`: fp32, one per column of `src`, added to q, k and v as they are read (only without `kv_src`)."""
    _, ld, n, stride = _columns(src, "src")
    if bias is not None:
        ops._need(bias, "bias", torch.float32, 1)
        if kv_src is not None or bias.shape[0] != ld:
            raise KernelError("qk_prepare: the bias has one element per column of src (and k, v come from src too)")
    kv_ptr, kv_ld, kv_n, kv_stride = None, 0, 0, 0
    if kv_src is not None:
        _, kv_ld, kv_n, kv_stride = _columns(kv_src, "kv_src")
        kv_ptr = kv_src.data_ptr()
    T = src.shape[-2]
    ops._need(q_out, "q_out", dims=2)
    sk, sv = (stored, stored) if stored else (dk, dv)
    if q_out.shape != (T, heads * sk):
        raise KernelError("qk_prepare: q_out must be [T, heads * (stored) key width]")
    num_pages = max_blocks = 0
    if pages is not None:
        ops._need(block_table, "block_table", torch.int32, 2)
        if pages.numel() % pages.shape[0] or pages.numel() // pages.shape[0] != page_elements(kv_heads, page_size, sk, sv):
            raise KernelError(f"qk_prepare: pages {tuple(pages.shape)} do not match the head geometry")
        num_pages, max_blocks = pages.shape[0], block_table.shape[1]
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    if norm not in (None, "before", "after"):
        raise KernelError(f"qk_prepare: norm {norm!r} is not 'before' or 'after'")
    norm_where = {"before": 1, "after": 2}[norm] if norm else (1 if q_norm is not None and k_norm is not None else 0)
    L = ops.lib("attention_kv.cu")
    build.check(L, L.mlb_qk_prepare(
        src.data_ptr(), ld, n, stride, q_col, k_col, v_col, kv_ptr, kv_ld, kv_n, kv_stride, ops._ptr(q_norm), ops._ptr(k_norm),
        float(eps), norm_where, ops._ptr(freq) if rot_dims else None, int(rot_dims), float(magnitude), coef, every, positions.data_ptr(),
        token_seq.data_ptr(), ops._ptr(block_table), max_blocks, num_pages, page_size, q_out.data_ptr(), ops.dtype_tag(q_out),
        ops._ptr(pages), ops.dtype_tag(pages) if pages is not None else ops.F32, T, heads, kv_heads, dk, dv, sk, sv,
        ops._ptr(bias), ops._ptr(error_flag), ops._stream()))


def row_norm_columns(src: torch.Tensor, out: torch.Tensor, col_a: int, n_a: int, w_a: Optional[torch.Tensor], col_b: int = 0, n_b: int = 0,
                     w_b: Optional[torch.Tensor] = None, eps: float = 1e-6) -> None:
    """out [T, N] fp32 = src (fp32 rows or [S, T, N] partial results, summed in order) with the columns [col_a, col_a + n_a) and
    [col_b, col_b + n_b) each divided by the root mean square over the whole block and multiplied by its weight (fp32, of the
    block's length; None: no weight)."""
    _, ld, n, stride = _columns(src, "src")
    ops._need(out, "out", torch.float32, 2)
    T = src.shape[-2]
    if tuple(out.shape) != (T, ld):
        raise KernelError("row_norm_columns: out must be [T, columns of src]")
    for w, cnt in ((w_a, n_a), (w_b, n_b)):
        if w is not None:
            ops._need(w, "weight", torch.float32, 1)
            if w.shape[0] != cnt:
                raise KernelError("row_norm_columns: a weight has the length of its block of columns")
    L = ops.lib("attention_kv.cu")
    build.check(L, L.mlb_row_norm_columns(src.data_ptr(), ld, n, stride, T, ld, int(col_a), int(n_a), ops._ptr(w_a), int(col_b), int(n_b),
                                          ops._ptr(w_b), float(eps), out.data_ptr(), ops._stream()))


def gate_heads(o: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor], gate_col: int, heads: int, dv: int, stored: int,
               per_head: bool = False) -> None:
    """out[T, heads * dv] = the first dv elements of each head of o[T, heads * stored], times sigmoid(gate columns from
    gate_col of fp32 rows or partial results) when a gate is given: heads * dv gate columns, or `heads` with `per_head`."""
    ops._need(o, "o", dims=2); ops._need(out, "out", dims=2)
    T = o.shape[0]
    if o.shape[1] != heads * stored or out.shape != (T, heads * dv) or o.dtype != out.dtype:
        raise KernelError("gate_heads: shapes do not agree")
    g_ptr, g_ld, g_n, g_stride = None, 0, 1, 0
    if gate is not None:
        _, g_ld, g_n, g_stride = _columns(gate, "gate")
        g_ptr = gate.data_ptr()
    L = ops.lib("attention_kv.cu")
    build.check(L, L.mlb_gate_heads(o.data_ptr(), out.data_ptr(), ops.dtype_tag(o), g_ptr, g_ld, g_n, g_stride, int(gate_col), T, heads,
                                    dv, stored, 1 if per_head else 0, ops._stream()))


def paged_attention_kv(q: torch.Tensor, pages: torch.Tensor, out: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                       block_table: torch.Tensor, page_size: int, heads: int, kv_heads: int, dk: int, dv: int, scale: float,
                       window: Optional[int], gate: Optional[torch.Tensor], gate_col: int,
                       error_flag: Optional[torch.Tensor], chunk: Optional[int] = None, gate_per_head: bool = False,
                       sink: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """`chunk`: a query sees only the keys of its own block of `chunk` positions (blocks counted from position 0).
    `gate_per_head`: the gate has one column per head.  `sink` [heads] fp32: exp(sink) joins each head's denominator.
    `softcap` > 0: scores become softcap * tanh(score / softcap).
    out[T, heads * dv] = softmax(q k^T * scale) v (* sigmoid(gate columns gate_col.. of fp32 rows or partial results))."""
    ops._need(q, "q", dims=2); ops._need(out, "out", dims=2); ops._need(block_table, "block_table", torch.int32, 2)
    T = q.shape[0]
    if q.shape[1] != heads * dk or out.shape != (T, heads * dv):
        raise KernelError("paged_attention_kv: shapes do not agree")
    if pages.numel() // pages.shape[0] != page_elements(kv_heads, page_size, dk, dv):
        raise KernelError(f"paged_attention_kv: pages {tuple(pages.shape)} do not match the head geometry")
    g_ptr, g_ld, g_n, g_stride = None, 0, 1, 0
    if gate is not None:
        _, g_ld, g_n, g_stride = _columns(gate, "gate")
        g_ptr = gate.data_ptr()
    if sink is not None:
        ops._need(sink, "sink", torch.float32, 1)
        if sink.shape[0] != heads:
            raise KernelError("paged_attention_kv: one sink per head")
    L = ops.lib("attention_kv.cu")
    build.check(L, L.mlb_paged_attention_kv(
        q.data_ptr(), ops.dtype_tag(q), pages.data_ptr(), ops.dtype_tag(pages), out.data_ptr(), ops.dtype_tag(out),
        positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], pages.shape[0], page_size, T,
        heads, kv_heads, dk, dv, int(window or 0), int(chunk or 0), float(scale), g_ptr, g_ld, g_n, g_stride, int(gate_col),
        1 if gate_per_head else 0, ops._ptr(sink), float(softcap or 0.0), ops._ptr(error_flag), ops._stream()))
