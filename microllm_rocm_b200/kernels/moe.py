"""Routing of tokens to experts on the device (`csrc/moe.cu`): choice and weights from the router's logits; the list of
(token, choice) pairs sorted by expert; the weighted sum of the experts' results."""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build, ops
from .build import KernelError

SOURCE = "moe.cu"
ops.register_signatures(SOURCE, {
    "mlb_moe_select": [c_void_p, c_longlong, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                       c_int, c_void_p],
    "mlb_moe_align": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "mlb_moe_combine": [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                        c_void_p, c_int, c_void_p, c_int, c_void_p],
})


SCORINGS = {"top_softmax": 0, "softmax_all": 1}


def sources():
    return [(SOURCE, {})]


def select(logits: torch.Tensor, experts: int, bias: Optional[torch.Tensor], top: int, ids: torch.Tensor, weights: torch.Tensor,
           gate_col: int = -1, gate_out: Optional[torch.Tensor] = None, scoring: str = "top_softmax") -> None:
    """logits [T, N] fp32 (or [S, T, N] partial sums of a split product), N >= experts: the router's logits in the first
    `experts` columns, bias [experts] fp32 added here.  ids [T, top] int32 and weights [T, top] fp32 receive the chosen
    experts in order of their logits and the softmax over the chosen logits.  gate_col >= 0 and gate_out [T] fp32:
    sigmoid of that column per token.  `scoring` "softmax_all": s = softmax over all `experts` columns, the choice goes by
    s + bias (a correction that only steers the choice) and the weights are the chosen s, not renormalised."""
    if scoring not in SCORINGS:
        raise KernelError(f"moe.select: scoring {scoring!r} is not one of {', '.join(SCORINGS)}")
    n_partials, stride, first = 1, 0, logits
    if logits.dim() == 3:
        ops._need(logits, "logits", torch.float32, 3)
        n_partials, stride, first = logits.shape[0], logits.shape[1] * logits.shape[2], logits[0]
    ops._need(first, "logits", torch.float32, 2)
    ops._need(ids, "ids", torch.int32, 2); ops._need(weights, "weights", torch.float32, 2)
    T, N = first.shape
    if N < experts or tuple(ids.shape) != (T, top) or tuple(weights.shape) != (T, top) or gate_col >= N:
        raise KernelError("moe.select: shapes do not agree")
    if bias is not None:
        ops._need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != experts:
            raise KernelError("moe.select: one bias per expert")
    if (gate_col >= 0) != (gate_out is not None):
        raise KernelError("moe.select: the gate's column and its output come together")
    if gate_out is not None:
        ops._need(gate_out, "gate_out", torch.float32, 1)
        if gate_out.shape[0] != T:
            raise KernelError("moe.select: one gate per token")
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_moe_select(first.data_ptr(), first.stride(0), n_partials, stride, ops._ptr(bias), int(gate_col), T,
                                    int(experts), int(top), ids.data_ptr(), weights.data_ptr(), ops._ptr(gate_out), SCORINGS[scoring],
                                    ops._stream()))


def align(ids: torch.Tensor, experts: int, offsets: torch.Tensor, sorted_pairs: torch.Tensor,
          error_flag: Optional[torch.Tensor] = None, passthrough: int = 0) -> None:
    """ids [T, top] -> offsets [experts + 1], sorted_pairs [T * top] (indices t * top + j grouped by expert).  Ids in
    [experts, experts + passthrough) are choices without an expert: they are left out of the list (offsets[experts] then
    counts fewer pairs than T * top)."""
    ops._need(ids, "ids", torch.int32); ops._need(offsets, "offsets", torch.int32, 1)
    ops._need(sorted_pairs, "sorted_pairs", torch.int32, 1)
    if offsets.shape[0] != experts + 1 or sorted_pairs.shape[0] != ids.numel():
        raise KernelError("moe.align: shapes do not agree")
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_moe_align(ids.data_ptr(), ids.numel(), int(experts), offsets.data_ptr(), sorted_pairs.data_ptr(),
                                   ops._ptr(error_flag), int(passthrough), ops._stream()))


def combine(y: torch.Tensor, weights: torch.Tensor, out: torch.Tensor, shared: Optional[torch.Tensor] = None,
            gate: Optional[torch.Tensor] = None, col_scale: Optional[torch.Tensor] = None, ids: Optional[torch.Tensor] = None,
            experts: int = 0, x: Optional[torch.Tensor] = None) -> None:
    """out[t] = (sum_j weights[t, j] * y[t * top + j] + gate[t] * shared[t]) * col_scale; shared may be [S, T, W]
    partial sums.  With `ids` [T, top], `experts` and `x` [T, W]: a choice whose id is `experts` or more has no expert
    behind it and adds weights[t, j] * x[t] instead of a row of y."""
    ops._need(y, "y", torch.float32, 2); ops._need(weights, "weights", torch.float32, 2); ops._need(out, "out", torch.float32, 2)
    T, top = weights.shape
    W = out.shape[1]
    if out.shape[0] != T or tuple(y.shape) != (T * top, W):
        raise KernelError("moe.combine: shapes do not agree")
    n_shared, stride = 0, 0
    if shared is not None:
        n_shared, stride = ops._partials(shared, out.shape, "moe.combine shared")
    for name, t, n in (("gate", gate, T), ("col_scale", col_scale, W)):
        if t is not None:
            ops._need(t, name, torch.float32, 1)
            if t.shape[0] != n:
                raise KernelError(f"moe.combine: {name} has the wrong length")
    if ids is not None:
        ops._need(ids, "ids", torch.int32, 2); ops._need(x, "x", dims=2)
        if tuple(ids.shape) != (T, top) or tuple(x.shape) != (T, W):
            raise KernelError("moe.combine: ids are [T, top] and x is [T, W]")
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_moe_combine(y.data_ptr(), weights.data_ptr(), ops._ptr(shared), n_shared, stride, ops._ptr(gate),
                                     ops._ptr(col_scale), out.data_ptr(), T, W, top, ops._ptr(ids), int(experts), ops._ptr(x),
                                     ops.dtype_tag(x) if x is not None else ops.F32, ops._stream()))
