"""Kernels of mixers that carry a fixed-size state per sequence: the short causal convolution over time
(`csrc/short_conv.cu`) and the gated delta rule (`csrc/delta_rule.cu`).  All of it is fp32 arithmetic on fp32 inputs;
only the last kernel of the delta rule writes the compute dtype."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build, ops
from .attention_kv import _columns
from .build import KernelError

MAX_TAPS = 17
MAX_WIDTH = 256

ops.register_signatures("short_conv.cu", {
    "mlb_short_conv": [c_void_p, c_longlong, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "mlb_short_conv_state": [c_void_p, c_longlong, c_int, c_longlong, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                             c_int, c_void_p],
})
ops.register_signatures("delta_rule.cu", {
    "mlb_delta_prepare": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_longlong, c_int, c_int, c_void_p, c_void_p, c_longlong,
                          c_int, c_longlong, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "mlb_take_columns": [c_void_p, c_longlong, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p],
    "mlb_linear_scan": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "mlb_delta_scan": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                       c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "mlb_delta_output": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_int, c_void_p, c_void_p, c_longlong, c_int,
                         c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
})


def conv_sources():
    return [("short_conv.cu", {})]


def delta_sources():
    return [("delta_rule.cu", {})]


def short_conv(u: torch.Tensor, col0: int, weight: torch.Tensor, state: Optional[torch.Tensor], slots: torch.Tensor, ctx,
               out: torch.Tensor, silu: bool, update_state: bool = True) -> None:
    """out[t, c] = act(sum_j weight[c, j] * u[t - taps + 1 + j, col0 + c]) over the time of each sequence of the step
    `ctx`; inputs before the step come from `state` [slots, taps - 1, C] (zero before position 0).  Then the state
    moves on to hold the step's last inputs (unless `update_state` is False: a run that reads another run's state)."""
    _, ld, n, stride = _columns(u, "u")
    ops._need(weight, "weight", torch.float32, 2); ops._need(out, "out", torch.float32, 2)
    C, taps = weight.shape
    T = u.shape[-2]
    if out.shape != (T, C) or col0 < 0 or col0 + C > ld or not 1 <= taps <= MAX_TAPS:
        raise KernelError("short_conv: shapes do not agree")
    num_slots = 1
    if taps > 1:
        ops._need(state, "state", torch.float32, 3)
        if tuple(state.shape[1:]) != (taps - 1, C):
            raise KernelError(f"short_conv: the state must be [slots, {taps - 1}, {C}], got {tuple(state.shape)}")
        num_slots = state.shape[0]
    L = ops.lib("short_conv.cu")
    build.check(L, L.mlb_short_conv(u.data_ptr(), ld, n, stride, col0, weight.data_ptr(), ops._ptr(state), slots.data_ptr(), num_slots,
                                    ctx.seq_starts.data_ptr(), ctx.seq_pos0.data_ptr(), ctx.token_seq.data_ptr(), out.data_ptr(),
                                    out.shape[1], T, ctx.num_seqs, C, taps, 1 if silu else 0, ops._ptr(ctx.error_flag), ops._stream()))
    if taps > 1 and update_state:
        build.check(L, L.mlb_short_conv_state(u.data_ptr(), ld, n, stride, col0, state.data_ptr(), slots.data_ptr(), num_slots,
                                              ctx.seq_starts.data_ptr(), ctx.num_seqs, C, taps, ops._stream()))


def _pre(pre: Optional[torch.Tensor], T: int, width: int, what: str):
    if pre is None:
        return None, 0, 1, 0
    _, ld, n, stride = _columns(pre, what)
    if pre.shape[-2] != T or ld != width:
        raise KernelError(f"{what} must be [T, {width}] or its partial results")
    return pre.data_ptr(), ld, n, stride


def take_columns(src: torch.Tensor, col0: int, out: torch.Tensor, activation: Optional[str] = None) -> None:
    """out[t, c] = act(src[t, col0 + c]), `src` fp32 rows or their [S, T, N] partial results (summed), in out's dtype;
    `activation` None or "tanh"."""
    if activation not in (None, "tanh"):
        raise KernelError(f"take_columns: activation {activation!r}")
    _, ld, n, stride = _columns(src, "src")
    ops._need(out, "out", dims=2)
    if out.shape[0] != src.shape[-2] or col0 < 0 or col0 + out.shape[1] > ld:
        raise KernelError("take_columns: shapes do not agree")
    L = ops.lib("delta_rule.cu")
    build.check(L, L.mlb_take_columns(src.data_ptr(), ld, n, stride, col0, out.shape[1], out.shape[0], out.data_ptr(),
                                      ops.dtype_tag(out), 1 if activation == "tanh" else 0, ops._stream()))


def delta_prepare(qkv: torch.Tensor, proj: torch.Tensor, beta_col: int, a_col: int, w2: Optional[torch.Tensor], dt_bias: torch.Tensor,
                  a_log: torch.Tensor, qn: torch.Tensor, kn: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, heads: int,
                  kv_heads: int, dk: int, pre: Optional[torch.Tensor] = None) -> None:
    """Unit-vector q (times dk^-1/2) and k per kv head from the first 2 * kv_heads * dk columns of `qkv`; per head
    beta = sigmoid(proj[:, beta_col + h]) and the decay g = exp(-exp(a_log[h]) * softplus(w2 proj[:, a_col:] + dt_bias)).
    `pre` [T, heads * dk] (or partial results): w2 proj[:, a_col:] already made by a product; else it is made here."""
    ops._need(qkv, "qkv", torch.float32, 2)
    _, ld, n, stride = _columns(proj, "proj")
    T = qkv.shape[0]
    if (w2 is None) == (pre is None):
        raise KernelError("delta_prepare: either the second projection's weight or its result")
    rank = w2.shape[-1] if w2 is not None else 1
    pre_args = _pre(pre, T, heads * dk, "delta_prepare pre")
    for name, t, shape in ((("w2", w2, (heads * dk, rank)),) if w2 is not None else ()) + (("dt_bias", dt_bias, (heads * dk,)), ("a_log", a_log, (heads,)),
                           ("qn", qn, (T, kv_heads * dk)), ("kn", kn, (T, kv_heads * dk)), ("g", g, (T, heads * dk)),
                           ("beta", beta, (T, heads))):
        ops._need(t, name, torch.float32)
        if tuple(t.shape) != shape:
            raise KernelError(f"delta_prepare: {name} must be {shape}, got {tuple(t.shape)}")
    L = ops.lib("delta_rule.cu")
    build.check(L, L.mlb_delta_prepare(qkv.data_ptr(), qkv.shape[1], proj.data_ptr(), ld, n, stride, beta_col, a_col, ops._ptr(w2),
                                       *pre_args, dt_bias.data_ptr(), a_log.data_ptr(), qn.data_ptr(), kn.data_ptr(), g.data_ptr(),
                                       beta.data_ptr(), T, heads, kv_heads, dk, rank, ops._stream()))


def delta_scan(qn: torch.Tensor, kn: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, v: torch.Tensor, o: torch.Tensor,
               state: torch.Tensor, slots: torch.Tensor, ctx, heads: int, kv_heads: int, dk: int, dv: int) -> None:
    """The recurrence over the step's tokens; `v` is a column view [T, heads * dv] (row pitch v.stride(0)) of fp32 rows,
    `state` [slots, heads, dk, dv] fp32."""
    ops._need(state, "state", torch.float32, 4); ops._need(o, "o", torch.float32, 2)
    if tuple(state.shape[1:]) != (heads, dk, dv) or v.dtype != torch.float32 or v.stride(1) != 1 or o.shape != (v.shape[0], heads * dv):
        raise KernelError("delta_scan: shapes do not agree")
    L = ops.lib("delta_rule.cu")
    build.check(L, L.mlb_delta_scan(qn.data_ptr(), kn.data_ptr(), g.data_ptr(), beta.data_ptr(), v.data_ptr(), v.stride(0),
                                    o.data_ptr(), state.data_ptr(), slots.data_ptr(), state.shape[0], ctx.seq_starts.data_ptr(),
                                    ctx.seq_pos0.data_ptr(), ctx.num_seqs, heads, kv_heads, dk, dv, ops._ptr(ctx.error_flag),
                                    ops._stream()))


def delta_output(o: torch.Tensor, weight: torch.Tensor, proj: torch.Tensor, g_col: int, w2: Optional[torch.Tensor], out: torch.Tensor,
                 heads: int, dv: int, eps: float, pre: Optional[torch.Tensor] = None) -> None:
    """out = o / rms(o) per head * weight * sigmoid(w2 proj[:, g_col:g_col + rank]) in out's dtype; `pre` as in delta_prepare."""
    ops._need(o, "o", torch.float32, 2); ops._need(weight, "weight", torch.float32, 1)
    ops._need(out, "out", dims=2)
    _, ld, n, stride = _columns(proj, "proj")
    T = o.shape[0]
    if (w2 is None) == (pre is None):
        raise KernelError("delta_output: either the second projection's weight or its result")
    if w2 is not None:
        ops._need(w2, "w2", torch.float32, 2)
    rank = w2.shape[1] if w2 is not None else 1
    pre_args = _pre(pre, T, heads * dv, "delta_output pre")
    if o.shape != (T, heads * dv) or out.shape != o.shape or weight.shape[0] != dv or (w2 is not None and w2.shape[0] != heads * dv):
        raise KernelError("delta_output: shapes do not agree")
    L = ops.lib("delta_rule.cu")
    build.check(L, L.mlb_delta_output(o.data_ptr(), weight.data_ptr(), proj.data_ptr(), ld, n, stride, g_col, ops._ptr(w2), *pre_args,
                                      out.data_ptr(), ops.dtype_tag(out), T, heads, dv, rank, float(eps), ops._stream()))


RULES = {"decayed_sum": 1, "bonus_read": 2}


def linear_scan(rule: str, q: torch.Tensor, k: torch.Tensor, decay: torch.Tensor, v: torch.Tensor, o: torch.Tensor, state: torch.Tensor,
                slots: torch.Tensor, ctx, heads: int, dk: int, dv: int, bonus: Optional[torch.Tensor] = None) -> None:
    """A recurrence with one decay per head and key channel over the step's tokens, per head with S [dk, dv]:
      "decayed_sum":  S <- diag(decay_t) S + k_t v_t^T;  o_t = S^T q_t
      "bonus_read":   o_t = (S + diag(bonus) k_t v_t^T)^T q_t;  then S <- diag(decay_t) S + k_t v_t^T
    q, k, decay [T, heads * dk] and v, o [T, heads * dv] fp32; `state` [slots, heads, dk, dv] fp32 (taken as zero for a
    sequence that starts at position 0); `bonus` [heads, dk]."""
    if rule not in RULES:
        raise KernelError(f"linear_scan: rule {rule!r} is not one of {', '.join(RULES)}")
    T = q.shape[0]
    for name, t, shape in (("q", q, (T, heads * dk)), ("k", k, (T, heads * dk)), ("decay", decay, (T, heads * dk)),
                           ("v", v, (T, heads * dv)), ("o", o, (T, heads * dv))):
        ops._need(t, name, torch.float32, 2)
        if tuple(t.shape) != shape:
            raise KernelError(f"linear_scan: {name} must be {shape}, got {tuple(t.shape)}")
    ops._need(state, "state", torch.float32, 4)
    if tuple(state.shape[1:]) != (heads, dk, dv):
        raise KernelError(f"linear_scan: the state must be [slots, {heads}, {dk}, {dv}], got {tuple(state.shape)}")
    if rule == "bonus_read":
        ops._need(bonus, "bonus", torch.float32, 2)
        if tuple(bonus.shape) != (heads, dk):
            raise KernelError(f"linear_scan: bonus must be [{heads}, {dk}]")
    L = ops.lib("delta_rule.cu")
    build.check(L, L.mlb_linear_scan(RULES[rule], q.data_ptr(), k.data_ptr(), decay.data_ptr(), ops._ptr(bonus), v.data_ptr(), v.stride(0),
                                     o.data_ptr(), state.data_ptr(), slots.data_ptr(), state.shape[0], ctx.seq_starts.data_ptr(),
                                     ctx.seq_pos0.data_ptr(), ctx.num_seqs, heads, heads, dk, dv, ops._ptr(ctx.error_flag), ops._stream()))
