"""Kernels around a linear recurrence with a decay per key channel (`csrc/linear_attention.cu`): the blend of every token's
input with the previous token's, what enters the recurrence (q, k, v gathered, the decay made from a two-step narrow
projection), and the per-head norm and gate of its result.  The recurrence itself is `recurrent.linear_scan`."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build, ops
from .attention_kv import _columns
from .build import KernelError

MAX_WIDTH = 256
DECAY_FORMS = {"sigmoid_root": 0, "double_exp": 1}
GATE_ACTS = {"sigmoid": 0, "silu": 1}

ops.register_signatures("linear_attention.cu", {
    "mlb_token_shift": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                        c_int, c_void_p, c_void_p],
    "mlb_token_shift_state": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    "mlb_decay_prepare": [c_void_p, c_longlong, c_int, c_longlong, c_int, c_void_p, c_longlong, c_int, c_longlong, c_int,
                          c_void_p, c_longlong, c_int, c_longlong, c_int, c_float, c_void_p, c_longlong, c_int, c_longlong, c_int,
                          c_int, c_int, c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_void_p, c_int, c_float, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "mlb_head_norm_gate": [c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_longlong, c_int, c_int, c_void_p, c_int, c_int,
                           c_int, c_int, c_float, c_void_p],
    "mlb_lightning_prepare": [c_void_p, c_longlong, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_void_p],
    "mlb_row_norm_gate": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
})


def sources():
    return [("linear_attention.cu", {}), ("delta_rule.cu", {})]


def token_shift(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, ctx, out: torch.Tensor,
                update_state: bool = True) -> None:
    """out[s, t] = x[t] + (x[t-1] - x[t]) * mu[s] for every blend s; x[t-1] of a sequence's first token of the step is its
    row of `state` [slots, width] fp32 (zeros at position 0), which then moves on to the step's last token."""
    ops._need(x, "x", dims=2); ops._need(mu, "mu", torch.float32, 2); ops._need(state, "state", torch.float32, 2)
    T, W = x.shape
    if mu.shape[1] != W or state.shape[1] != W or tuple(out.shape) != (mu.shape[0], T, W) or out.dtype != x.dtype or not out.is_contiguous():
        raise KernelError("token_shift: shapes do not agree")
    L = ops.lib("linear_attention.cu")
    build.check(L, L.mlb_token_shift(x.data_ptr(), ops.dtype_tag(x), mu.data_ptr(), state.data_ptr(), slots.data_ptr(), state.shape[0],
                                     ctx.seq_starts.data_ptr(), ctx.seq_pos0.data_ptr(), ctx.token_seq.data_ptr(), out.data_ptr(), T, W,
                                     mu.shape[0], ops._ptr(ctx.error_flag), ops._stream()))
    if update_state:
        build.check(L, L.mlb_token_shift_state(x.data_ptr(), ops.dtype_tag(x), state.data_ptr(), slots.data_ptr(), state.shape[0],
                                               ctx.seq_starts.data_ptr(), ctx.num_seqs, W, ops._stream()))


def decay_prepare(q_src, q_col: int, k_src, k_col: int, v_src, v_col: int, q_scale: float, *, narrow=None, a_col: int = 0,
                  w2: Optional[torch.Tensor] = None, narrow_act: Optional[str] = None, pre=None, bias: Optional[torch.Tensor],
                  form: str, tau: float = 1.0, q_out: torch.Tensor, k_out: torch.Tensor, v_out: torch.Tensor, decay: torch.Tensor) -> None:
    """q_out = q * q_scale, k_out = k, v_out = v (column blocks of fp32 rows or of K-split partial results) and
    decay = f(W2 act(a) + bias) per (token, head, key channel): f "sigmoid_root": sigmoid(z)^(1/tau), "double_exp":
    exp(-exp(z)).  W2 act(a) is `pre` when a product made it, else made here from the `narrow` columns from a_col and `w2`."""
    if form not in DECAY_FORMS:
        raise KernelError(f"decay_prepare: form {form!r} is not one of {', '.join(DECAY_FORMS)}")
    if (pre is None) == (narrow is None or w2 is None):
        raise KernelError("decay_prepare: either the second projection's result, or its weight and the narrow input")
    T, HK, HV = q_out.shape[0], q_out.shape[1], v_out.shape[1]
    for name, t, shape in (("q_out", q_out, (T, HK)), ("k_out", k_out, (T, HK)), ("v_out", v_out, (T, HV)), ("decay", decay, (T, HK))):
        ops._need(t, name, torch.float32, 2)
        if tuple(t.shape) != shape:
            raise KernelError(f"decay_prepare: {name} must be {shape}")

    def cols(t, what, width, col):
        if t is None:
            return None, 0, 1, 0
        _, ld, n, stride = _columns(t, what)
        if t.shape[-2] != T or col < 0 or col + width > ld:
            raise KernelError(f"decay_prepare: {what} has no columns {col}..{col + width}")
        return t.data_ptr(), ld, n, stride
    rank = w2.shape[1] if w2 is not None else 0
    if w2 is not None:
        ops._need(w2, "w2", torch.float32, 2)
        if w2.shape[0] != HK:
            raise KernelError("decay_prepare: w2 must be [heads * key width, rank]")
    if bias is not None:
        ops._need(bias, "bias", torch.float32, 1)
    L = ops.lib("linear_attention.cu")
    build.check(L, L.mlb_decay_prepare(*cols(q_src, "q", HK, q_col), q_col, *cols(k_src, "k", HK, k_col), k_col, *cols(v_src, "v", HV, v_col), v_col,
                                       float(q_scale), *cols(narrow if pre is None else None, "narrow", rank, a_col), a_col, rank,
                                       1 if narrow_act == "tanh" else 0, ops._ptr(w2) if pre is None else None, *cols(pre, "pre", HK, 0),
                                       ops._ptr(bias), DECAY_FORMS[form], float(tau), q_out.data_ptr(), k_out.data_ptr(), v_out.data_ptr(),
                                       decay.data_ptr(), T, HK, HV, ops._stream()))


def head_norm_gate(o: torch.Tensor, weight: Optional[torch.Tensor], gate, gate_col: int, gate_act: str, out: torch.Tensor, heads: int,
                   dv: int, eps: float) -> None:
    """out = o / rms(o) per head * weight * act(gate columns from gate_col) in out's dtype; `weight` [dv] (shared by the
    heads), [heads * dv] or None; `gate` fp32 rows or partial results, or None."""
    ops._need(o, "o", torch.float32, 2); ops._need(out, "out", dims=2)
    T = o.shape[0]
    if o.shape != (T, heads * dv) or out.shape != o.shape or not 0 < dv <= MAX_WIDTH:
        raise KernelError("head_norm_gate: shapes do not agree")
    if gate_act not in GATE_ACTS:
        raise KernelError(f"head_norm_gate: gate activation {gate_act!r}")
    per_head = 0
    if weight is not None:
        ops._need(weight, "weight", torch.float32, 1)
        if weight.shape[0] not in (dv, heads * dv):
            raise KernelError("head_norm_gate: the weight must have dv or heads * dv elements")
        per_head = 1 if weight.shape[0] == heads * dv and heads > 1 else 0
    g_ptr, g_ld, g_n, g_stride = None, 0, 1, 0
    if gate is not None:
        _, g_ld, g_n, g_stride = _columns(gate, "gate")
        g_ptr = gate.data_ptr()
    L = ops.lib("linear_attention.cu")
    build.check(L, L.mlb_head_norm_gate(o.data_ptr(), ops._ptr(weight), per_head, g_ptr, g_ld, g_n, g_stride, int(gate_col),
                                        GATE_ACTS[gate_act], out.data_ptr(), ops.dtype_tag(out), T, heads, dv, float(eps), ops._stream()))


def lightning_prepare(proj, q_col: int, k_col: int, v_col: int, head_decay: torch.Tensor, q_out: torch.Tensor, k_out: torch.Tensor,
                      v_out: torch.Tensor, decay: torch.Tensor, heads: int, dk: int, dv: int) -> None:
    """q_out, k_out [T, heads * dk], v_out [T, heads * dv] = silu of the column blocks of `proj` (fp32 rows or partial results)
    from q_col, k_col, v_col; decay [T, heads * dk] = head_decay[head] (fp32 [heads]) for every key channel of the head."""
    _, ld, n, stride = _columns(proj, "proj")
    T = proj.shape[-2]
    ops._need(head_decay, "head_decay", torch.float32, 1)
    for name, t, shape in (("q_out", q_out, (T, heads * dk)), ("k_out", k_out, (T, heads * dk)), ("decay", decay, (T, heads * dk)),
                           ("v_out", v_out, (T, heads * dv))):
        ops._need(t, name, torch.float32, 2)
        if tuple(t.shape) != shape:
            raise KernelError(f"lightning_prepare: {name} must be {shape}")
    if head_decay.shape[0] != heads or max(q_col, k_col) + heads * dk > ld or v_col + heads * dv > ld:
        raise KernelError("lightning_prepare: shapes do not agree")
    L = ops.lib("linear_attention.cu")
    build.check(L, L.mlb_lightning_prepare(proj.data_ptr(), ld, n, stride, int(q_col), int(k_col), int(v_col), head_decay.data_ptr(),
                                           q_out.data_ptr(), k_out.data_ptr(), v_out.data_ptr(), decay.data_ptr(), T, heads, dk, dv, ops._stream()))


def row_norm_gate(o: torch.Tensor, weight: Optional[torch.Tensor], gate, gate_col: int, out: torch.Tensor, eps: float) -> None:
    """out = o / rms(o) over the whole row * weight * sigmoid(gate columns from gate_col) in out's dtype; `weight` [width] fp32
    or None; `gate` fp32 rows or partial results, or None."""
    ops._need(o, "o", torch.float32, 2); ops._need(out, "out", dims=2)
    T, width = o.shape
    if tuple(out.shape) != (T, width):
        raise KernelError("row_norm_gate: shapes do not agree")
    if weight is not None:
        ops._need(weight, "weight", torch.float32, 1)
        if weight.shape[0] != width:
            raise KernelError("row_norm_gate: the weight has the row's length")
    g_ptr, g_ld, g_n, g_stride = None, 0, 1, 0
    if gate is not None:
        _, g_ld, g_n, g_stride = _columns(gate, "gate")
        g_ptr = gate.data_ptr()
        if gate_col + width > g_ld:
            raise KernelError("row_norm_gate: the gate has no such columns")
    L = ops.lib("linear_attention.cu")
    build.check(L, L.mlb_row_norm_gate(o.data_ptr(), ops._ptr(weight), g_ptr, g_ld, g_n, g_stride, int(gate_col), out.data_ptr(),
                                       ops.dtype_tag(out), T, width, float(eps), ops._stream()))
