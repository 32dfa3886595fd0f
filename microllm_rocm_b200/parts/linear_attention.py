"""Two linear-attention mixers whose state is one matrix per head, decayed per key channel (no softmax, no cache that
grows with the tokens):

`gated_linear_attention`
  q = Wq x * dim^-1/2,  k = Wk x  (heads x dim),  v = Wv x  (heads x vdim)
  a = f(Wa2 (Wa1 x) + bias) per head and key channel, f = sigmoid(.)^(1/tau)
  per head, S [dim, vdim] from zero:  S <- diag(a_t) S + k_t v_t^T;  o_t = S^T q_t
  o / rms(o) per head * weight (one row of vdim, shared by the heads) * silu(Wg x),  then Wo
  Every projection that reads x (q, k, v, g, a1) is one fused product.

`token_shift_wkv`
  every projection reads its own blend of the token's input and the previous token's:  x_s = x_t + (x_(t-1) - x_t) * mu_s
  for s in r, k, v, g, w (x_(-1) = 0);  r, k, v = Wr x_r, Wk x_k, Wv x_v  (heads x dim each),  gate = silu(Wg x_g)
  w = exp(-exp(Ww2 tanh(Ww1 x_w) + w0)) per head and key channel
  per head:  o_t = (S + diag(u) k_t v_t^T)^T r_t  (the bonus u for the present token only);  then S <- diag(w_t) S + k_t v_t^T
  o / rms(o) per head * weight (heads x dim) * gate,  then Wo.  The previous token's x is part of the state.

`lightning_attention`
  q, k = silu(Wq x), silu(Wk x)  (heads x dim),  v = silu(Wv x)  (heads x vdim);  one FIXED decay per head, a constant d_h
  per head, S [dim, vdim] from zero:  S <- d_h S + k_t v_t^T;  o_t = S^T q_t  (no other scale)
  the heads side by side are divided by their root mean square TOGETHER, times a weight of heads x vdim, times
  sigmoid(Wg x) element by element, then Wo.  q, k, v and the gate are one fused product.

The second step of the narrow projection (Wa2, Ww2) runs as a product when its inner width suits the product kernels
(a multiple of 8), else inside the kernel that needs its result, in fp32.  Decays, their exponentials, the recurrence,
its state and the output norm are fp32 whatever the compute dtype.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import gemm_bf16, linear_attention, recurrent
from ..kernels.linear import linear
from .base import CompositeNeed, FixedStateNeed, Mixer, PositionEncoding, Runtime, StepContext, WeightSpec, register_mixer


def _check_widths(kind: str, dk: int, dv: int) -> None:
    if not (0 < dk <= recurrent.MAX_WIDTH and 0 < dv <= recurrent.MAX_WIDTH):
        raise ValueError(f"{kind}: widths {dk}/{dv} must be in 1..{recurrent.MAX_WIDTH}")


@register_mixer("gated_linear_attention")
class GatedLinearAttention(Mixer):
    graph_safe = True

    def __init__(self, params: dict, rt: Runtime, position: Optional[PositionEncoding] = None):
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.nh = int(params["num_heads"])
        self.dk, self.dv = int(params["dim"]), int(params["vdim"])
        self.a_rank = int(params["a_rank"])
        self.tau = float(params["tau"])
        self.eps = float(params.get("eps", 1e-6))
        self.q_scale = float(params.get("q_scale", self.dk ** -0.5))
        _check_widths("gated_linear_attention", self.dk, self.dv)
        if not self.tau > 0:
            raise ValueError("gated_linear_attention: tau must be positive")
        names = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", gate="g_proj.weight", o="o_proj.weight",
                     a1="a_proj.0.weight", a2="a_proj.1.weight", a_bias="a_proj.1.bias", norm="o_norm.weight")
        names.update(params.get("names", {}))
        self.names = names
        self.rt = rt
        # columns of the fused input projection: q | k | v | gate | a1
        self.qk_cols, self.v_cols = self.nh * self.dk, self.nh * self.dv
        self.k_col, self.v_col = self.qk_cols, 2 * self.qk_cols
        self.g_col = self.v_col + self.v_cols
        self.a_col = self.g_col + self.v_cols
        self.in_rows = self.a_col + self.a_rank
        self.a_product = self.a_rank % 8 == 0
        self.w_in = self.w_o = self.w_a2 = self.a_bias = self.norm_w = None

    def cache_need(self):
        return CompositeNeed((("state", FixedStateNeed((self.nh, self.dk, self.dv), torch.float32)),))

    def _pieces(self):
        n = self.names
        return [(n["q"], 0), (n["k"], self.k_col), (n["v"], self.v_col), (n["gate"], self.g_col), (n["a1"], self.a_col)]

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, W = self.names, self.hidden
        return {n["q"]: WeightSpec((self.qk_cols, W)), n["k"]: WeightSpec((self.qk_cols, W)), n["v"]: WeightSpec((self.v_cols, W)),
                n["gate"]: WeightSpec((self.v_cols, W)), n["a1"]: WeightSpec((self.a_rank, W)),
                n["a2"]: WeightSpec((self.qk_cols, self.a_rank), role="matrix" if self.a_product else "vector", init=("normal", 0.1)),
                n["a_bias"]: WeightSpec((self.qk_cols,), role="vector", init=("normal", 0.5)),
                n["norm"]: WeightSpec((self.dv,), role="vector", init=("one_plus_normal", 0.1)),
                n["o"]: WeightSpec((W, self.v_cols))}

    def fused_tensors(self):
        return {"in_proj.weight": (WeightSpec((self.in_rows, self.hidden)), self._pieces())}

    def kernel_sources(self):
        own = linear_attention.sources()
        return own if self.rt.is_fp32 else own + gemm_bf16.sources(engine_only=True)

    def bind(self, tensors):
        n = self.names
        self.w_in = tensors["in_proj.weight"] if "in_proj.weight" in tensors else torch.cat([tensors[name] for name, _ in self._pieces()], 0).contiguous()
        self.w_a2, self.a_bias, self.norm_w, self.w_o = tensors[n["a2"]], tensors[n["a_bias"]], tensors[n["norm"]], tensors[n["o"]]

    def replay_key(self):
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None
        return ("gated_linear_attention", self.hidden, self.nh, self.dk, self.dv, self.a_rank, self.tau, self.eps, self.q_scale)

    def own_tensors(self):
        return [self.w_in, self.w_o, self.w_a2, self.a_bias, self.norm_w]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        T, flag, f32 = x.shape[0], ctx.error_flag, torch.float32
        state = cache["state"]
        buf = lambda role, shape, dtype=f32: ctx.buffer("gla." + role, shape, dtype)
        proj = linear(x, self.w_in, None, f32, partials_ok=True, error_flag=flag, alloc=lambda shape, dtype: buf("proj", shape, dtype))
        pre = None
        if self.a_product:
            narrow = buf("a", (T, self.a_rank), self.rt.dtype)
            recurrent.take_columns(proj, self.a_col, narrow)
            pre = linear(narrow, self.w_a2, None, f32, partials_ok=True, error_flag=flag, alloc=lambda shape, dtype: buf("a_pre", shape, dtype))
        q, k, decay = buf("q", (T, self.qk_cols)), buf("k", (T, self.qk_cols)), buf("decay", (T, self.qk_cols))
        v = buf("v", (T, self.v_cols))
        linear_attention.decay_prepare(proj, 0, proj, self.k_col, proj, self.v_col, self.q_scale, pre=pre,
                                       narrow=None if self.a_product else proj, a_col=self.a_col, w2=None if self.a_product else self.w_a2,
                                       bias=self.a_bias, form="sigmoid_root", tau=self.tau, q_out=q, k_out=k, v_out=v, decay=decay)
        o = buf("o", (T, self.v_cols))
        recurrent.linear_scan("decayed_sum", q, k, decay, v, o, state.storage, state.slots, ctx, self.nh, self.dk, self.dv)
        gated = buf("gated", (T, self.v_cols), self.rt.dtype)
        linear_attention.head_norm_gate(o, self.norm_w, proj, self.g_col, "silu", gated, self.nh, self.dv, self.eps)
        return linear(gated, self.w_o, None, f32, partials_ok=True, error_flag=flag, alloc=lambda shape, dtype: buf("out", shape, dtype))


@register_mixer("lightning_attention")
class LightningAttention(Mixer):
    graph_safe = True

    def __init__(self, params: dict, rt: Runtime, position: Optional[PositionEncoding] = None):
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.nh = int(params["num_heads"])
        self.dk, self.dv = int(params["dim"]), int(params["vdim"])
        self.decay_values = tuple(float(d) for d in params["decay"])
        self.eps = float(params.get("eps", 1e-6))
        _check_widths("lightning_attention", self.dk, self.dv)
        if len(self.decay_values) != self.nh:
            raise ValueError("lightning_attention: one decay per head")
        names = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", gate="g_proj.weight", o="o_proj.weight", norm="o_norm.weight")
        names.update(params.get("names", {}))
        self.names = names
        self.rt = rt
        # columns of the fused input projection: q | k | v | gate
        self.qk_cols, self.v_cols = self.nh * self.dk, self.nh * self.dv
        self.k_col, self.v_col = self.qk_cols, 2 * self.qk_cols
        self.g_col = self.v_col + self.v_cols
        self.in_rows = self.g_col + self.v_cols
        self.head_decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)     # a constant of the design, not a weight
        self.w_in = self.w_o = self.norm_w = None

    def cache_need(self):
        return CompositeNeed((("state", FixedStateNeed((self.nh, self.dk, self.dv), torch.float32)),))

    def _pieces(self):
        n = self.names
        return [(n["q"], 0), (n["k"], self.k_col), (n["v"], self.v_col), (n["gate"], self.g_col)]

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, W = self.names, self.hidden
        return {n["q"]: WeightSpec((self.qk_cols, W)), n["k"]: WeightSpec((self.qk_cols, W)), n["v"]: WeightSpec((self.v_cols, W)),
                n["gate"]: WeightSpec((self.v_cols, W)), n["norm"]: WeightSpec((self.v_cols,), role="vector", init=("one_plus_normal", 0.1)),
                n["o"]: WeightSpec((W, self.v_cols))}

    def fused_tensors(self):
        return {"in_proj.weight": (WeightSpec((self.in_rows, self.hidden)), self._pieces())}

    def kernel_sources(self):
        own = linear_attention.sources()
        return own if self.rt.is_fp32 else own + gemm_bf16.sources(engine_only=True)

    def bind(self, tensors):
        n = self.names
        self.w_in = tensors["in_proj.weight"] if "in_proj.weight" in tensors else torch.cat([tensors[name] for name, _ in self._pieces()], 0).contiguous()
        self.norm_w, self.w_o = tensors[n["norm"]], tensors[n["o"]]

    def replay_key(self):
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None
        return ("lightning_attention", self.hidden, self.nh, self.dk, self.dv, self.decay_values, self.eps)

    def own_tensors(self):
        return [self.w_in, self.w_o, self.norm_w]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        T, flag, f32 = x.shape[0], ctx.error_flag, torch.float32
        state = cache["state"]
        buf = lambda role, shape, dtype=f32: ctx.buffer("lightning." + role, shape, dtype)
        proj = linear(x, self.w_in, None, f32, partials_ok=True, error_flag=flag, alloc=lambda shape, dtype: buf("proj", shape, dtype))
        q, k, decay = buf("q", (T, self.qk_cols)), buf("k", (T, self.qk_cols)), buf("decay", (T, self.qk_cols))
        v = buf("v", (T, self.v_cols))
        linear_attention.lightning_prepare(proj, 0, self.k_col, self.v_col, self.head_decay, q, k, v, decay, self.nh, self.dk, self.dv)
        o = buf("o", (T, self.v_cols))
        recurrent.linear_scan("decayed_sum", q, k, decay, v, o, state.storage, state.slots, ctx, self.nh, self.dk, self.dv)
        gated = buf("gated", (T, self.v_cols), self.rt.dtype)
        linear_attention.row_norm_gate(o, self.norm_w, proj, self.g_col, gated, self.eps)
        return linear(gated, self.w_o, None, f32, partials_ok=True, error_flag=flag, alloc=lambda shape, dtype: buf("out", shape, dtype))


@register_mixer("token_shift_wkv")
class TokenShiftWKV(Mixer):
    graph_safe = True
    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, params: dict, rt: Runtime, position: Optional[PositionEncoding] = None):
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.nh, self.d = int(params["num_heads"]), int(params["dim"])
        self.w_rank = int(params["w_rank"])
        self.eps = float(params.get("eps", 1e-6))
        _check_widths("token_shift_wkv", self.d, self.d)
        names = dict(r="r_proj.weight", k="k_proj.weight", v="v_proj.weight", g="g_proj.weight", o="o_proj.weight", w1="w_proj.0.weight",
                     w2="w_proj.1.weight", w0="w_bias", u="bonus", norm="o_norm.weight", mu_r="mix.r", mu_k="mix.k", mu_v="mix.v",
                     mu_g="mix.g", mu_w="mix.w")
        names.update(params.get("names", {}))
        self.names = names
        self.rt = rt
        self.cols = self.nh * self.d
        self.w_product = self.w_rank % 8 == 0
        self.mu = self.w_r = self.w_k = self.w_v = self.w_g = self.w_w1 = self.w_w2 = self.w0 = self.u = self.norm_w = self.w_o = None

    def cache_need(self):
        return CompositeNeed((("state", FixedStateNeed((self.nh, self.d, self.d), torch.float32)),
                              ("shift", FixedStateNeed((self.hidden,), torch.float32))))

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, W, C = self.names, self.hidden, self.cols
        specs = {n["mu_" + s]: WeightSpec((W,), role="vector", init=("normal", 0.3)) for s in self.BLENDS}
        specs.update({n[s]: WeightSpec((C, W)) for s in ("r", "k", "v", "g")})
        specs.update({n["w1"]: WeightSpec((self.w_rank, W)),
                      n["w2"]: WeightSpec((C, self.w_rank), role="matrix" if self.w_product else "vector", init=("normal", 0.1)),
                      n["w0"]: WeightSpec((C,), role="vector", init=("normal", 0.5)),
                      n["u"]: WeightSpec((self.nh, self.d), role="vector", init=("normal", 0.5)),
                      n["norm"]: WeightSpec((C,), role="vector", init=("one_plus_normal", 0.1)),
                      n["o"]: WeightSpec((W, C))})
        return specs

    def kernel_sources(self):
        own = linear_attention.sources()
        return own if self.rt.is_fp32 else own + gemm_bf16.sources(engine_only=True)

    def bind(self, tensors):
        n = self.names
        self.mu = torch.stack([tensors[n["mu_" + s]] for s in self.BLENDS], 0).contiguous()       # [5, W] fp32
        self.w_r, self.w_k, self.w_v, self.w_g = (tensors[n[s]] for s in ("r", "k", "v", "g"))
        self.w_w1, self.w_w2, self.w0, self.u = tensors[n["w1"]], tensors[n["w2"]], tensors[n["w0"]], tensors[n["u"]]
        self.norm_w, self.w_o = tensors[n["norm"]], tensors[n["o"]]

    def replay_key(self):
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None
        return ("token_shift_wkv", self.hidden, self.nh, self.d, self.w_rank, self.eps)

    def own_tensors(self):
        return [self.mu, self.w_r, self.w_k, self.w_v, self.w_g, self.w_w1, self.w_w2, self.w0, self.u, self.norm_w, self.w_o]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        T, flag, f32, C = x.shape[0], ctx.error_flag, torch.float32, self.cols
        state, shift = cache["state"], cache["shift"]
        buf = lambda role, shape, dtype=f32: ctx.buffer("wkv." + role, shape, dtype)
        blends = buf("blends", (len(self.BLENDS), T, self.hidden), self.rt.dtype)
        linear_attention.token_shift(x, self.mu, shift.storage, shift.slots, ctx, blends, update_state=shift.writable)
        product = lambda i, w, role: linear(blends[i], w, None, f32, partials_ok=True, error_flag=flag,
                                            alloc=lambda shape, dtype: buf(role, shape, dtype))
        r, k, v, g = product(0, self.w_r, "r"), product(1, self.w_k, "k"), product(2, self.w_v, "v"), product(3, self.w_g, "g")
        a = product(4, self.w_w1, "w1")
        pre = None
        if self.w_product:
            narrow = buf("w_narrow", (T, self.w_rank), self.rt.dtype)
            recurrent.take_columns(a, 0, narrow, activation="tanh")
            pre = linear(narrow, self.w_w2, None, f32, partials_ok=True, error_flag=flag, alloc=lambda shape, dtype: buf("w_pre", shape, dtype))
        rs, ks, vs, decay = buf("rs", (T, C)), buf("ks", (T, C)), buf("vs", (T, C)), buf("decay", (T, C))
        linear_attention.decay_prepare(r, 0, k, 0, v, 0, 1.0, pre=pre, narrow=None if self.w_product else a, a_col=0,
                                       w2=None if self.w_product else self.w_w2, narrow_act="tanh", bias=self.w0, form="double_exp",
                                       q_out=rs, k_out=ks, v_out=vs, decay=decay)
        o = buf("o", (T, C))
        recurrent.linear_scan("bonus_read", rs, ks, decay, vs, o, state.storage, state.slots, ctx, self.nh, self.d, self.d, bonus=self.u)
        gated = buf("gated", (T, C), self.rt.dtype)
        linear_attention.head_norm_gate(o, self.norm_w, g, 0, "silu", gated, self.nh, self.d, self.eps)
        return linear(gated, self.w_o, None, f32, partials_ok=True, error_flag=flag, alloc=lambda shape, dtype: buf("out", shape, dtype))
