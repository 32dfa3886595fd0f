"""Grouped-query attention over the paged cache.

  q, k, v = x Wq^T + bq, x Wk^T + bk, x Wv^T + bv      one fused product (the reference runs
                                                       three: src/model/model.cpp:457-476)
  q, k rotated by the position encoding's table; k, v stored into this run's pages
  head h attends with kv head h // (NH/NKV) over keys lo..pos, scale 1/sqrt(D) after the dot
  out = concat_heads(o) Wo^T

All sizes are parameters; `window` (keys visible, itself included) is per layer and may be
None.  The part never learns which layer or model it belongs to.  Formulas:
src/model/model.cpp:447-523 (prefill), :525-603 (decode); scale at :513-514.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..kernels import attention as attention_kernels
from ..kernels import gemm_bf16, ops
from ..kernels.linear import linear
from .base import Mixer, PagedKVNeed, PagedKVView, PositionEncoding, Runtime, StepContext, WeightSpec, register_mixer


ROPE_TABLE_MIN_TOKENS = 64          # from here on a step-wide table of sines and cosines pays
SHARED_KERNEL_WIDTHS = (32, 64, 128, 256)   # head sizes at which the tensor-core attention kernels of one width are built and tested


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, params: dict, rt: Runtime, position: Optional[PositionEncoding] = None):
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        self.qkv_bias = bool(params.get("qkv_bias", False))
        self.out_bias = bool(params.get("out_bias", False))
        self.window = params.get("window")
        self.scale = float(params.get("scale", 1.0 / math.sqrt(float(self.d))))
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        attention_kernels.check_head_dim(self.d)
        self.rt = rt
        self.rotary = position.rotary_table(self.d) if position is not None else None
        if self.rotary is not None and self.rotary.magnitude != 1.0:
            raise ValueError("this mixer's rotation kernels take plain cosines and sines; use `normed_attention` for a stretched table")
        if self.rotary is None:        # no rotation: an empty table makes the kernel pass q/k through
            self._no_rot = torch.zeros(0, dtype=torch.float32, device=rt.device)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    # --- declarations -----------------------------------------------------------------
    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        q, kv = self.nh * self.d, self.nkv * self.d
        specs = {"q_proj.weight": WeightSpec((q, self.hidden)), "k_proj.weight": WeightSpec((kv, self.hidden)),
                 "v_proj.weight": WeightSpec((kv, self.hidden)), "o_proj.weight": WeightSpec((self.hidden, q))}
        if self.qkv_bias:
            specs.update({"q_proj.bias": WeightSpec((q,), role="vector"), "k_proj.bias": WeightSpec((kv,), role="vector"),
                          "v_proj.bias": WeightSpec((kv,), role="vector")})
        if self.out_bias:
            specs["o_proj.bias"] = WeightSpec((self.hidden,), role="vector")
        return specs

    def fused_tensors(self):
        q, kv = self.nh * self.d, self.nkv * self.d
        fused = {"qkv_proj.weight": (WeightSpec((q + 2 * kv, self.hidden)),
                                     [("q_proj.weight", 0), ("k_proj.weight", q), ("v_proj.weight", q + kv)])}
        if self.qkv_bias:
            fused["qkv_proj.bias"] = (WeightSpec((q + 2 * kv,), role="vector"),
                                      [("q_proj.bias", 0), ("k_proj.bias", q), ("v_proj.bias", q + kv)])
        return fused

    def bind(self, tensors):
        # the loader hands over the fused tensors; a caller with the checkpoint's pieces gets them joined here
        if "qkv_proj.weight" in tensors:
            self.w_qkv = tensors["qkv_proj.weight"]
            self.b_qkv = tensors.get("qkv_proj.bias") if self.qkv_bias else None
        else:
            self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], 0).contiguous()
            if self.qkv_bias:
                self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]], 0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        self.b_o = tensors.get("o_proj.bias")

    def kernel_sources(self):
        if self.rt.is_fp32:
            return []
        return (gemm_bf16.sources(engine_only=True) + attention_kernels.mma_sources(self.d)
                + attention_kernels.tc_sources(self.d))

    def replay_key(self):
        if self.out_bias:
            return None                  # a bias on the output projection is added by a tensor-framework operation
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None                  # the library product would go through the tensor framework
        rotary = None if self.rotary is None else (self.rotary.inv_freq.data_ptr(), self.rotary.rotary_dim, self.rotary.interleaved)
        return ("attention", self.hidden, self.nh, self.nkv, self.d, self.qkv_bias, self.window, self.scale, rotary)

    def own_tensors(self):
        return [self.w_qkv, self.b_qkv, self.w_o]

    # --- launch plans frozen into a captured decode step ----------------------------------
    def plan_stale(self, ctx: StepContext, max_seq_len: int) -> bool:
        from ..kernels.device import sm_count
        return attention_kernels.decode_plan_stale(ctx, max_seq_len, sm_count(self.rt.device))

    def forget_plans(self, ctx: StepContext) -> None:
        attention_kernels.forget_plans(ctx)

    def plan_group(self):
        return ("attention", self.rt.device)          # the kernels' plans are kept per (group size, kv heads), for all layers

    # --- compute ------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: PagedKVView) -> torch.Tensor:
        T = x.shape[0]
        q = ctx.buffer("attention.q", (T, self.nh * self.d), self.rt.dtype)
        inv_freq, rot, inter = ((self.rotary.inv_freq, self.rotary.rotary_dim, self.rotary.interleaved)
                                if self.rotary is not None else (self._no_rot, 0, False))
        pages = cache.pages if cache.writable else None
        if (x.dtype == torch.bfloat16 and gemm_bf16.gemv_preferred(x, self.w_qkv)
                and gemm_bf16.gemv_fused_supported(x, self.w_qkv) and self.d % 16 == 0
                and (rot == 0 or (rot == self.d and not inter))):
            # a few tokens: projection, bias, rotation and the cache store in one weight-streaming kernel
            gemm_bf16.gemv_qkv_rope(x, self.w_qkv, self.b_qkv, ctx.positions, ctx.token_seq, cache.block_table,
                                    inv_freq if rot else None, q, pages, self.nh, self.nkv, self.d, ctx.error_flag)
        else:
            qkv = linear(x, self.w_qkv, None, torch.float32, partials_ok=True,    # [T, (NH+2NKV)*D] f32, or its partial sums
                         alloc=lambda shape, dtype: ctx.buffer("attention.qkv", shape, dtype), error_flag=ctx.error_flag)
            cos_sin = None
            if rot and T >= ROPE_TABLE_MIN_TOKENS and x.dtype == torch.bfloat16:
                # a prompt portion: the step's sines and cosines are made once and serve every layer and head
                # (a result of this step's positions: it lives in step_values, which every forward starts empty,
                # so a context that outlives its step -- a captured decode step -- never reads old angles)
                key = ("rope_table", id(self.rotary))
                cos_sin = ctx.step_values.get(key)
                if cos_sin is None:
                    table = ctx.buffer("attention.rope_table", (T, rot // 2, 2), torch.float32)
                    cos_sin = ctx.step_values[key] = ops.rope_table(ctx.positions, inv_freq, out=table)
            ops.rope_kv_write(qkv, self.b_qkv, ctx.positions, ctx.token_seq, cache.block_table, inv_freq, rot, inter,
                              q, pages, self.nh, self.nkv, self.d, ctx.error_flag, cos_sin)
        o = ctx.buffer("attention.o", (T, self.nh * self.d), self.rt.dtype)
        attention_kernels.paged_attention(q, cache.pages, o, ctx, cache.block_table, self.nh, self.nkv, self.d,
                                          self.scale, self.window,
                                          beside_mma_products=x.dtype == torch.bfloat16 and gemm_bf16.gemv_preferred(x, self.w_o))
        return linear(o, self.w_o, self.b_o, torch.float32, partials_ok=True, error_flag=ctx.error_flag,      # [T, H] f32, or its partial sums
                      alloc=lambda shape, dtype: ctx.buffer("attention.out", shape, dtype))


@register_mixer("normed_attention")
class NormedAttention(Mixer):
    """Grouped-query softmax attention with the steps some designs put between projection and scores, each an option:

      q, k, v = Wq x, Wk x, Wv x          `values="keys"`: there is no Wv and v is k AS PROJECTED (before norm and rotation)
      short causal convolution over time on every channel of q, k, v (`conv` taps > 1; weights [channels, taps], the last
          column is the current token's; the last taps - 1 projected rows of a sequence are kept in its state slot)
      per-head rms norm of q and k with one weight each, shared by the heads (`qk_norm`; `qk_norm_weight=False`: the
          plain quotient x / rms(x), no tensors; `qk_norm_where="after"`: behind the rotation instead of in front of it)
      rotation of the first `rotary_dim` elements of every head by the position encoding's table, in interleaved
          pairs (2i, 2i + 1), cosines and sines times the table's magnitude (a split-half table is refused)
      q times 1 + coef * ln(floor((p + 1) / every) + 1) at position p (`q_temp = (coef, every)`)
      score = q . k * scale, causal (optionally the last `window` keys; optionally only the keys of the query's own
          block of `chunk` positions, blocks counted from position 0 of the sequence), softmax
      concat_heads(o) * sigmoid(Wg x) (`gate`; `gate="head"`: Wg has one row per head and a head's whole output is multiplied
          by its one number), then Wo

    Further options: `bias` (q and k projections have biases, added as the projection is read; values that are the projected
    keys carry the key's bias), `qk_norm="row"` (q and k are each divided by the root mean square of their WHOLE projection
    row, before the split into heads, times a weight of the row's length), `softcap` (score <- cap * tanh(score / cap)),
    `sink` ("learned": one number per head whose exponential joins the softmax's denominator, with no key and no value,
    neither scaled nor capped; "zero": the same with the number fixed at 0, i.e. 1 is added to the denominator), and
    `kv_shared` (the layer has no key and value projections of its own: its run reads the pages another run wrote, with its
    own queries).

    Keys have `dim` elements per head and values `vdim`; the cache holds both widths (`PagedKVNeed.value_dim`).  All
    projections that read x are one fused product; norm, rotation, temperature, softmax and the gate are fp32.
    """
    graph_safe = True

    def __init__(self, params: dict, rt: Runtime, position: Optional[PositionEncoding] = None):
        from ..kernels import attention_kv
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.nh, self.nkv = int(params["num_heads"]), int(params["num_kv_heads"])
        self.dk, self.dv = int(params["dim"]), int(params.get("vdim", params["dim"]))
        self.scale = float(params.get("scale", 1.0 / math.sqrt(float(self.dk))))
        self.eps = float(params.get("eps", 1e-6))
        self.values = params.get("values", "projected")
        self.taps = int(params.get("conv", 1))
        self.has_gate = bool(params.get("gate", False))
        self.gate_per_head = params.get("gate") == "head"
        self.row_norm = params.get("qk_norm") == "row"
        self.qk_norm = bool(params.get("qk_norm", True)) and not self.row_norm
        self.has_bias = bool(params.get("bias", False))
        self.softcap = float(params["softcap"]) if params.get("softcap") else None
        self.sink_kind = params.get("sink")
        if self.sink_kind not in (None, "learned", "zero"):
            raise ValueError(f"normed_attention: sink {self.sink_kind!r} is not 'learned' or 'zero'")
        self.kv_shared = bool(params.get("kv_shared", False))
        self.q_temp = tuple(params["q_temp"]) if params.get("q_temp") else None
        self.window = params.get("window")
        self.chunk = int(params["chunk"]) if params.get("chunk") else None
        self.norm_weight = bool(params.get("qk_norm_weight", True))
        self.norm_where = params.get("qk_norm_where", "before")
        if self.norm_where not in ("before", "after"):
            raise ValueError(f"normed_attention: qk_norm_where {self.norm_where!r} is not 'before' or 'after'")
        if self.chunk is not None and self.chunk <= 0:
            raise ValueError("normed_attention: chunk must be positive")
        if self.values not in ("projected", "keys"):
            raise ValueError(f"normed_attention: values {self.values!r} is not 'projected' or 'keys'")
        if self.values == "keys" and self.dv != self.dk:
            raise ValueError("normed_attention: values that are the projected keys have the keys' width")
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        attention_kv.check_widths(self.dk, self.dv)
        if self.kv_shared and (self.taps > 1 or self.values == "keys"):
            raise ValueError("normed_attention: a layer that reads another layer's keys and values has no convolution and no value rule of its own")
        if self.has_bias and self.taps > 1:
            raise ValueError("normed_attention: biases and a convolution do not go together")
        names = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight", q_norm="q_norm.weight",
                     k_norm="k_norm.weight", gate="g_proj.weight", q_conv="q_conv.weight", k_conv="k_conv.weight",
                     v_conv="v_conv.weight", q_bias="q_proj.bias", k_bias="k_proj.bias", sink="sink")
        names.update(params.get("names", {}))
        self.names = names
        self.rt = rt
        table = position.rotary_table(self.dk) if position is not None else None
        if table is not None and not table.interleaved:
            raise ValueError("normed_attention turns interleaved pairs (2i, 2i + 1)")
        self.freq = table.inv_freq if table is not None else None
        self.rot_dims = table.rotary_dim if table is not None else 0
        self.magnitude = table.magnitude if table is not None else 1.0
        # columns of the fused input projection: q | k | v (if projected) | gate (if any)
        self.q_cols, self.k_cols = self.nh * self.dk, (0 if self.kv_shared else self.nkv * self.dk)
        self.v_cols = self.nkv * self.dv if self.values == "projected" and not self.kv_shared else 0
        self.g_cols = (self.nh if self.gate_per_head else self.nh * self.dv) if self.has_gate else 0
        self.conv_cols = self.q_cols + self.k_cols + self.v_cols
        # bf16: the attention itself runs on the tensor-core kernels of equal key and value widths; unequal widths are
        # stored with zeros up to one width that those kernels take (the plain kernel with the true widths otherwise,
        # and always in fp32, where every kernel is a plain one)
        self.stored = None
        if not rt.is_fp32:
            self.stored = next((w for w in SHARED_KERNEL_WIDTHS if w >= max(self.dk, self.dv)), None)
        if self.stored is not None and not attention_kernels.extras_supported(self.stored, self.softcap, self.sink_kind is not None):
            self.stored = None           # a cap or a sink that the kernels of one width do not take: the plain kernel
        self.w_in = self.w_o = self.q_norm_w = self.k_norm_w = self.w_conv = self.b_in = self.sink = None
        # rows of the fused projection; a gate of one row per head is padded to a multiple of 8 rows, which the products like
        self.in_rows = -(-(self.conv_cols + self.g_cols) // 8) * 8 if self.gate_per_head else self.conv_cols + self.g_cols

    # --- declarations -----------------------------------------------------------------
    def cache_need(self):
        from .base import CompositeNeed, FixedStateNeed
        kv = PagedKVNeed(self.nkv, self.dk, self.window, value_dim=self.dv) if self.stored is None else PagedKVNeed(self.nkv, self.stored, self.window)
        if self.taps <= 1:
            return kv
        return CompositeNeed((("kv", kv), ("conv", FixedStateNeed((self.taps - 1, self.conv_cols), torch.float32))))

    def _pieces(self):
        n = self.names
        pieces = [(n["q"], 0)] + ([] if self.kv_shared else [(n["k"], self.q_cols)])
        if self.v_cols:
            pieces.append((n["v"], self.q_cols + self.k_cols))
        if self.has_gate:
            pieces.append((n["gate"], self.conv_cols))
        return pieces

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        specs = {n["q"]: WeightSpec((self.q_cols, self.hidden)), n["o"]: WeightSpec((self.hidden, self.nh * self.dv))}
        if not self.kv_shared:
            specs[n["k"]] = WeightSpec((self.k_cols, self.hidden))
        if self.has_bias:
            specs[n["q_bias"]] = WeightSpec((self.q_cols,), role="vector", init=("normal", 0.1))
            if not self.kv_shared:
                specs[n["k_bias"]] = WeightSpec((self.k_cols,), role="vector", init=("normal", 0.1))
        if self.row_norm:
            specs[n["q_norm"]] = WeightSpec((self.q_cols,), role="vector", init=("one_plus_normal", 0.1))
            if not self.kv_shared:
                specs[n["k_norm"]] = WeightSpec((self.k_cols,), role="vector", init=("one_plus_normal", 0.1))
        if self.sink_kind == "learned":
            specs[n["sink"]] = WeightSpec((self.nh,), role="vector", init=("normal", 1.0))
        if self.v_cols:
            specs[n["v"]] = WeightSpec((self.v_cols, self.hidden))
        if self.has_gate:
            specs[n["gate"]] = WeightSpec((self.g_cols, self.hidden))
        if self.qk_norm and self.norm_weight:
            specs[n["q_norm"]] = WeightSpec((self.dk,), role="vector", init=("one_plus_normal", 0.1))
            specs[n["k_norm"]] = WeightSpec((self.dk,), role="vector", init=("one_plus_normal", 0.1))
        if self.taps > 1:
            for key, cols in (("q_conv", self.q_cols), ("k_conv", self.k_cols), ("v_conv", self.v_cols)):
                if cols:
                    specs[n[key]] = WeightSpec((cols, self.taps), role="vector", init=("normal", 0.5))
        return specs

    def fused_tensors(self):
        fused = {"in_proj.weight": (WeightSpec((self.in_rows, self.hidden)), self._pieces())}
        if self.has_bias:
            n = self.names
            fused["in_proj.bias"] = (WeightSpec((self.in_rows,), role="vector"),
                                     [(n["q_bias"], 0)] + ([] if self.kv_shared else [(n["k_bias"], self.q_cols)]))
        if self.taps > 1:
            n = self.names
            rows = [(n["q_conv"], 0), (n["k_conv"], self.q_cols)] + ([(n["v_conv"], self.q_cols + self.k_cols)] if self.v_cols else [])
            fused["conv.weight"] = (WeightSpec((self.conv_cols, self.taps), role="vector"), rows)
        return fused

    def kernel_sources(self):
        from ..kernels import attention_kv, recurrent
        own = attention_kv.sources() + (recurrent.conv_sources() if self.taps > 1 else [])
        if self.rt.is_fp32:
            return own
        own += gemm_bf16.sources(engine_only=True)
        if self.stored is not None:
            own += attention_kernels.mma_sources(self.stored) + attention_kernels.tc_sources(self.stored)
        return own

    def bind(self, tensors):
        n = self.names
        used = self.conv_cols + self.g_cols
        if "in_proj.weight" in tensors:
            self.w_in = tensors["in_proj.weight"]
            self.w_in[used:].zero_()                     # the padding rows: their columns of the product are never read
        else:
            pieces = [tensors[name] for name, _ in self._pieces()]
            if self.in_rows > used:
                pieces.append(torch.zeros((self.in_rows - used, self.hidden), dtype=pieces[0].dtype, device=pieces[0].device))
            self.w_in = torch.cat(pieces, 0).contiguous()
        if self.has_bias:
            if "in_proj.bias" in tensors:
                self.b_in = tensors["in_proj.bias"]
                self.b_in[self.q_cols + self.k_cols:].zero_()           # only q and k have biases
            else:
                self.b_in = torch.zeros((self.in_rows,), dtype=torch.float32, device=self.w_in.device)
                self.b_in[:self.q_cols] = tensors[n["q_bias"]]
                if not self.kv_shared:
                    self.b_in[self.q_cols:self.q_cols + self.k_cols] = tensors[n["k_bias"]]
        if self.sink_kind == "learned":
            self.sink = tensors[n["sink"]]
        elif self.sink_kind == "zero":
            self.sink = torch.zeros((self.nh,), dtype=torch.float32, device=self.w_in.device)
        if self.row_norm:
            self.q_norm_w = tensors[n["q_norm"]]
            self.k_norm_w = None if self.kv_shared else tensors[n["k_norm"]]
        if self.taps > 1:
            if "conv.weight" in tensors:
                self.w_conv = tensors["conv.weight"]
            else:
                keys = ["q_conv", "k_conv"] + (["v_conv"] if self.v_cols else [])
                self.w_conv = torch.cat([tensors[n[k]] for k in keys], 0).contiguous()
        self.w_o = tensors[n["o"]]
        if not self.row_norm:
            self.q_norm_w = tensors[n["q_norm"]] if self.qk_norm and self.norm_weight else None
            self.k_norm_w = tensors[n["k_norm"]] if self.qk_norm and self.norm_weight else None

    def replay_key(self):
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None
        rotary = None if self.freq is None else (self.freq.data_ptr(), self.rot_dims, self.magnitude)
        return ("normed_attention", self.hidden, self.nh, self.nkv, self.dk, self.dv, self.scale, self.eps, self.values, self.taps,
                self.has_gate, self.qk_norm, self.norm_weight, self.norm_where, self.q_temp, self.window, self.chunk, rotary,
                self.gate_per_head, self.row_norm, self.has_bias, self.softcap, self.sink_kind, self.kv_shared)

    def own_tensors(self):
        return [self.w_in, self.w_o, self.q_norm_w, self.k_norm_w, self.w_conv, self.b_in, self.sink if self.sink_kind == "learned" else None]

    def _shared_kernels(self, page_size: int) -> bool:
        """Whether the attention itself runs on the kernels of equal key and value widths."""
        return self.stored is not None and attention_kernels.mma_supported(self.stored, page_size)

    def plan_stale(self, ctx: StepContext, max_seq_len: int) -> bool:
        from ..kernels.device import sm_count
        return attention_kernels.decode_plan_stale(ctx, max_seq_len, sm_count(self.rt.device))

    def forget_plans(self, ctx: StepContext) -> None:
        attention_kernels.forget_plans(ctx)

    def plan_group(self):
        return ("attention", self.rt.device)

    # --- compute ------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        from ..kernels import attention_kv, recurrent
        T, dt, flag = x.shape[0], self.rt.dtype, ctx.error_flag
        kv_view = cache["kv"] if isinstance(cache, dict) else cache
        proj = linear(x, self.w_in, None, torch.float32, partials_ok=True, error_flag=flag,
                      alloc=lambda shape, dtype: ctx.buffer("normed_attention.proj", shape, dtype))
        src, q_col, k_col = proj, 0, self.q_cols
        v_col = self.q_cols + self.k_cols if self.v_cols else k_col
        if self.row_norm:
            # q and k divided by the root mean square of their whole rows; the partial results become plain rows on the way
            src = ctx.buffer("normed_attention.rows", (T, self.in_rows), torch.float32)
            attention_kv.row_norm_columns(proj, src, 0, self.q_cols, self.q_norm_w, self.q_cols, self.k_cols, self.k_norm_w, self.eps)
            proj = src
        if self.taps > 1:
            state = cache["conv"]
            src = ctx.buffer("normed_attention.conv", (T, self.conv_cols), torch.float32)
            recurrent.short_conv(proj, 0, self.w_conv, state.storage, state.slots, ctx, src, silu=False, update_state=state.writable)
        sk = self.stored or self.dk
        sv = self.stored or self.dv
        q = ctx.buffer("normed_attention.q", (T, self.nh * sk), dt)
        head_norms = (None, None) if self.row_norm else (self.q_norm_w, self.k_norm_w)       # the rows' norm has been applied above
        attention_kv.qk_prepare(src, q_col, k_col, v_col, q_norm=head_norms[0], k_norm=head_norms[1], eps=self.eps, freq=self.freq,
                                rot_dims=self.rot_dims, magnitude=self.magnitude, q_temp=self.q_temp, positions=ctx.positions,
                                token_seq=ctx.token_seq, block_table=kv_view.block_table,
                                pages=kv_view.pages if kv_view.writable and not self.kv_shared else None, page_size=kv_view.page_size, q_out=q,
                                heads=self.nh, kv_heads=self.nkv, dk=self.dk, dv=self.dv, error_flag=flag, stored=self.stored,
                                norm=self.norm_where if self.qk_norm else None, bias=self.b_in)
        o = ctx.buffer("normed_attention.o", (T, self.nh * self.dv), dt)
        gate = proj if self.has_gate else None
        if self._shared_kernels(kv_view.page_size):
            wide = o if (sv == self.dv and gate is None) else ctx.buffer("normed_attention.o_stored", (T, self.nh * sv), dt)
            attention_kernels.paged_attention(q, kv_view.pages, wide, ctx, kv_view.block_table, self.nh, self.nkv, sk, self.scale,
                                              self.window, beside_mma_products=gemm_bf16.gemv_preferred(x, self.w_o), chunk=self.chunk,
                                              sink=self.sink, softcap=self.softcap or 0.0)
            if wide is not o:
                attention_kv.gate_heads(wide, o, gate, self.conv_cols, self.nh, self.dv, sv, per_head=self.gate_per_head)
        elif self.stored is not None and self.sink is None and not self.softcap:
            # a page size the tensor-core kernels do not take: the plain kernel of one width
            wide = ctx.buffer("normed_attention.o_stored", (T, self.nh * sv), dt)
            attention_kernels.paged_attention(q, kv_view.pages, wide, ctx, kv_view.block_table, self.nh, self.nkv, sk, self.scale, self.window,
                                              chunk=self.chunk)
            attention_kv.gate_heads(wide, o, gate, self.conv_cols, self.nh, self.dv, sv, per_head=self.gate_per_head)
        elif self.stored is not None:
            # the same with a sink or a cap: the plain kernel of two widths, told that both are the stored one
            wide = ctx.buffer("normed_attention.o_stored", (T, self.nh * sv), dt)
            attention_kv.paged_attention_kv(q, kv_view.pages, wide, ctx.positions, ctx.token_seq, kv_view.block_table, kv_view.page_size,
                                            self.nh, self.nkv, sk, sv, self.scale, self.window, None, 0, flag, chunk=self.chunk,
                                            sink=self.sink, softcap=self.softcap or 0.0)
            attention_kv.gate_heads(wide, o, gate, self.conv_cols, self.nh, self.dv, sv, per_head=self.gate_per_head)
        else:
            attention_kv.paged_attention_kv(q, kv_view.pages, o, ctx.positions, ctx.token_seq, kv_view.block_table, kv_view.page_size,
                                            self.nh, self.nkv, self.dk, self.dv, self.scale, self.window, gate, self.conv_cols, flag,
                                            chunk=self.chunk, gate_per_head=self.gate_per_head, sink=self.sink, softcap=self.softcap or 0.0)
        return linear(o, self.w_o, None, torch.float32, partials_ok=True, error_flag=flag,
                      alloc=lambda shape, dtype: ctx.buffer("normed_attention.out", shape, dtype))
