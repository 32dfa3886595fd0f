"""Routed experts: every token runs `top` of `experts` small gated feed-forwards and adds their results up.

  z = Wr x + b                       fp32 (one product with the shared gate's row stacked under the router's)
  chosen = the `top` largest z;  w = softmax over the chosen z only
  y = sum_j w_j * down_e(silu(gate_e x) * up_e x)          e = chosen_j
  y += sigmoid(Wsg x) * shared(x)    a shared expert of the same form that every token runs (optional, its gate too)

`scoring="softmax_all"`: s = softmax(z) over ALL router outputs; the `top` largest s + correction are chosen (the correction,
a tensor named by `router_bias_name`, only steers the choice) and the weights are the chosen s themselves, not renormalised.
`identity` = n: the router has experts + n outputs, and the last n have no expert behind them: a token that chooses one gets
its own input back, times the weight.

Nothing is counted on the host: the router writes the choices, a kernel sorts the (token, choice) pairs by expert,
and two grouped products (`kernels/grouped.py`) walk the sorted list, so the part is safe to capture.  The experts'
matrices live stacked on the device ([E, 2 ff, W] gate over up, and [E, W, ff]); the loader streams every expert's
pieces straight into their rows.  The shared expert is the ordinary gated feed-forward part under its own prefix.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import gemm_bf16, grouped, moe
from ..kernels.linear import linear
from .base import FEED_FORWARDS, FeedForward, Runtime, StepContext, WeightSpec, make, register_feed_forward, scratch


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    scales_output = True          # forward(..., out_scale=) multiplies the result per column

    def __init__(self, params: dict, rt: Runtime):
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.inter = int(params["expert_size"])
        if not 0 < self.top <= self.experts + int(params.get("identity", 0)):
            raise ValueError(f"routed experts: top {self.top} of {self.experts + int(params.get('identity', 0))}")
        # local names: expert e's matrices are expert_names[i].format(e); router, its bias, the shared expert's gate row
        self.expert_names = tuple(params.get("expert_names", ("experts.{}.gate_proj.weight", "experts.{}.up_proj.weight",
                                                              "experts.{}.down_proj.weight")))
        self.n_router = params.get("router_name", "router.weight")
        self.n_router_bias = params.get("router_bias_name")            # None: no bias
        self.scoring = params.get("scoring", "top_softmax")
        if self.scoring not in moe.SCORINGS:
            raise ValueError(f"routed experts: scoring {self.scoring!r} is not one of {', '.join(moe.SCORINGS)}")
        self.identity = int(params.get("identity", 0))                 # router outputs behind the experts' that pass the input on
        if self.identity < 0:
            raise ValueError("routed experts: identity must not be negative")
        self.outputs = self.experts + self.identity                    # what the router chooses among
        self.shared = None
        self.shared_prefix = ""
        self.n_shared_gate = None
        shared = params.get("shared")
        if shared is not None:                                         # a PartSpec of a feed-forward
            self.shared = make(FEED_FORWARDS, "feed-forward", shared, rt)
            self.shared_prefix = shared.params.get("prefix", "")
            self.n_shared_gate = params.get("shared_gate_name")        # None: the shared expert is added ungated
        self.rt = rt
        # the router's rows and (behind them) the shared gate's row are ONE matrix on the device, its rows padded to a
        # multiple of 8: one product gives every logit
        self.has_gate = self.shared is not None and self.n_shared_gate is not None
        self.router_rows = -(-(self.outputs + (1 if self.has_gate else 0)) // 8) * 8
        self.w_gate_up = self.w_down = self.w_router = self.b_router = None

    # --- declarations -----------------------------------------------------------------
    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {}
        for e in range(self.experts):
            g, u, d = (n.format(e) for n in self.expert_names)
            specs[g] = WeightSpec((self.inter, self.hidden))
            specs[u] = WeightSpec((self.inter, self.hidden))
            specs[d] = WeightSpec((self.hidden, self.inter))
        specs[self.n_router] = WeightSpec((self.outputs, self.hidden))
        if self.n_router_bias:
            specs[self.n_router_bias] = WeightSpec((self.outputs,), role="vector")
        if self.shared is not None:
            for name, ws in self.shared.weight_specs().items():
                specs[self.shared_prefix + name] = ws
            if self.n_shared_gate:
                specs[self.n_shared_gate] = WeightSpec((1, self.hidden))
        return specs

    def fused_tensors(self):
        ff, E = self.inter, self.experts
        gate_up, down = [], []
        for e in range(E):
            g, u, d = (n.format(e) for n in self.expert_names)
            gate_up += [(g, e * 2 * ff), (u, e * 2 * ff + ff)]
            down.append((d, e * self.hidden))
        router = [(self.n_router, 0)] + ([(self.n_shared_gate, self.outputs)] if self.has_gate else [])
        fused = {"experts.gate_up": (WeightSpec((E * 2 * ff, self.hidden)), gate_up),
                 "experts.down": (WeightSpec((E * self.hidden, ff)), down),
                 "router.rows": (WeightSpec((self.router_rows, self.hidden)), router)}
        if self.shared is not None:
            for dest, (spec, pieces) in self.shared.fused_tensors().items():
                fused[self.shared_prefix + dest] = (spec, [(self.shared_prefix + n, row) for n, row in pieces])
        return fused

    def kernel_sources(self):
        own = grouped.sources() + moe.sources() + ([] if self.rt.is_fp32 else gemm_bf16.sources(engine_only=True))
        return own + (self.shared.kernel_sources() if self.shared is not None else [])

    def bind(self, tensors):
        ff, E = self.inter, self.experts
        if "experts.gate_up" in tensors:
            gate_up, down, router = tensors["experts.gate_up"], tensors["experts.down"], tensors["router.rows"]
            router[self.outputs + (1 if self.has_gate else 0):].zero_()  # the padding rows: their logits are never read
        else:                                  # the checkpoint's pieces: stack them
            names = [[n.format(e) for n in self.expert_names] for e in range(E)]
            gate_up = torch.cat([tensors[n] for g, u, _ in names for n in (g, u)], 0).contiguous()
            down = torch.cat([tensors[d] for _, _, d in names], 0).contiguous()
            router = torch.zeros((self.router_rows, self.hidden), dtype=tensors[self.n_router].dtype, device=tensors[self.n_router].device)
            router[:self.outputs] = tensors[self.n_router]
            if self.has_gate:
                router[self.outputs] = tensors[self.n_shared_gate].reshape(-1)
        self.w_gate_up = gate_up.view(E, 2 * ff, self.hidden)
        self.w_down = down.view(E, self.hidden, ff)
        self.w_router = router
        self.b_router = tensors[self.n_router_bias] if self.n_router_bias else None
        if self.shared is not None:
            n = len(self.shared_prefix)
            self.shared.bind({k[n:]: v for k, v in tensors.items() if k.startswith(self.shared_prefix)})

    def replay_key(self):
        shared = None
        if self.shared is not None:
            shared = self.shared.replay_key()
            if shared is None:
                return None
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None                  # the library product would go through the tensor framework
        return ("routed_experts", self.hidden, self.experts, self.top, self.inter, shared, self.has_gate, self.b_router is not None,
                self.scoring, self.identity)

    def own_tensors(self):
        own = [self.w_gate_up, self.w_down, self.w_router, self.b_router]
        return own + (self.shared.own_tensors() if self.shared is not None else [])

    # --- compute ------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, out_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, W, E, top, ff = x.shape[0], self.hidden, self.experts, self.top, self.inter
        dev, P = x.device, x.shape[0] * self.top
        flag = ctx.error_flag if ctx is not None else None
        buf = lambda role, shape, dtype: scratch(ctx, "routed." + role, shape, dtype, dev)
        ids = buf("ids", (T, top), torch.int32)
        weights = buf("weights", (T, top), torch.float32)
        gate = buf("shared_gate", (T,), torch.float32) if self.has_gate else None
        # every logit from one product (bf16 operands are multiplied exactly and summed in fp32; the fp32 path is fp32
        # throughout); bias, choice, weights and the gate's sigmoid follow in fp32
        logits = linear(x, self.w_router, None, torch.float32, partials_ok=True, error_flag=flag,
                        alloc=lambda shape, dtype: buf("logits", shape, dtype))
        moe.select(logits, self.outputs, self.b_router, top, ids, weights, self.outputs if self.has_gate else -1, gate, scoring=self.scoring)
        offsets = buf("offsets", (E + 1,), torch.int32)
        order = buf("order", (P,), torch.int32)
        moe.align(ids, E, offsets, order, flag, passthrough=self.identity)
        row_tile = grouped.row_tile_for(P, E, True, grouped.mma_supported(x, self.w_gate_up))
        act = buf("act", (P, ff), self.rt.dtype)
        grouped.grouped_silu_mul(x, self.w_gate_up, act, rows=P, group_offsets=offsets, a_rows=order, a_row_div=top,
                                 row_tile=row_tile, alloc=lambda shape, dtype: buf("gate_up", shape, dtype))
        y = buf("y", (P, W), torch.float32)
        grouped.grouped_linear(act, self.w_down, y, rows=P, group_offsets=offsets, c_rows=order, row_tile=row_tile)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        out = buf("out", (T, W), torch.float32)
        if self.identity:
            moe.combine(y, weights, out, shared=shared, gate=gate, col_scale=out_scale, ids=ids, experts=E, x=x)
        else:
            moe.combine(y, weights, out, shared=shared, gate=gate, col_scale=out_scale)
        return out
