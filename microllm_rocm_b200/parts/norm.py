"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * w, all in fp32 (`one_plus`: the checkpoint stores w - 1, a weight around zero)
(reference: src/ops/ops.cpp:684-699; fused with the residual add at :702-740).
LayerNorm: y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b, all in fp32; besides the plain form it offers the
step of a block that normalises AFTER its sums: x <- norm(alpha * x + weighted results), in place."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import Norm, Runtime, WeightSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, params: dict, rt: Runtime):
        self.prefix = params.get("prefix", "")
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = params.get("name", "weight")         # the weight's local name in the checkpoint
        self.absent = bool(params.get("absent", False))  # a norm in front of a sub-layer that the layer leaves out: no weight, never run
        self.one_plus = bool(params.get("one_plus", False))   # the stored tensor is the weight minus one: 1 is added once, at bind, in fp32
        self.rt = rt
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if self.absent:
            return {}
        return {self.name: WeightSpec((self.size,), role="vector", init=("normal", 0.1) if self.one_plus else ("one_plus_normal", 0.1))}

    def bind(self, tensors):
        self.weight = tensors.get(self.name) if self.absent else tensors[self.name]
        if self.one_plus and self.weight is not None:
            self.weight = (self.weight.to(torch.float32) + 1.0).contiguous()

    def replay_key(self):
        return ("rmsnorm", self.size, self.eps)

    def own_tensors(self):
        return [self.weight]

    def forward(self, x, out, rows=None):
        ops.rmsnorm(x, self.weight, self.eps, out, rows=rows)

    def add_forward(self, residual, delta, out, scale=None):
        """`scale` [width] fp32: the delta is multiplied by it, column by column, before it is added."""
        if scale is not None:
            ops.add_scaled_rmsnorm(residual, delta, scale, self.weight, self.eps, out)
        else:
            ops.add_rmsnorm(residual, delta, self.weight, self.eps, out)


@register_norm("layernorm")
class LayerNorm(Norm):
    def __init__(self, params: dict, rt: Runtime):
        self.prefix = params.get("prefix", "")
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = params.get("name", "weight")
        self.bias_name = params.get("bias_name", "bias")
        self.absent = bool(params.get("absent", False))
        self.rt = rt
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if self.absent:
            return {}
        return {self.name: WeightSpec((self.size,), role="vector", init=("one_plus_normal", 0.1)),
                self.bias_name: WeightSpec((self.size,), role="vector", init=("normal", 0.1))}

    def kernel_sources(self):
        return [("layernorm.cu", {})]

    def bind(self, tensors):
        self.weight, self.bias = tensors.get(self.name), tensors.get(self.bias_name)
        if not self.absent and (self.weight is None or self.bias is None):
            raise KeyError(f"layer norm: {self.name} or {self.bias_name} is missing")

    def replay_key(self):
        return ("layernorm", self.size, self.eps)

    def own_tensors(self):
        return [self.weight, self.bias]

    def forward(self, x, out, rows=None):
        ops.layernorm(x, self.weight, self.bias, self.eps, out, rows=rows)

    def add_forward(self, residual, delta, out, scale=None):
        # the pre-norm use (residual += delta, then a normed copy) has no kernel of its own yet: two steps
        if scale is not None:
            ops.add_scaled_inplace(residual, delta, scale)
        else:
            ops.add_inplace(residual, delta)
        ops.layernorm(residual, self.weight, self.bias, self.eps, out)

    def post_forward(self, stream: torch.Tensor, alpha: float, terms, copy: Optional[torch.Tensor]) -> None:
        """stream <- norm(alpha * stream + sum_i s_i * d_i) in place (fp32); `copy` receives the new stream in its dtype."""
        ops.scale_add_layernorm(stream, alpha, terms, self.weight, self.bias, self.eps, copy)
