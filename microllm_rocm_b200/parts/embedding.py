"""Token embedding (gather of table rows into the fp32 residual stream; optionally plus a row of a second table chosen
by a hash of the token and the one before it, whose last value is part of a sequence's state) and the LM head
(product of selected, normalised rows with the head matrix, or with the embedding table
when the two are tied).  Reference: embedding src/ops/ops.cpp:581-618; tied head as a
product with the transposed table, no copy, src/model/model.cpp:1122-1125."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..kernels.linear import linear
from .base import Part, Runtime, WeightSpec, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    def __init__(self, params: dict, rt: Runtime):
        self.name = params["name"]
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))       # the gathered rows are multiplied by it (fp32)
        # an rms norm of the gathered rows with a weight of its own: (local name of the weight, eps), or None
        self.norm = (str(params["norm"][0]), float(params["norm"][1])) if params.get("norm") else None
        self.norm_weight: Optional[torch.Tensor] = None
        # a second table of buckets + 1 rows: row (previous token * mul_prev + token * mul_cur) mod buckets is added, the last
        # row for a sequence's first token.  {"name", "buckets", "mul_prev", "mul_cur"} or None
        bg = params.get("bigram")
        self.bigram = dict(name=str(bg["name"]), buckets=int(bg["buckets"]), mul_prev=int(bg["mul_prev"]), mul_cur=int(bg["mul_cur"])) if bg else None
        if self.bigram and self.bigram["buckets"] <= 0:
            raise ValueError("token_embedding: bigram buckets must be positive")
        self.bigram_table: Optional[torch.Tensor] = None
        self.rt = rt
        self.table: Optional[torch.Tensor] = None

    def cache_need(self):
        """What the embedding keeps per sequence between steps: the last token it saw (one int), when rows are chosen by pairs."""
        from .base import FixedStateNeed
        return FixedStateNeed((1,), torch.int32) if self.bigram else None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {self.name: WeightSpec((self.vocab, self.hidden), role="table")}
        if self.bigram:
            specs[self.bigram["name"]] = WeightSpec((self.bigram["buckets"] + 1, self.hidden), role="table")
        if self.norm:
            specs[self.norm[0]] = WeightSpec((self.hidden,), role="vector", init=("one_plus_normal", 0.1))
        return specs

    def kernel_sources(self):
        return [("residual.cu", {})] if self.scale != 1.0 or self.bigram else []

    def bind(self, tensors):
        self.table = tensors[self.name]
        if self.bigram:
            self.bigram_table = tensors[self.bigram["name"]]
        if self.norm:
            self.norm_weight = tensors[self.norm[0]]

    def forward(self, token_ids: torch.Tensor, ctx=None, state=None) -> torch.Tensor:
        """`ctx`, `state`: the step and the view of this part's per-sequence state; needed only with a pair table."""
        out = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32, device=token_ids.device)
        if self.bigram and (ctx is None or state is None):
            raise RuntimeError("token_embedding: a pair table needs the step's context and the sequences' state")
        one_pass = self.bigram and self.scale == 1.0 and self.bigram_table.dtype == self.table.dtype      # both rows gathered and added at once
        if one_pass:
            pass
        elif self.scale != 1.0:
            ops.embed_gather_scaled(self.table, token_ids, out, self.scale)
        else:
            ops.embed_gather(self.table, token_ids, out)
        if self.bigram:
            b = self.bigram
            ops.bigram_add(out, self.bigram_table, ctx, state.storage, state.slots, b["buckets"], b["mul_prev"], b["mul_cur"],
                           update_state=state.writable, token_table=self.table if one_pass else None)
        if self.norm:
            ops.rmsnorm(out, self.norm_weight, self.norm[1], out)          # in place, fp32
        return out


@register_head("lm_head")
class LMHead(Part):
    def __init__(self, params: dict, rt: Runtime):
        self.name = params["name"]
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.softcap = float(params["softcap"]) if params.get("softcap") else None      # logits <- cap * tanh(logits / cap)
        self.rt = rt
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if self.tied_to is not None:
            return {}
        return {self.name: WeightSpec((self.vocab, self.hidden), role="matrix")}

    def bind(self, tensors):
        self.weight = tensors[self.tied_to if self.tied_to is not None else self.name]

    def kernel_sources(self):
        own = [("residual.cu", {})] if self.softcap else []
        if self.rt.is_fp32:
            return own
        from ..kernels import gemm_bf16
        return own + gemm_bf16.sources(engine_only=True)

    def forward(self, rows: torch.Tensor, error_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
        """rows [R, H] in the compute dtype -> logits [R, V] fp32.  `error_flag`: the step's device flag."""
        logits = linear(rows, self.weight, None, torch.float32, partials_ok=True, error_flag=error_flag)
        if logits.dim() == 3:
            # a weight-streaming kernel: with this many output rows it does not split K, so the one
            # partial result is the product itself
            if logits.shape[0] != 1:        # a small vocabulary with a long K: add the partial results up
                total = torch.zeros(logits.shape[1:], dtype=torch.float32, device=logits.device)
                ops.add_inplace(total, logits)
                logits = total
            else:
                logits = logits[0]
        if self.softcap:
            if not logits.is_contiguous():
                logits = logits.contiguous()
            ops.softcap_rows(logits, self.softcap)
        return logits
