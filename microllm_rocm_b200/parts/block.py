"""Pre-norm residual block:  x += a1 * mixer(norm1(x));  x += a2 * feed_forward(norm2(x)).
Each residual add is fused into the norm that follows it (the reference does so on its
decode path only: src/model/model.cpp:862-870 `add_rms_norm`), so the block passes the
residual stream on together with a delta that has not been added yet.

a1 and a2 are 1 unless the block is given `residual_scale` (a number m) and/or `layer_scale` (the local names of
two learned per-column vectors s1, s2): then a1 = m * s1 and a2 = m * s2, element by element, in fp32.  a1 is
applied where the mixer's result is added; a2 is handed to a feed-forward that can multiply its own result
(`FeedForward.scales_output`), else applied by one more pass over the result.  The delta a block returns is always
ready to be added as it is.  A layer may have no feed-forward (kind "none"): the block then ends after the mixer."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import (Block, FeedForward, Mixer, Norm, Runtime, StepContext, WeightSpec, register_block,
                   register_feed_forward)


@register_feed_forward("none")
class NoFeedForward(FeedForward):
    """A layer without a feed-forward."""
    absent = True

    def __init__(self, params: dict, rt: Runtime):
        pass

    def replay_key(self):
        return ("none",)


@register_block("pre_norm_residual")
class PreNormResidualBlock(Block):
    def __init__(self, params: dict, rt: Runtime, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm,
                 feed_forward: FeedForward):
        self.rt = rt
        self.prefix = params.get("prefix", "")
        self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward = mixer_norm, mixer, ffn_norm, feed_forward
        self.has_ff = not getattr(feed_forward, "absent", False)
        self.residual_scale = float(params.get("residual_scale", 1.0))
        self.layer_scale = tuple(params["layer_scale"]) if params.get("layer_scale") else None   # (name of s1, name of s2)
        self.size = int(params["size"]) if self.layer_scale or self.residual_scale != 1.0 else 0
        self.scaled = bool(self.layer_scale) or self.residual_scale != 1.0
        self.a1: Optional[torch.Tensor] = None
        self.a2: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if not self.layer_scale:
            return {}
        names = self.layer_scale if self.has_ff else self.layer_scale[:1]
        return {n: WeightSpec((self.size,), role="vector", init=("one_plus_normal", 0.1)) for n in names}

    def kernel_sources(self):
        return [("residual.cu", {})] if self.scaled else []

    def bind(self, tensors):
        if not self.scaled:
            return
        m = self.residual_scale
        device = self.rt.device
        one = lambda name: (tensors[name] * m).contiguous() if self.layer_scale else torch.full((self.size,), m, dtype=torch.float32, device=device)
        self.a1 = one(self.layer_scale[0] if self.layer_scale else None)
        self.a2 = one(self.layer_scale[1] if self.layer_scale else None) if self.has_ff else None

    def replay_key(self):
        keys = [p.replay_key() for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)]
        if not self.has_ff:
            return None                  # the block returns no pending delta: its runs are issued call by call
        return None if any(k is None for k in keys) else ("pre_norm_residual", self.rt.dtype, self.scaled, *keys)

    def own_tensors(self):
        own = [t for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) for t in p.own_tensors()]
        return own + [self.a1, self.a2]

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext, cache):
        normed = ctx.buffer("block.normed", tuple(residual.shape), self.rt.dtype)
        if delta is None:
            self.mixer_norm.forward(residual, normed)
        else:
            self.mixer_norm.add_forward(residual, delta, normed)
        mixed = self.mixer.forward(normed, ctx, cache)
        if not self.has_ff:
            if self.scaled:
                ops.add_scaled_inplace(residual, mixed, self.a1)
            else:
                ops.add_inplace(residual, mixed)
            return residual, None
        normed2 = ctx.buffer("block.normed2", tuple(residual.shape), self.rt.dtype)
        if self.scaled:
            self.ffn_norm.add_forward(residual, mixed, normed2, scale=self.a1)
        else:
            self.ffn_norm.add_forward(residual, mixed, normed2)
        if not self.scaled:
            return residual, self.feed_forward.forward(normed2, ctx)
        if getattr(self.feed_forward, "scales_output", False):
            return residual, self.feed_forward.forward(normed2, ctx, out_scale=self.a2)
        # a feed-forward that cannot scale its own result: one pass over it (split partial sums are added up on the way)
        out = self.feed_forward.forward(normed2, ctx)
        scaled = ctx.buffer("block.scaled_delta", tuple(residual.shape), torch.float32)
        scaled.zero_()
        ops.add_scaled_inplace(scaled, out, self.a2)
        return residual, scaled


@register_block("post_norm_residual")
class PostNormResidualBlock(Block):
    """Norm after the sum:  x <- norm1(alpha * x + mixer(x));  x <- norm2(alpha * x + feed_forward(x)).  The sublayers read
    the stream itself, so the stream that leaves a block is final (no delta is handed on) and, on the bf16 path, travels
    with a bf16 copy for the products that read it; the sums and norms are fp32.  A mixer that is several mixers side
    by side may hand over its weighted terms (`forward_terms`): the norm kernel adds them, no pass of its own."""
    carries_no_delta = True

    def __init__(self, params: dict, rt: Runtime, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, feed_forward: FeedForward):
        self.rt = rt
        self.prefix = params.get("prefix", "")
        self.alpha = float(params.get("alpha", 1.0))
        self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward = mixer_norm, mixer, ffn_norm, feed_forward
        self.has_ff = not getattr(feed_forward, "absent", False)
        for norm in (mixer_norm, ffn_norm) if self.has_ff else (mixer_norm,):
            if not hasattr(norm, "post_forward"):
                raise TypeError("post_norm_residual needs norms that can normalise a scaled sum in place (post_forward)")

    def replay_key(self):
        keys = [p.replay_key() for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)]
        return None if any(k is None for k in keys) else ("post_norm_residual", self.rt.dtype, self.alpha, *keys)

    def own_tensors(self):
        return [t for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) for t in p.own_tensors()]

    def _reads(self, stream: torch.Tensor, ctx: StepContext):
        """What the sublayers' products read: the stream itself (fp32 path) or its bf16 copy."""
        if self.rt.is_fp32:
            return stream, None
        return None, ctx.buffer("block.stream_copy", tuple(stream.shape), self.rt.dtype)

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext, cache):
        if delta is not None:            # a block of another arrangement ran before this one
            ops.add_inplace(residual, delta)
        x, copy = self._reads(residual, ctx)
        if x is None:
            x = copy
            if ctx.step_values.get("block.stream_copy_of") != residual.data_ptr():
                ops.cast_f32_bf16(residual, copy)            # the first block of a step: nobody has made the copy yet
        terms = self.mixer.forward_terms(x, ctx, cache) if hasattr(self.mixer, "forward_terms") else [(1.0, self.mixer.forward(x, ctx, cache))]
        self.mixer_norm.post_forward(residual, self.alpha, terms, copy)
        if self.has_ff:
            self.ffn_norm.post_forward(residual, self.alpha, [(1.0, self.feed_forward.forward(x, ctx))], copy)
        if copy is not None:
            ctx.step_values["block.stream_copy_of"] = residual.data_ptr()
        return residual, None


@register_block("sandwich_residual")
class SandwichResidualBlock(Block):
    """A norm on both sides of every sublayer:  x += post1(mixer(pre1(x)));  x += post2(feed_forward(pre2(x))), all four rms
    norms with weights.  The two norms in front are the layer's `mixer_norm` and `ffn_norm`; the two behind are the block's
    own tensors (`post_names`).  A sublayer's result is normalised, added, and the stream normalised again for the next
    sublayer in ONE kernel; a mixer that is several mixers side by side hands over its weighted terms (`forward_terms`) and
    that kernel adds them.  The stream that leaves the block is final (no delta is handed on)."""
    carries_no_delta = True

    def __init__(self, params: dict, rt: Runtime, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, feed_forward: FeedForward):
        self.rt = rt
        self.prefix = params.get("prefix", "")
        self.size, self.eps = int(params["size"]), float(params["eps"])
        self.post_names = tuple(params.get("post_names", ("post_mixer_norm.weight", "post_ffn_norm.weight")))
        self.one_plus = bool(params.get("one_plus", False))      # the two weights behind the sublayers are stored minus one
        self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward = mixer_norm, mixer, ffn_norm, feed_forward
        self.has_ff = not getattr(feed_forward, "absent", False)
        if self.has_ff and not (hasattr(ffn_norm, "weight") and getattr(ffn_norm, "eps", None) == self.eps and hasattr(ffn_norm, "size")):
            raise TypeError("sandwich_residual fuses the norm in front of the feed-forward: it must be an rms norm with the block's eps")
        self.w_post1: Optional[torch.Tensor] = None
        self.w_post2: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        names = self.post_names if self.has_ff else self.post_names[:1]
        init = ("normal", 0.1) if self.one_plus else ("one_plus_normal", 0.1)
        return {n: WeightSpec((self.size,), role="vector", init=init) for n in names}

    def kernel_sources(self):
        return [("post_norm.cu", {})]

    def bind(self, tensors):
        take = (lambda t: (t.to(torch.float32) + 1.0).contiguous()) if self.one_plus else (lambda t: t)
        self.w_post1 = take(tensors[self.post_names[0]])
        self.w_post2 = take(tensors[self.post_names[1]]) if self.has_ff else None

    def replay_key(self):
        keys = [p.replay_key() for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)]
        return None if any(k is None for k in keys) else ("sandwich_residual", self.rt.dtype, self.size, self.eps, *keys)

    def own_tensors(self):
        own = [t for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) for t in p.own_tensors()]
        return own + [self.w_post1, self.w_post2]

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext, cache):
        if delta is not None:            # a block of another arrangement ran before this one
            ops.add_inplace(residual, delta)
        normed = ctx.buffer("block.normed", tuple(residual.shape), self.rt.dtype)
        self.mixer_norm.forward(residual, normed)
        terms = self.mixer.forward_terms(normed, ctx, cache) if hasattr(self.mixer, "forward_terms") else [(1.0, self.mixer.forward(normed, ctx, cache))]
        if not self.has_ff:
            ops.normed_add_rmsnorm(residual, terms, self.w_post1, self.eps)
            return residual, None
        normed2 = ctx.buffer("block.normed2", tuple(residual.shape), self.rt.dtype)
        ops.normed_add_rmsnorm(residual, terms, self.w_post1, self.eps, next_weight=self.ffn_norm.weight, out=normed2)
        ops.normed_add_rmsnorm(residual, [(1.0, self.feed_forward.forward(normed2, ctx))], self.w_post2, self.eps)
        return residual, None
