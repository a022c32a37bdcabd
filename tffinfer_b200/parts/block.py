"""Arrangements of the parts around the residual stream.  ``pre_norm`` is the
reference's Qwen3 block (src/core/model/qwen3/QWen3Creator.cpp:62-151):
``x = x + mixer(norm(x)); x = x + ffn(norm(x))``, the stream kept in float32."""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import Block, LayerContext


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, mixer, feed_forward, mixer_norm=None, ffn_norm=None, extra_norms=None):
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm, extra_norms)
        if mixer_norm is None or (ffn_norm is None and feed_forward is not None):
            raise ValueError("the pre_norm arrangement needs mixer_norm, and ffn_norm where there is a feed-forward")

    @staticmethod
    def _normed(norm, consumer, x, ctx: LayerContext, act_dtype):
        """The norm's output for ``consumer``.  A part that does nothing with its input but hand it to the kernel
        library's products says so (``takes_deferred_norm``); it may then get the norm not yet run, which the
        library folds into the product where that saves a kernel."""
        if getattr(consumer, "takes_deferred_norm", False) and hasattr(norm, "deferred"):
            d = norm.deferred(x, ctx.ops, act_dtype)
            if d is not None:
                return d
        return norm.forward(x, ctx.ops, act_dtype)

    def forward(self, x, ctx: LayerContext, act_dtype):
        h = self._normed(self.mixer_norm, self.mixer, x, ctx, act_dtype)
        x = self.mixer.forward(h, ctx, residual=x)
        if self.feed_forward is None:         # a layer of a mixer alone
            return x
        h = self._normed(self.ffn_norm, self.feed_forward, x, ctx, act_dtype)
        x = self.feed_forward.forward(h, ctx, residual=x)
        return x


@register_part("block", "parallel_pre_norm")
class ParallelPreNormBlock(Block):
    """The mixer and the feed-forward side by side, each behind a norm of its own, both norms reading the same
    residual: ``x <- x + (mixer(norm1(x)) + ffn(norm2(x)))``.  Both norms run before either sublayer adds to the stream
    (one kernel for the two where the kernel library has it); a layer without a feed-forward is the mixer alone."""

    def __init__(self, mixer, feed_forward, mixer_norm=None, ffn_norm=None, extra_norms=None):
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm, extra_norms)
        if mixer_norm is None or (ffn_norm is None and feed_forward is not None):
            raise ValueError("the parallel_pre_norm arrangement needs mixer_norm, and ffn_norm where there is a feed-forward")

    def forward(self, x, ctx: LayerContext, act_dtype):
        if self.feed_forward is None:
            return self.mixer.forward(self.mixer_norm.forward(x, ctx.ops, act_dtype), ctx, residual=x)
        pair = getattr(ctx.ops, "rmsnorm_pair", None)
        if pair is not None and hasattr(self.mixer_norm, "weight") and hasattr(self.ffn_norm, "weight") \
                and self.mixer_norm.eps == self.ffn_norm.eps:
            h1 = torch.empty((x.shape[0], x.shape[1]), dtype=act_dtype, device=x.device)
            h2 = torch.empty_like(h1)
            pair(x, self.mixer_norm.weight, self.ffn_norm.weight, self.mixer_norm.eps, h1, h2)
        else:
            h1 = self.mixer_norm.forward(x, ctx.ops, act_dtype)
            h2 = self.ffn_norm.forward(x, ctx.ops, act_dtype)
        x = self.mixer.forward(h1, ctx, residual=x)
        return self.feed_forward.forward(h2, ctx, residual=x)
