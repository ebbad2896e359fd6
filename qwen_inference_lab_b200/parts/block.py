"""Arrangement of a layer's parts: norm -> mixer -> + -> norm -> feed-forward -> +.

The pre-norm order of the reference's ``DecoderBlock.forward`` (qil/model.py:48-71).
The block owns no sizes: it is given a norm, a mixer, a second norm and a
feed-forward, each already built, so different layers of one model may hold
different kinds of each.  ``feed_forward`` may be None: the layer is then its mixer
alone (a second norm given all the same only claims its tensor).

Two options for other designs.  A learned scale per feature on each branch before it joins the stream
(``scales``: the two tensors' names): x <- x + s1 * mixer(norm1 x), x <- x + s2 * ff(norm2 x); a part that sets
``takes_out_scale`` applies the scale in its last kernel, the others' results are scaled and added by a kernel
of the block's.  And parts that run on the stream after the feed-forward (``after``: each ``forward(ctx, x) -> x``).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Param, Part


class PreNormBlock(Part):
    def __init__(self, mixer_norm, mixer, ff_norm, feed_forward, *, scales=None, after=()):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.ff_norm, self.feed_forward = ff_norm, feed_forward
        self.after = list(after)
        self.graph_safe = True
        self.mixer_scale = self.ff_scale = None
        self._scale_names = scales
        if scales is not None:
            width = mixer_norm.width
            self.mixer_scale = Param((width,), init="norm", std=0.05)
            self.ff_scale = Param((width,), init="norm", std=0.05, optional=feed_forward is None)

    def named_params(self):
        if self._scale_names is None:
            return {}
        return {self._scale_names[0]: self.mixer_scale, self._scale_names[1]: self.ff_scale}

    def children(self):
        return [part for part in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward, *self.after)
                if part is not None]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        for scale in (self.mixer_scale, self.ff_scale):      # the kernels read the scales as float32
            if scale is not None and scale.data is not None:
                scale.data = scale.data.to(torch.float32).contiguous()

    def _scaled(self, ctx, part, norm, x, scale, *cache):
        """x + scale * part(norm(x)), by the part's own last kernel where it can."""
        if getattr(part, "takes_out_scale", False):
            if getattr(part, "takes_norm", False):
                return part.forward(ctx, x, *cache, residual=x, norm=norm, out_scale=scale)
            return part.forward(ctx, norm.forward(ctx, x), *cache, residual=x, out_scale=scale)
        if getattr(part, "takes_norm", False):
            branch = part.forward(ctx, x, *cache, norm=norm)
        else:
            branch = part.forward(ctx, norm.forward(ctx, x), *cache)
        return ops.scaled_add(x, branch, scale)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, x, cache):
        """x [N, hidden] is the residual stream; returned updated (possibly in place)."""
        if self.mixer_scale is not None:
            x = self._scaled(ctx, self.mixer, self.mixer_norm, x, self.mixer_scale.data, cache)
            if self.feed_forward is not None:
                x = self._scaled(ctx, self.feed_forward, self.ff_norm, x, self.ff_scale.data)
            for part in self.after:
                x = part.forward(ctx, x)
            return x
        x = self._plain(ctx, x, cache)
        for part in self.after:
            x = part.forward(ctx, x)
        return x

    def _plain(self, ctx, x, cache):
        if getattr(self.mixer, "takes_norm", False):
            x = self.mixer.forward(ctx, x, cache, residual=x, norm=self.mixer_norm)
        else:
            x = self.mixer.forward(ctx, self.mixer_norm.forward(ctx, x), cache, residual=x)
        if self.feed_forward is None:       # a layer without a feed-forward
            return x
        if getattr(self.feed_forward, "takes_norm", False):
            return self.feed_forward.forward(ctx, x, residual=x, norm=self.ff_norm)
        return self.feed_forward.forward(ctx, self.ff_norm.forward(ctx, x), residual=x)
