"""Mixture of experts: a router picks a few small gated feed-forwards per token.

    logits  = R x + b                              float32
    chosen  = the ``top`` largest logits           (the lower index wins a tie)
    weights = softmax over the chosen logits alone
    y       = sum_chosen weight_e * down_e(act(gate_e x, up_e x))  (+ shared(x), an expert that every token uses)

The experts' matrices are stacked after loading ([experts, ff, width] and [experts, width, ff]); the
tokens are grouped by expert on the device and the products run over the groups
(``kernels.ops.moe_experts``), so nothing about a step's routing reaches the host and a step of single
tokens can be recorded into a CUDA graph.  A token's result is summed in the order of its own choice
and does not depend on the rest of the batch.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, Param


class RoutedExperts(FeedForward):
    """names: dict with ``router`` (its weight's full name), ``router_bias`` (or None) and ``expert``: a function
    (index, "gate" | "up" | "down") -> tensor name.  ``activation``: ``clamped_swish`` (with ``limit`` and
    ``alpha``) or ``silu``.  ``shared``: a feed-forward part that runs for every token and is added, or None."""
    graph_safe = True

    def __init__(self, hidden_size, expert_size, n_experts, top, *, names, activation="silu", limit=0.0, alpha=1.0,
                 shared=None):
        self.hidden_size, self.expert_size = int(hidden_size), int(expert_size)
        self.n_experts, self.top = int(n_experts), int(top)
        if not 1 <= self.top <= self.n_experts:
            raise ValueError(f"{top} of {n_experts} experts per token")
        self.activation, self.limit, self.alpha = activation, float(limit), float(alpha)
        self.shared = shared
        self.router = Param((n_experts, hidden_size), std=0.5)
        self.router_bias = Param((n_experts,), init="zeros") if names.get("router_bias") else None
        self.gate = [Param((expert_size, hidden_size), std=0.1) for _ in range(n_experts)]
        self.up = [Param((expert_size, hidden_size), std=0.1) for _ in range(n_experts)]
        self.down = [Param((hidden_size, expert_size), std=0.1) for _ in range(n_experts)]
        self._names = {names["router"]: self.router}
        if self.router_bias is not None:
            self._names[names["router_bias"]] = self.router_bias
        for index in range(n_experts):
            self._names[names["expert"](index, "gate")] = self.gate[index]
            self._names[names["expert"](index, "up")] = self.up[index]
            self._names[names["expert"](index, "down")] = self.down[index]
        self._gate = self._up = self._down = None

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [self.shared] if self.shared is not None else []

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        stack = lambda params: torch.stack([p.data for p in params]).contiguous()
        self._gate, self._up, self._down = stack(self.gate), stack(self.up), stack(self.down)
        for param in (*self.gate, *self.up, *self.down):
            param.data = None
        if self.router_bias is not None:
            self.router_bias.data = self.router_bias.data.to(self.router.data.dtype)

    def forward(self, ctx, x, residual=None):
        chosen, weights = ops.moe_route(x, self.router.data, self.router_bias.data if self.router_bias else None, self.top)
        out = ops.moe_experts(x, chosen, weights, self._gate, self._up, self._down, self.activation, limit=self.limit,
                              alpha=self.alpha, residual=residual,
                              out=None if residual is not None else ctx.empty(x.shape, dtype=ctx.stream_dtype))
        if self.shared is not None:
            out = self.shared.forward(ctx, x, residual=out)
        return out
