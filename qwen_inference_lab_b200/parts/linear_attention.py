"""Gated linear attention: a recurrent mixer whose state is a matrix per head, decayed per key channel.

Per head, with d key channels and e value channels, for the tokens of a sequence in order:

    a_t = sigmoid(A2 (A1 x_t) + b)^(1/tau)          decay per key channel, float32
    S_t = diag(a_t) S_(t-1) + k_t v_t^T              S_0 = 0, float32, one per request and layer call
    o_t = S_t^T (q_t * q_scale)
    y_t = W_o ( rmsnorm_e(o_t; w) * silu(W_g x_t) )  the norm is over a head's e values, w shared by heads

q, k, v, the gate and the low-rank input of the decay are one stacked product; the recurrence, the norm
and the gate are one kernel that walks every segment of the step from the request's state slot
(``kernels.ops.gla_scan``), so prompt portions of any length and single decoded tokens take the same path
and the result does not depend on the cut.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, Param, StateSpec
from .linear import Linear, StackedLinear


class GatedLinearAttention(Mixer):
    """names: dict with keys q, k, v, g, o, a1, a2 (projection names) and norm (the output norm's weight).
    ``suffixes``: what the checkpoint appends to a projection's name for weight and bias."""
    graph_safe = True

    def __init__(self, hidden_size, n_heads, key_dim, value_dim, decay_rank, *, tau, norm_eps, names,
                 q_scale=None, suffixes=(".weight", ".bias"), norm_suffix=".weight"):
        self.hidden_size, self.n_heads = int(hidden_size), int(n_heads)
        self.key_dim, self.value_dim, self.decay_rank = int(key_dim), int(value_dim), int(decay_rank)
        self.tau, self.norm_eps = float(tau), float(norm_eps)
        if not self.tau > 0:
            raise ValueError("tau must be positive")
        self.q_scale = float(q_scale) if q_scale is not None else self.key_dim ** -0.5
        kw, vw = self.n_heads * self.key_dim, self.n_heads * self.value_dim
        self.projection = StackedLinear(hidden_size, [(names["q"], kw), (names["k"], kw), (names["v"], vw),
                                                      (names["g"], vw), (names["a1"], self.decay_rank)],
                                        suffixes=suffixes)
        self.columns = (0, kw, 2 * kw, 2 * kw + vw, 2 * kw + 2 * vw)
        self.decay_up = Param((kw, self.decay_rank), std=0.2)
        self.decay_bias = Param((kw,), init="zeros")
        self.norm_weight = Param((self.value_dim,), init="norm", std=0.05)
        self._names = {names["a2"] + suffixes[0]: self.decay_up, names["a2"] + suffixes[1]: self.decay_bias,
                       names["norm"] + norm_suffix: self.norm_weight}
        self.out = Linear(vw, hidden_size, name=names["o"], suffixes=suffixes)
        self._needs_scratch = False

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [self.projection, self.out]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        common = self.projection._weight().dtype
        for param in (self.decay_up, self.decay_bias, self.norm_weight):
            param.data = param.data.to(common).contiguous()
        self._needs_scratch = ops.gla_scan_needs_scratch(self.key_dim, self.value_dim)

    def cache_spec(self):
        return StateSpec((self.n_heads, self.key_dim, self.value_dim), torch.float32)

    takes_norm = True

    def forward(self, ctx, x, cache, residual=None, norm=None):
        """x [N, hidden] -> [N, hidden] (+ residual); ``cache`` is a StateView with one slot per request row."""
        n = x.shape[0]
        projected = self.projection.forward(ctx, x, norm=norm)
        mixed = ctx.empty((n, self.n_heads * self.value_dim))
        scratch = None
        if self._needs_scratch:
            scratch = ctx.empty((n, self.n_heads * self.value_dim), dtype=torch.float32)
        ops.gla_scan(projected, self.columns, self.decay_up.data, self.decay_bias.data, self.tau, self.q_scale,
                     self.norm_weight.data, self.norm_eps, cache.slots, ctx.seg_start, ctx.seg_len, ctx.seg_row,
                     ctx.n_segments, self.n_heads, self.key_dim, self.value_dim, mixed, scratch=scratch)
        return self.out.forward(ctx, mixed, residual=residual)
