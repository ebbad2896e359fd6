"""A per-layer input from the token itself, added to the residual stream after a layer's feed-forward.

A side table holds one row per token id; layer i owns the columns [i * dim, (i + 1) * dim) of it.  With e the
token's slice and x the stream:

    g = gelu_tanh(G x) * e            G [dim, width]
    y = P g                           P [width, dim]
    x <- x + y / sqrt(mean(y^2) + eps) * w

The gate product runs on the stream's rows in the activation dtype, the norm of the branch and the sum are
float32.  Kernels: a cast of the stream (when it is float32 under bfloat16 activations), the gate product, the
activation times the table's slice, the second product with a float32 result, the normed add.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Param, Part
from .linear import Linear


class TokenSideInput(Part):
    """``table`` is the Param of the whole side table [vocab, layers * dim], shared by all layers under the one
    checkpoint name ``names["table"]``; ``index`` says which slice is this layer's.  names: table, gate, proj, norm."""
    graph_safe = True

    def __init__(self, hidden_size, dim, index, eps, *, table, names, suffixes=(".weight", ".bias"), norm_suffix=".weight"):
        self.hidden_size, self.dim, self.index, self.eps = int(hidden_size), int(dim), int(index), float(eps)
        if table.shape[1] < (self.index + 1) * self.dim:
            raise ValueError(f"a side table of {table.shape[1]} columns has no slice {index} of {dim}")
        self.table = table
        self.gate = Linear(hidden_size, dim, name=names["gate"], suffixes=suffixes)
        self.proj = Linear(dim, hidden_size, name=names["proj"], suffixes=suffixes)
        self.norm_weight = Param((hidden_size,), init="norm", std=0.05)
        self._names = {names["table"]: self.table, names["norm"] + norm_suffix: self.norm_weight}

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [self.gate, self.proj]

    def forward(self, ctx, x):
        rows = x if x.dtype == ctx.dtype else ops.cast(x, ctx.dtype)
        gated = self.gate.forward(ctx, rows)
        ops.activation(gated, "gelu_tanh", table=self.table.data, ids=ctx.token_ids, first_col=self.index * self.dim,
                       out=gated)
        branch = self.proj.forward(ctx, gated, out_float32=True)
        return ops.rms_scale_add(x, branch, self.norm_weight.data, self.eps)
