"""Debisun written plainly: one function per mechanism, whole sequences, no cache, no batching.

A slow restatement of the design's equations for the tests to compare the engine with.  It shares no
code with the engine: weights come as a dict of checkpoint name -> CPU tensor, the configuration as the
dict that config.json holds.  ``dtype`` is the arithmetic's precision (float32 or float64); the
bfloat16 yardstick (``low``) rounds the outputs of projections, short convolutions and activations, and
nothing of what the design computes in 32 bits (norms, scores, softmax, routers, the residual sum).

Notation: T tokens at positions t = 0..T-1, width W, H query heads, G key/value heads, d the size of a
query or key head, e the size of a value head, R rows of a layer's distance table, M its largest
distance, C the chunk size of the mask.
"""
from __future__ import annotations

import math

import torch


def _round(x, low):
    return x if low is None else x.to(low).to(x.dtype)


def linear(x, weight, low=None):
    """y = x W^T, W stored [out, in]; inputs and result rounded when the arithmetic is low precision."""
    return _round(_round(x, low) @ weight.to(x.dtype).t(), low)


def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * w + b with the variance as the mean of squared deviations."""
    mean = x.mean(dim=-1, keepdim=True)
    var = (x - mean).pow(2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight.to(x.dtype) + bias.to(x.dtype)


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight.to(x.dtype)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def squared_relu(z):
    return torch.clamp(z, min=0.0) ** 2


def short_convolution(u, taps_weight, low=None):
    """u [T, channels], taps_weight [channels, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before t = 0."""
    T, channels = u.shape
    taps = taps_weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, channels, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + taps_weight[:, j].to(u.dtype) * padded[j:j + T]
    return _round(y, low)


def distance_bucket(n: int, rows: int, farthest: int) -> int:
    """Row of the distance table for a distance n >= 0: one row per distance below R/2, then rows that
    grow with the logarithm of the distance up to ``farthest``, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(farthest / half) * (rows - half))))


def sink_softmax(scores):
    """p_j = exp(s_j) / (1 + sum_j exp(s_j)): a sink of score zero that carries no value."""
    peak = torch.clamp(scores.max(), min=0.0)
    e = torch.exp(scores - peak)
    return e / (torch.exp(-peak) + e.sum())


def chunk_attention(q, k, v, m, table):
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].

    score[i, j] = cap * tanh(q_i . k_j * scale / cap) + table[bucket(i - j), h] for the j <= i of i's chunk
    (floor(i / C) = floor(j / C)); softmax with the sink; times v.  Head h reads key/value head floor(h / (H/G)).
    """
    T, H, _ = q.shape
    G = k.shape[1]
    group = H // G
    rows = table.shape[0]
    size = (m.get("mask") or {}).get("size")
    cap = m.get("softcap")
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for i in range(T):
        first = (i // size) * size if size else 0
        rows_of = torch.tensor([distance_bucket(i - j, rows, m["bias_max"]) for j in range(first, i + 1)])
        for h in range(H):
            g = h // group
            scores = (k[first:i + 1, g] @ q[i, h]) * m["scale"]
            if cap:
                scores = cap * torch.tanh(scores / cap)
            scores = scores + table[rows_of, h].to(q.dtype)
            out[i, h] = sink_softmax(scores) @ v[first:i + 1, g]
    return out


def attention_mixer(h, w, prefix, m, low=None):
    """Projections, the short convolution on every channel of q, k and v, the attention, the output product."""
    T = h.shape[0]
    q = short_convolution(linear(h, w[prefix + "q"], low), w[prefix + "q.conv"], low)
    k = short_convolution(linear(h, w[prefix + "k"], low), w[prefix + "k.conv"], low)
    v = short_convolution(linear(h, w[prefix + "v"], low), w[prefix + "v.conv"], low)
    mixed = chunk_attention(q.view(T, m["heads"], m["dim"]), k.view(T, m["kv_heads"], m["dim"]),
                            v.view(T, m["kv_heads"], m["vdim"]), m, w[prefix + "rel"])
    return linear(_round(mixed.reshape(T, -1), low), w[prefix + "o"], low)


def dense_ff(h, w, prefix, low=None):
    """down(relu(up h)^2)."""
    return linear(_round(squared_relu(linear(h, w[prefix + "up"], low)), low), w[prefix + "down"], low)


def route(h, w, prefix, router):
    """(chosen [T, top], weights [T, top]): softmax over all outputs of the router, the choice by score plus the
    correction, the weights from the scores alone, divided by their sum and multiplied by the router's scale."""
    scores = torch.softmax(h @ w[prefix + "router"].to(h.dtype).t(), dim=-1)
    chosen = torch.topk(scores + w[prefix + "correction"].to(h.dtype), router["top"], dim=-1).indices
    picked = torch.gather(scores, 1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * router["scale"]


def route_margin(h, w, prefix, router):
    """Per token, how far the last chosen output's choice score lies above the best one that was not chosen, as a
    fraction of the larger of the two outputs' scores (infinite when every output is chosen).  Rounding moves a
    score by a fraction of itself, so a small value here is a close call that rounding can flip."""
    scores = torch.softmax(h @ w[prefix + "router"].to(h.dtype).t(), dim=-1)
    order = (scores + w[prefix + "correction"].to(h.dtype)).sort(dim=-1, descending=True)
    top = router["top"]
    if top >= scores.shape[1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    raw = torch.gather(scores, 1, order.indices[:, top - 1:top + 1]).max(dim=-1).values
    return (order.values[:, top - 1] - order.values[:, top]) / raw.clamp(min=1e-30)


def moe_ff(h, w, prefix, mlp, low=None):
    """Routed experts (the last ``identity`` of the router's outputs hand the input through), plus the shared
    expert times a sigmoid gate of one number per token."""
    router = mlp["router"]
    chosen, weights = route(_round(h, low), w, prefix, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for slot in range(router["top"]):
            index = int(chosen[t, slot])
            if index >= router["experts"]:
                y = _round(h[t:t + 1], low)
            else:
                y = dense_ff(h[t:t + 1], w, f"{prefix}e{index}.", low)
            out[t] += weights[t, slot] * y[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(_round(h, low) @ w[prefix + "shared.sg"].to(h.dtype).t())
        out = out + gate * dense_ff(h, w, prefix + "shared.", low)
    return out


def token_side(x, tokens, w, prefix, index, dim, eps, low=None):
    """The per-layer token input: e = this layer's part of the side table's row; g = gelu(gate x) * e;
    y = proj g; the result is rms_norm(y) with the layer's own weight."""
    e = w["side.embed"][tokens][:, index * dim:(index + 1) * dim].to(x.dtype)
    g = _round(gelu_tanh(linear(x, w[prefix + "side.gate"], low)) * e, low)
    return rms_norm(linear(g, w[prefix + "side.proj"], low), w[prefix + "side.norm"], eps)


def forward(config, w, tokens, dtype=torch.float64, low=None, return_layers=False, margins=None):
    """Logits [T, vocab] of a whole sequence (and the residual stream after every layer).  ``margins``: a list
    that receives every routed layer's ``route_margin`` per token."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = config["norm"]["eps"]
    side = config.get("token_side")
    x = w["embed"][tokens].to(dtype)
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = _round(layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps), low)
        x = x + attention_mixer(h, w, p + "mix.", layer["mixer"], low) * w[p + "ls1"].to(dtype)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = _round(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), low)
            y = dense_ff(h, w, p + "mlp.", low) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp, low)
            if margins is not None and mlp["kind"] == "moe":
                margins.append(route_margin(h, w, p + "mlp.", mlp["router"]))
            x = x + y * w[p + "ls2"].to(dtype)
        if side:
            x = x + token_side(x, tokens, w, p, i, side["dim"], eps, low)
        after.append(x.clone())
    h = _round(layer_norm(x, w["final.norm"], w["final.norm.b"], eps), low)
    logits = _round(h, low) @ w["head"].to(dtype).t()
    return (logits, torch.stack(after)) if return_layers else logits
