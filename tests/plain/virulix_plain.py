"""Virulix written plainly: one function per mechanism, whole sequences, no cache, no batching.

A slow restatement of the design's equations for the tests to compare the engine with.  It shares no
code with the engine: weights come as a dict of checkpoint name -> CPU tensor, the configuration as the
dict that config.json holds.  ``dtype`` is the arithmetic's precision (float32 or float64); the
bfloat16 yardstick rounds the outputs of projections and activations, and nothing of what the design
computes in 32 bits.

Notation: T tokens, positions t = 0..T-1, width W, H query heads, G key/value heads, d the size of a
query or key head, e the size of a value head.
"""
from __future__ import annotations

import math

import torch


def _round(x, low):
    """The value after a trip through the low-precision type (``low`` None: no rounding)."""
    return x if low is None else x.to(low).to(x.dtype)


def linear(x, weight, bias=None, low=None):
    """y = x W^T (+ b); inputs and result rounded when the arithmetic is low precision."""
    y = _round(x, low) @ weight.to(x.dtype).t()
    if bias is not None:
        y = y + bias.to(x.dtype)
    return _round(y, low)


def offset_rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w): the weight is stored around zero."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * (1.0 + weight.to(x.dtype))


def plain_rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight.to(x.dtype)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((t + 1) / every) + 1) per position."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(torch.float64) + 1.0)


def distance_slopes(heads):
    """slope_h = 2^(-8 (h + 1) / H)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float64)


def biased_attention(q, k, v, scale):
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].

    score[i, j] = q_i . k_j * scale - slope_h (i - j) for j <= i; softmax over j; times v.
    Query head h reads key/value head floor(h / (H / G)).
    """
    T, H, _ = q.shape
    G = k.shape[1]
    group = H // G
    slopes = distance_slopes(H).to(q.dtype)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // group
        for i in range(T):
            scores = (k[: i + 1, g] @ q[i, h]) * scale
            distance = (i - torch.arange(i + 1)).to(q.dtype)
            weights = torch.softmax(scores - slopes[h] * distance, dim=0)
            out[i, h] = weights @ v[: i + 1, g]
    return out


def attention_mixer(h, w, prefix, m, shared_kv=None, low=None):
    """The attention mixer over a whole sequence.  Returns (output [T, W], (k, v) as the cache holds them).

    ``m`` is the layer's ``mixer`` dict; ``shared_kv``: the (k, v) of the layer named by ``kv_from``.
    """
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, w[prefix + "q"], w[prefix + "q.b"], low).reshape(T, H, d)
    if shared_kv is None:
        k = linear(h, w[prefix + "k"], w[prefix + "k.b"], low).reshape(T, G, d)
        v = linear(h, w[prefix + "v"], w[prefix + "v.b"], low).reshape(T, G, e)
    else:
        k, v = shared_kv
    if m.get("q_temp"):
        temperature = query_temperature(torch.arange(T), m["q_temp"]["coef"], m["q_temp"]["every"])
        q = q * temperature.to(q.dtype)[:, None, None]
    mixed = biased_attention(q, k, v, m["scale"]).reshape(T, H * e)
    return linear(mixed, w[prefix + "o"], None, low), (k, v)


def gated_linear_recurrence(q, k, v, alpha, state=None):
    """Per head: S_t = diag(alpha_t) S_(t-1) + k_t v_t^T ; o_t = S_t^T q_t.

    q, k, alpha [T, H, d]; v [T, H, e]; state [H, d, e] or None (zeros).  Returns (o [T, H, e], state).
    """
    T, H, d = q.shape
    e = v.shape[-1]
    S = torch.zeros(H, d, e, dtype=q.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, e, dtype=q.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out, S


def gla_mixer(h, w, prefix, m, eps, low=None):
    """The gated-linear-attention mixer over a whole sequence -> [T, W]."""
    T = h.shape[0]
    H, d, e, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = linear(h, w[prefix + "q"], None, low).reshape(T, H, d) * d ** -0.5
    k = linear(h, w[prefix + "k"], None, low).reshape(T, H, d)
    v = linear(h, w[prefix + "v"], None, low).reshape(T, H, e)
    z = linear(linear(h, w[prefix + "a1"], None, low), w[prefix + "a2"], w[prefix + "a2.b"], low).reshape(T, H, d)
    alpha = torch.sigmoid(z) ** (1.0 / tau)
    o, _ = gated_linear_recurrence(q, k, v, alpha)
    o = plain_rms_norm(o, w[prefix + "norm"], eps).reshape(T, H * e)
    gate = linear(h, w[prefix + "g"], None, low)
    gate = _round(gate * torch.sigmoid(gate), low)
    return linear(o * gate, w[prefix + "o"], None, low)


def dense_feed_forward(h, w, prefix, low=None):
    gate = _round(gelu_tanh(linear(h, w[prefix + "gate"], w[prefix + "gate.b"], low)), low)
    up = linear(h, w[prefix + "up"], w[prefix + "up.b"], low)
    return linear(gate * up, w[prefix + "down"], w[prefix + "down.b"], low)


def clamped_expert(h, w, prefix, limit, low=None):
    """g = min(W_gate h, limit); u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(linear(h, w[prefix + "gate"], None, low), max=limit)
    u = torch.clamp(linear(h, w[prefix + "up"], None, low), min=-limit, max=limit)
    y = _round(g * torch.sigmoid(1.702 * g) * (u + 1.0), low)
    return linear(y, w[prefix + "down"], None, low)


def route(h, w, prefix, top, low=None):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over those alone."""
    logits = _round(h, low) @ w[prefix + "router"].to(h.dtype).t() + w[prefix + "router.b"].to(h.dtype)
    values, chosen = logits.topk(top, dim=-1)
    return chosen, torch.softmax(values, dim=-1)


def routed_feed_forward(h, w, prefix, mlp, low=None):
    top = mlp["router"]["top"]
    chosen, weights = route(h, w, prefix, top, low)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for slot in range(top):
            expert = int(chosen[t, slot])
            out[t] += weights[t, slot] * clamped_expert(h[t:t + 1], w, f"{prefix}e{expert}.", mlp["expert"]["limit"], low)[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, prefix + "shared.", mlp["shared"]["limit"], low)
    return out


def forward(tokens, w, config, dtype=torch.float32, low=None, residuals=None):
    """Logits [T, vocab] of a whole sequence.  ``residuals``: a list that receives the residual stream
    after every layer."""
    eps = config["norm"]["eps"]
    w = {name: value.to(dtype) if value.is_floating_point() else value for name, value in w.items()}
    x = w["embed"][torch.as_tensor(tokens)]
    kv = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = offset_rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            source = layer["mixer"].get("kv_from")
            mixed, kv[i] = attention_mixer(h, w, p + "mix.", layer["mixer"], None if source is None else kv[source], low)
        elif layer["type"] == "gla":
            mixed = gla_mixer(h, w, p + "mix.", layer["mixer"], eps, low)
        else:
            raise ValueError(f"unknown mixer {layer['type']}")
        x = x + mixed
        mlp = layer.get("mlp")
        if mlp:
            h = offset_rms_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + dense_feed_forward(h, w, p + "mlp.", low)
            elif mlp["kind"] == "moe":
                x = x + routed_feed_forward(h, w, p + "mlp.", mlp, low)
            else:
                raise ValueError(f"unknown feed-forward {mlp['kind']}")
        if residuals is not None:
            residuals.append(x.clone())
    x = offset_rms_norm(x, w["final.norm"], eps)
    return linear(x, w["head"], None, low)
