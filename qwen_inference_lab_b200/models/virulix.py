"""Virulix as an arrangement of parts, with the checkpoint's tensor names.

Layer i (tensors ``l<i>.*``) is pre-norm around a mixer and, where it has one, a feed-forward; both norms
store their weight around zero (``1 + w``).  The residual stream, the norms, attention scores, routers and
the recurrent state are float32 whatever the activation dtype is.

``attention``  biased projections q, k, v (``.b``), no rotation; the query is multiplied by a temperature
               that grows with the logarithm of the position; score = q.k * scale - 2^(-8 (h + 1) / H) * (i - j);
               causal softmax; ``kv_from: j`` reads the pages layer j wrote with its own queries.
``gla``        gated linear attention with a decay per key channel (``parts.linear_attention``).
``dense``      down(gelu_tanh(gate x) * up x), all three with biases.
``moe``        a float32 router (``router``, ``router.b``) picks ``top`` of ``experts`` small feed-forwards
               ``e<k>`` with a clamped swish; a shared expert (``shared``) may run for every token.
Then ``final.norm`` and ``head``.
"""
from __future__ import annotations

import torch

from ..config.model_config import VirulixConfig
from ..config.registry import register
from ..parts import (DecoderModel, ExactRMSNorm, GatedLinearAttention, GatedMLP, GroupedQueryAttention, LayerCall,
                     Linear, PreNormBlock, RoutedExperts, TokenEmbedding)

BARE = ("", ".b")          # this design's tensors carry the projection's own name; biases add ".b"
SWISH_ALPHA = 1.702        # the experts' activation: g * sigmoid(1.702 g)


def distance_slopes(heads: int) -> list:
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def _feed_forward(width, mlp, prefix):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return GatedMLP(width, mlp["ff"], names={k: prefix + k for k in ("gate", "up", "down")},
                        activation="gelu_tanh", bias=True, suffixes=BARE)
    shared = None
    if mlp.get("shared"):
        shared = GatedMLP(width, mlp["shared"]["ff"], names={k: f"{prefix}shared.{k}" for k in ("gate", "up", "down")},
                          activation="clamped_swish", limit=mlp["shared"]["limit"], alpha=SWISH_ALPHA, suffixes=BARE)
    return RoutedExperts(width, mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"]["top"],
                         names=dict(router=prefix + "router", router_bias=prefix + "router.b",
                                    expert=lambda index, which: f"{prefix}e{index}.{which}"),
                         activation="clamped_swish", limit=mlp["expert"]["limit"], alpha=SWISH_ALPHA, shared=shared)


DEFAULT_DECAY_RANK = 16    # for random weights; a checkpoint's own ``a1`` tensor says it otherwise


def _mixer(width, kind, m, prefix, eps, shapes):
    names = {k: prefix + k for k in ("q", "k", "v", "o", "g", "a1", "a2", "norm")}
    if kind == "attention":
        temperature = m.get("q_temp")
        return GroupedQueryAttention(
            width, m["heads"], m["kv_heads"], m["dim"], names=names, bias=True, out_bias=False, scale=m.get("scale"),
            v_head_dim=m["vdim"], distance_slopes=distance_slopes(m["heads"]),
            q_temperature=(temperature["coef"], temperature["every"]) if temperature else None,
            reads_shared_cache=m.get("kv_from") is not None, suffixes=BARE)
    # the width of the decay's low-rank projection is a size that only the tensor's shape gives
    rank = shapes[prefix + "a1"][0] if shapes and prefix + "a1" in shapes else m.get("rank", DEFAULT_DECAY_RANK)
    return GatedLinearAttention(width, m["heads"], m["dim"], m["vdim"], rank, tau=m["tau"], norm_eps=eps, names=names,
                                suffixes=BARE, norm_suffix="")


def build_virulix(config: VirulixConfig, tensor_shapes=None) -> DecoderModel:
    width, eps = config.width, config.eps
    norm = lambda name, optional=False: ExactRMSNorm(width, eps, name=name, offset=1.0, suffix="", optional=optional)
    layers, order = [], []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}."
        mlp = layer.get("mlp")
        layers.append(PreNormBlock(norm(prefix + "norm1"), _mixer(width, layer["type"], layer["mixer"], prefix + "mix.", eps, tensor_shapes),
                                   norm(prefix + "norm2", optional=mlp is None), _feed_forward(width, mlp, prefix + "mlp.")))
        order.append(LayerCall(i, layer["mixer"].get("kv_from") if layer["type"] == "attention" else None))
    return DecoderModel(config=config, embedding=TokenEmbedding(config.vocab_size, width, name="embed", suffix=""),
                        layers=layers, order=order, final_norm=norm("final.norm"),
                        head=Linear(width, config.vocab_size, name="head", suffixes=BARE),
                        max_positions=config.max_positions, stream_dtype=torch.float32)


ARCHITECTURE = register(VirulixConfig.architecture, VirulixConfig.model_type, VirulixConfig, build_virulix, shape_aware=True)
