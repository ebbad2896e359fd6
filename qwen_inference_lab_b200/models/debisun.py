"""Debisun as an arrangement of parts, with the checkpoint's tensor names.

Layer i (tensors ``l<i>.*``) is pre-norm around an attention mixer and, where it has one, a feed-forward; the
norms are layer norms with weight and bias (``norm1``, ``norm1.b``), each branch joins the stream through a
learned scale per feature (``ls1``, ``ls2``), and after the feed-forward the layer adds an input from the token
itself (``side.*``, ``parts.side_input``).  The residual stream, the norms, attention scores and routers are
float32 whatever the activation dtype is.

``attention``  projections q, k, v without biases, each followed by a short causal convolution over time
               (``q.conv`` ...), no rotation; score = cap * tanh(q.k * scale / cap) + rel[row(i - j), h] with a
               table per layer whose rows stand for distances (``parts.attention.distance_rows``); a position sees
               its own chunk of ``mask.size`` positions; the softmax has a sink (one added to its denominator).
``dense``      down(relu(up x)^2).
``moe``        scores = softmax of the router over experts and identity outputs; the choice goes by score +
               ``correction``, the weights are the chosen scores, normalised and times ``router.scale``; experts
               ``e<k>`` are dense feed-forwards; identity outputs hand the input through; a shared expert
               (``shared``) runs for every token, times sigmoid(``shared.sg`` . x).
Then ``final.norm`` and ``head``.
"""
from __future__ import annotations

import torch

from ..config.model_config import DebisunConfig
from ..config.registry import register
from ..parts import (DecoderModel, GroupedQueryAttention, LayerCall, LayerNorm, Linear, Param, PlainMLP, PreNormBlock,
                     RoutedExperts, TokenEmbedding, TokenSideInput)

BARE = ("", ".b")            # this design's tensors carry the projection's own name; biases add ".b"
ACTIVATION = "relu2"         # of every feed-forward: the square of relu
DEFAULT_TABLE_ROWS = 32      # for random weights; a checkpoint's own ``rel`` tensor says it otherwise


def _feed_forward(width, mlp, prefix):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PlainMLP(width, mlp["ff"], names={k: prefix + k for k in ("up", "down")}, activation=ACTIVATION,
                        suffixes=BARE)
    router = mlp["router"]
    shared = None
    if mlp.get("shared"):
        shared = PlainMLP(width, mlp["shared"]["ff"], names={k: f"{prefix}shared.{k}" for k in ("up", "down")},
                          activation=ACTIVATION, suffixes=BARE)
    return RoutedExperts(width, mlp["expert"]["ff"], router["experts"], router["top"],
                         names=dict(router=prefix + "router", correction=prefix + "correction",
                                    expert=lambda index, which: f"{prefix}e{index}.{which}"),
                         activation=ACTIVATION, gated=False, routing="softmax_all",
                         weight_scale=router.get("scale", 1.0), identity=router.get("identity", 0), shared=shared,
                         shared_gate=prefix + "shared.sg" if shared is not None else None)


def _mixer(width, m, prefix, shapes):
    names = {k: prefix + k for k in ("q", "k", "v", "o")}
    names["distance_bias"] = prefix + "rel"
    rows = shapes[prefix + "rel"][0] if shapes and prefix + "rel" in shapes else m.get("bias_rows", DEFAULT_TABLE_ROWS)
    return GroupedQueryAttention(
        width, m["heads"], m["kv_heads"], m["dim"], names=names, bias=False, scale=m["scale"], v_head_dim=m["vdim"],
        suffixes=BARE, conv_taps=m.get("conv") or 0, conv_suffix=".conv", softcap=m.get("softcap") or 0.0,
        distance_bias=(rows, m["bias_max"]), chunk=(m.get("mask") or {}).get("size", 0), sink=True)


def build_debisun(config: DebisunConfig, tensor_shapes=None) -> DecoderModel:
    width, eps = config.width, config.eps
    norm = lambda name, optional=False: LayerNorm(width, eps, name=name, suffixes=BARE, optional=optional)
    side_table = Param((config.vocab_size, len(config.layers) * config.side_dim)) if config.side_dim else None
    layers = []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}."
        mlp = layer.get("mlp")
        after = []
        if side_table is not None:
            after.append(TokenSideInput(width, config.side_dim, i, eps, table=side_table, suffixes=BARE, norm_suffix="",
                                        names=dict(table="side.embed", gate=prefix + "side.gate",
                                                   proj=prefix + "side.proj", norm=prefix + "side.norm")))
        layers.append(PreNormBlock(norm(prefix + "norm1"), _mixer(width, layer["mixer"], prefix + "mix.", tensor_shapes),
                                   norm(prefix + "norm2", optional=mlp is None), _feed_forward(width, mlp, prefix + "mlp."),
                                   scales=(prefix + "ls1", prefix + "ls2"), after=after))
    return DecoderModel(config=config, embedding=TokenEmbedding(config.vocab_size, width, name="embed", suffix=""),
                        layers=layers, order=[LayerCall(i) for i in range(len(layers))], final_norm=norm("final.norm"),
                        head=Linear(width, config.vocab_size, name="head", suffixes=BARE),
                        max_positions=config.max_positions, stream_dtype=torch.float32)


ARCHITECTURE = register(DebisunConfig.architecture, DebisunConfig.model_type, DebisunConfig, build_debisun, shape_aware=True)
