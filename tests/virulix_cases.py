"""Small Virulix configurations and random weights for the tests.

The sizes differ from layer to layer and between the cases: value heads of another size than key heads,
groups of one, two and three query heads per key/value head, one to three experts per token, layers with and
without a shared expert, a layer without a feed-forward, a layer that reads another layer's pages, a
recurrent state that one block holds and one that is spread over several.
"""
import json
from pathlib import Path

import torch

import qwen_inference_lab_b200.models  # noqa: F401  (registers the architectures)
from qwen_inference_lab_b200.config import registry
from qwen_inference_lab_b200.weights import write_safetensors
from tests.plain import virulix_plain as plain


def attention(heads, kv_heads, dim, vdim, scale, q_temp=None, kv_from=None):
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if q_temp:
        mixer["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def moe(experts, top, ff, limit, shared=None):
    mlp = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=limit))
    if shared:
        mlp["shared"] = dict(ff=shared[0], limit=shared[1])
    return mlp


CASE_A = dict(architecture="Virulix", vocab=211, width=80, norm=dict(eps=1e-5), layers=[
    dict(type="gla", mixer=dict(heads=3, dim=24, vdim=40, tau=7.0), mlp=moe(5, 2, 24, 1.5, shared=(40, 0.7))),
    dict(type="attention", mixer=attention(6, 2, 24, 40, 0.31, q_temp=(0.4, 5)), mlp=dict(kind="dense", ff=56)),
    dict(type="attention", mixer=attention(6, 2, 24, 40, 0.2, kv_from=1), mlp=None),
    dict(type="gla", mixer=dict(heads=1, dim=72, vdim=16, tau=3.0, rank=5), mlp=moe(3, 1, 16, 4.0)),
    dict(type="attention", mixer=attention(4, 4, 16, 16, 0.25, q_temp=(1.5, 1)), mlp=moe(4, 3, 8, 0.9, shared=(8, 2.0))),
])
# a state too wide for one block (320 value columns), heads of 80 with values of 8, one key/value head
CASE_B = dict(architecture="Virulix", vocab=97, width=64, norm=dict(eps=1e-6), layers=[
    dict(type="attention", mixer=attention(2, 1, 80, 8, 0.11, q_temp=(0.25, 16)), mlp=moe(7, 2, 32, 2.0, shared=(16, 1.0))),
    dict(type="gla", mixer=dict(heads=1, dim=8, vdim=320, tau=16.0, rank=3), mlp=dict(kind="dense", ff=40)),
    dict(type="gla", mixer=dict(heads=2, dim=40, vdim=24, tau=2.0), mlp=None),
])
CASES = {"A": dict(config=CASE_A, seed=5, page_size=4, lengths=(70, 9, 33, 120, 1, 50)),
         "B": dict(config=CASE_B, seed=6, page_size=16, lengths=(40, 3, 150, 64, 25))}


def make_weights(config: dict, seed: int) -> dict:
    """Checkpoint name -> CPU float32 tensor holding bfloat16-representable values.  Norm weights lie
    around zero (the design adds one), biases are not zero, routers are wide enough to choose clearly."""
    entry = registry.lookup(config)
    model = entry.build(entry.config_class.from_dict(config))
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, param in model.all_named_params().items():
        draw = torch.randn(param.shape, generator=generator)
        leaf = name.split(".")[-1]
        if name.endswith(".b"):
            value = draw * (1.0 if "router" in name or ".a2" in name else 0.1)
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            value = draw * 0.1
        elif leaf == "norm":
            value = 1.0 + draw * 0.1
        elif leaf == "router":
            value = draw * 0.5
        elif leaf == "embed":
            value = draw
        elif leaf == "a2":
            value = draw * 0.8
        else:
            value = draw * (param.shape[-1] ** -0.5)
        weights[name] = value.to(torch.bfloat16).float()
    return weights


def write_folder(config: dict, seed: int, folder) -> dict:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    weights = make_weights(config, seed)
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(folder / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return weights


def random_tokens(config, count, seed):
    return torch.randint(0, config["vocab"], (count,), generator=torch.Generator().manual_seed(seed)).tolist()


def plain_rows(requests, weights, config, low=None):
    """{(id, position): logits row} of the plain implementation (float32 arithmetic; ``low`` rounds what the
    design allows in bfloat16)."""
    rows = {}
    for rid, tokens in requests.items():
        logits = plain.forward(tokens, weights, config, torch.float32, low)
        for position in range(len(tokens)):
            rows[(rid, position)] = logits[position].float()
    return rows
