"""Small Debisun configurations and random weights for the tests.

The sizes differ from layer to layer and between the cases: value heads larger and smaller than key heads and
equal to them, groups of one to four query heads per key/value head, one to five taps (one tap: no state at
all), chunks of 7 to 128 positions (odd ones too), distance tables of 8 to 32 rows, one to three experts per
token with and without identity outputs and a shared expert, a layer without a feed-forward, a model with and
one without the per-token side input.
"""
import json
from pathlib import Path

import torch

import qwen_inference_lab_b200.models  # noqa: F401  (registers the architectures)
from qwen_inference_lab_b200.config import registry
from qwen_inference_lab_b200.weights import write_safetensors
from tests.plain import debisun_plain as plain


def attention(heads, kv_heads, dim, vdim, scale, conv, softcap, bias_max, rows, chunk):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, conv=conv, softcap=softcap,
                bias_max=bias_max, bias_rows=rows, mask=dict(size=chunk))


def moe(experts, identity, top, scale, ff, shared=None):
    mlp = dict(kind="moe", router=dict(experts=experts, identity=identity, top=top, scale=scale), expert=dict(ff=ff))
    if shared:
        mlp["shared"] = dict(ff=shared)
    return mlp


CASE_A = dict(architecture="Debisun", vocab=211, width=80, norm=dict(eps=1e-5), token_side=dict(dim=8), layers=[
    dict(type="attention", mixer=attention(6, 2, 24, 40, 0.21, 4, 15.0, 100, 16, 48), mlp=moe(5, 2, 3, 1.7, 24, shared=40)),
    dict(type="attention", mixer=attention(4, 4, 16, 16, 0.3, 2, 30.0, 64, 8, 20), mlp=dict(kind="dense", ff=56)),
    dict(type="attention", mixer=attention(3, 1, 32, 8, 0.15, 3, 8.0, 300, 24, 64), mlp=None),
    dict(type="attention", mixer=attention(2, 2, 16, 24, 0.25, 1, 12.0, 30, 10, 7), mlp=moe(3, 0, 1, 1.0, 8)),
])
CASE_B = dict(architecture="Debisun", vocab=97, width=64, norm=dict(eps=1e-6), layers=[
    dict(type="attention", mixer=attention(2, 1, 80, 80, 0.1, 3, 50.0, 500, 32, 128), mlp=moe(7, 1, 2, 2.5, 32, shared=16)),
    dict(type="attention", mixer=attention(8, 2, 16, 16, 0.28, 5, 10.0, 40, 10, 33), mlp=dict(kind="dense", ff=40)),
])
# awkward sizes: nothing a multiple of 4 or 8, heads of 20 with values of 12, nine taps, a chunk of one position (a token sees
# itself and the sink), a chunk longer than every request, a table of four rows, every router output chosen, more
# identity outputs than experts, one head
CASE_C = dict(architecture="Debisun", vocab=53, width=70, norm=dict(eps=1e-5), token_side=dict(dim=3), layers=[
    dict(type="attention", mixer=attention(5, 5, 20, 12, 0.22, 9, 5.0, 9, 4, 1), mlp=moe(2, 3, 5, 0.6, 11, shared=9)),
    dict(type="attention", mixer=attention(1, 1, 48, 48, 0.14, 2, 40.0, 1000, 6, 4096), mlp=dict(kind="dense", ff=37)),
    dict(type="attention", mixer=attention(6, 3, 10, 14, 0.3, 3, 9.0, 50, 12, 17), mlp=moe(6, 0, 2, 1.3, 10)),
])
CASES = {"A": dict(config=CASE_A, seed=5, page_size=4, lengths=(70, 9, 33, 120, 1, 50)),
         "B": dict(config=CASE_B, seed=6, page_size=16, lengths=(40, 3, 150, 64, 25)),
         "C": dict(config=CASE_C, seed=7, page_size=2, lengths=(31, 2, 77, 20, 45))}


def make_weights(config: dict, seed: int) -> dict:
    """Checkpoint name -> CPU float32 tensor holding bfloat16-representable values: norm weights and layer scales
    around one, norm biases and corrections small, distance tables and routers wide enough to matter."""
    entry = registry.lookup(config)
    model = entry.build(entry.config_class.from_dict(config))
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, param in model.all_named_params().items():
        draw = torch.randn(param.shape, generator=generator)
        leaf = name.split(".")[-1]
        if name.endswith(".b"):
            value = draw * 0.1
        elif leaf in ("norm1", "norm2", "norm") or name == "final.norm":
            value = 1.0 + draw * 0.1
        elif leaf in ("ls1", "ls2"):
            value = 0.7 + draw * 0.2
        elif leaf == "rel":
            value = draw
        elif leaf == "conv":
            value = draw * 0.6
        elif leaf == "correction":
            value = draw * 0.05
        elif leaf == "router":
            value = draw * 0.5
        elif leaf == "embed":
            value = draw
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
    """{(id, position): logits row} of the plain implementation (float64 arithmetic; with ``low`` float32
    arithmetic that rounds what the design allows in bfloat16)."""
    rows = {}
    for rid, tokens in requests.items():
        logits = plain.forward(config, weights, tokens, torch.float64 if low is None else torch.float32, low)
        for position in range(len(tokens)):
            rows[(rid, position)] = logits[position].float()
    return rows


CLOSE_CALL = 0.1       # a router margin below this fraction of the score is a choice that bfloat16 rounding can flip


def close_calls(requests, weights, config):
    """The (id, position) whose choice of experts is a close call in some layer: bfloat16 runs are not judged
    there (another expert is another function; the float32 runs are judged everywhere)."""
    found = set()
    for rid, tokens in requests.items():
        margins = []
        plain.forward(config, weights, tokens, torch.float64, margins=margins)
        if margins:
            smallest = torch.stack(margins).min(dim=0).values
            found |= {(rid, int(p)) for p in (smallest < CLOSE_CALL).nonzero().flatten()}
    return found
