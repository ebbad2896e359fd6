"""Virulix on the GPU: every mechanism alone against its plain function, then whole models under four ways of
cutting the work, long decoding, slots and pages used again, generation through the engine and the replay program."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import harness
from tests import virulix_cases as cases
from tests.plain import virulix_plain as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["float32", "bfloat16"]


def low_of(dtype):
    return None if dtype == torch.float32 else torch.bfloat16


def close(actual, expected, dtype, scale=1.0):
    """float32: element by element.  bfloat16: the expected rows carry the plain implementation's own bfloat16
    roundings, and a sum taken in another order lands an ulp of the largest term away, so the bar is on the
    root mean square of the difference (1 % of the rows' own) and on the largest one (5 % of the largest value)."""
    actual, expected = actual.float().cpu(), expected.float()
    if dtype == torch.float32:
        torch.testing.assert_close(actual, expected, atol=2e-5 * scale, rtol=2e-5)
        return
    assert torch.isfinite(actual).all()
    difference = actual - expected
    assert difference.pow(2).mean().sqrt() <= 0.01 * expected.pow(2).mean().sqrt(), \
        f"rms difference {difference.pow(2).mean().sqrt():.3e} against rows of {expected.pow(2).mean().sqrt():.3e}"
    assert difference.abs().max() <= 0.05 * expected.abs().max(), \
        f"largest difference {difference.abs().max():.3e} against a largest value of {expected.abs().max():.3e}"


def fill(part, seed, dtype, scales=None):
    """Random parameters, bfloat16-representable; returns name -> CPU float32."""
    generator = torch.Generator().manual_seed(seed)
    values = {}
    for name, param in part.all_named_params().items():
        std = (scales or {}).get(name.split(".")[-1], param.shape[-1] ** -0.5 if len(param.shape) > 1 else 0.3)
        value = (torch.randn(param.shape, generator=generator) * std).to(torch.bfloat16)
        values[name] = value.float()
        param.data = value.to(dtype).cuda()
    part.finalize(torch.device("cuda"), dtype)
    return values


def rows(count, width, seed):
    return (torch.randn(count, width, generator=torch.Generator().manual_seed(seed))).to(torch.bfloat16).float()


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_exact_norm_of_a_float32_stream(dtype):
    from qwen_inference_lab_b200.kernels import ops
    x = torch.randn(7, 100, generator=torch.Generator().manual_seed(0)) * 3
    w = (torch.randn(100, generator=torch.Generator().manual_seed(1)) * 0.2).to(torch.bfloat16).float()
    out = ops.rmsnorm_exact(x.cuda(), w.to(dtype).cuda(), 1e-3, 1.0, out_dtype=dtype)
    assert out.dtype == dtype
    expected = plain.offset_rms_norm(x, w, 1e-3)
    close(out, expected if dtype == torch.float32 else expected.to(torch.bfloat16), dtype, scale=0.1)
    picked = ops.rmsnorm_exact(x.cuda(), w.to(dtype).cuda(), 1e-3, 0.0, out_dtype=torch.float32,
                               rows=torch.tensor([5, 0], dtype=torch.int32, device="cuda"))
    close(picked, plain.plain_rms_norm(x[[5, 0]], w, 1e-3), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("kind", ["silu", "gelu_tanh", "clamped_swish"])
def test_gated_activations(dtype, kind):
    from qwen_inference_lab_b200.kernels import ops
    gate_up = rows(11, 2 * 37, 3) * 2
    g, u = gate_up[:, :37], gate_up[:, 37:]
    if kind == "silu":
        expected = g * torch.sigmoid(g) * u
    elif kind == "gelu_tanh":
        expected = plain.gelu_tanh(g) * u
    else:
        gc, uc = g.clamp(max=1.25), u.clamp(-1.25, 1.25)
        expected = gc * torch.sigmoid(1.702 * gc) * (uc + 1)
    out = ops.gated_activation(gate_up.to(dtype).cuda(), kind, limit=1.25, alpha=1.702)
    close(out, expected, dtype, scale=0.5)


def attention_part(dtype, heads=6, kv_heads=2, dim=24, vdim=40, hidden=64, temperature=(0.4, 5), seed=1):
    from qwen_inference_lab_b200.parts import GroupedQueryAttention
    from qwen_inference_lab_b200.models.virulix import BARE, distance_slopes
    part = GroupedQueryAttention(hidden, heads, kv_heads, dim, names={k: "m." + k for k in "qkvo"}, bias=True,
                                 out_bias=False, scale=0.3, v_head_dim=vdim, distance_slopes=distance_slopes(heads),
                                 q_temperature=temperature, suffixes=BARE)
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=0.3)
    if temperature:
        mixer["q_temp"] = dict(coef=temperature[0], every=temperature[1])
    return part, fill(part, seed, dtype), mixer


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("shape", [dict(), dict(heads=3, kv_heads=3, dim=16, vdim=16, temperature=None),
                                   dict(heads=4, kv_heads=1, dim=8, vdim=72, temperature=(2.0, 1))])
def test_attention_mixer_whole_cut_and_side_by_side(dtype, shape):
    """Value heads larger and smaller than key heads, groups of 1, 3 and 4, with and without the temperature; two
    requests of unequal length share every step, cut into portions down to one token."""
    part, w, mixer = attention_part(dtype, **shape)
    x = {"a": rows(45, 64, 10), "b": rows(19, 64, 11)}
    expected = {rid: plain.attention_mixer(v, w, "m.", mixer, low=low_of(dtype))[0] for rid, v in x.items()}
    body = lambda ctx, h, view: part.forward(ctx, h, view)
    for cuts in ({"a": [45], "b": [19]}, {"a": [7, 2, 1, 20, 1, 1, 13], "b": [1, 2, 16]}):
        out = harness.run_part(part, 64, dtype, body, x, cuts, page_size=4, num_pages=20)
        for rid in x:
            close(out[rid], expected[rid], dtype, scale=0.3)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("far", [0, 3, 4, 127, 128, 129, 255, 256])
def test_a_far_key_that_outweighs_its_distance(dtype, far):
    """One key far back (at a page's first or last slot, at the edge of a key tile, the very first token) points
    along the last query with a length that beats the distance bias: the output must be that key's value.  Pages
    are shuffled and the rest of the pool is NaN."""
    from qwen_inference_lab_b200.kernels import ops
    heads, kv_heads, d, e, page, T = 4, 2, 16, 24, 4, 300
    g = torch.Generator().manual_seed(far)
    q = torch.randn(T, heads, d, generator=g).to(torch.bfloat16).float()
    k = (torch.randn(T, kv_heads, d, generator=g) * 0.1).to(torch.bfloat16).float()
    v = torch.randn(T, kv_heads, e, generator=g).to(torch.bfloat16).float()
    slopes = plain.distance_slopes(heads).float()
    # the steepest head loses 0.25 a position: the key gets what that costs over its distance and 20 more
    for kv in range(kv_heads):
        direction = q[T - 1, kv * 2] / q[T - 1, kv * 2].norm()
        k[far, kv] = (direction * ((0.25 * (T - 1 - far) + 20) / (0.5 * q[T - 1, kv * 2].norm()))).to(torch.bfloat16).float()
    expected = plain.biased_attention(q, k, v, 0.5)
    assert (expected[T - 1, 0] - v[far, 0]).abs().max() < 1e-3           # head 0 sees nothing but the far key
    n_pages = T // page
    order = torch.randperm(n_pages + 9, generator=g)[:n_pages]
    pool = torch.full((n_pages + 9, kv_heads * page * (d + e)), float("nan"))
    for position in range(T):
        base = pool[order[position // page]]
        for kv in range(kv_heads):
            at = (kv * page + position % page) * d
            base[at:at + d] = k[position, kv]
            at = kv_heads * page * d + (kv * page + position % page) * e
            base[at:at + e] = v[position, kv]
    table = torch.full((2, n_pages + 3), -1, dtype=torch.int32)
    table[1, :n_pages] = order.int()
    picks = torch.tensor([T - 1, far, max(far - 1, 0), min(far + 1, T - 1), 0, 150], dtype=torch.int64)
    out = torch.empty(len(picks), heads * e, dtype=dtype, device="cuda")
    ops.attention_generic(q[picks].reshape(len(picks), -1).to(dtype).cuda().contiguous(), pool.to(dtype).cuda(), out,
                          picks.int().cuda(), torch.ones(len(picks), dtype=torch.int32, device="cuda"), table.cuda(),
                          heads, kv_heads, d, page, 0, 0.5, v_dim=e, slopes=slopes.cuda())
    close(out, expected[picks].reshape(len(picks), -1), dtype, scale=0.3)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("query", [259, 299])
@pytest.mark.parametrize("far", [0, 5, 63, 64, 127, 128, 200])
def test_a_far_key_through_the_mixer_in_prompts_and_in_decoding(dtype, far, query):
    """The same through the mixer (in bfloat16 with equal head sizes: the tensor-core kernels): projections that
    copy slices of the input, so that the test sets queries, keys and values through it.  The far key stands out
    for the query at position 259 (inside a prompt portion) or 299 (a single decoded token)."""
    from qwen_inference_lab_b200.parts import GroupedQueryAttention
    from qwen_inference_lab_b200.models.virulix import BARE, distance_slopes
    heads, kv_heads, d, T = 4, 2, 16, 300
    part = GroupedQueryAttention(128, heads, kv_heads, d, names={k: "m." + k for k in "qkvo"}, bias=True, out_bias=False,
                                 scale=0.5, v_head_dim=d, distance_slopes=distance_slopes(heads), suffixes=BARE)
    eye = torch.eye(128)
    values = {"m.q": eye[:64], "m.k": eye[64:96], "m.v": eye[96:128], "m.o": torch.eye(128)[:, :64].contiguous(),
              "m.q.b": torch.zeros(64), "m.k.b": torch.zeros(32), "m.v.b": torch.zeros(32)}
    for name, param in part.all_named_params().items():
        param.data = values[name].to(dtype).cuda()
    part.finalize(torch.device("cuda"), dtype)
    g = torch.Generator().manual_seed(far)
    x = torch.randn(T, 128, generator=g)
    x[:, 64:96] *= 0.1
    x = x.to(torch.bfloat16).float()
    for kv in range(kv_heads):
        q = x[query, kv * 32:kv * 32 + 16]
        x[far, 64 + kv * 16:64 + (kv + 1) * 16] = q / q.norm() * ((0.25 * (query - far) + 20) / (0.5 * q.norm()))
    x = x.to(torch.bfloat16).float()
    q, k, v = x[:, :64].reshape(T, heads, d), x[:, 64:96].reshape(T, kv_heads, d), x[:, 96:].reshape(T, kv_heads, d)
    expected = plain.biased_attention(q, k, v, 0.5).reshape(T, 64)
    assert (expected[query, :16] - v[far, 0]).abs().max() < 0.01        # head 0 sees nothing but the far key
    body = lambda ctx, h, view: part.forward(ctx, h, view)
    cuts = [70, 130, 3, 2, 60, 1, 1] + [1] * 33
    out = harness.run_part(part, 128, dtype, body, {"a": x}, {"a": cuts}, page_size=16, num_pages=24)["a"]
    close(out[:, :64], expected, dtype, scale=0.3)
    assert out[:, 64:].abs().max() == 0


def test_heads_of_128_take_the_tensor_memory_kernel_with_the_distance_bias(monkeypatch):
    """Whole 128-token tiles of a prompt go to the tcgen05 kernel, which takes the slopes too; the leftovers and single
    tokens to the tiled ones.  The far key of the test above would be too blunt here: random rows, every position."""
    from qwen_inference_lab_b200.kernels import attention_tc
    calls = []
    original = attention_tc.prefill
    monkeypatch.setattr(attention_tc, "prefill", lambda *a, **k: (calls.append(k.get("slopes_log2") is not None), original(*a, **k))[1])
    part, w, mixer = attention_part(torch.bfloat16, heads=4, kv_heads=2, dim=128, vdim=128, temperature=(0.3, 64))
    x = {"a": rows(330, 64, 12), "b": rows(140, 64, 13)}
    expected = {rid: plain.attention_mixer(v, w, "m.", mixer, low=torch.bfloat16)[0] for rid, v in x.items()}
    body = lambda ctx, h, view: part.forward(ctx, h, view)
    for cuts in ({"a": [330], "b": [140]}, {"a": [129, 1, 200], "b": [7, 133]}):
        out = harness.run_part(part, 64, torch.bfloat16, body, x, cuts, page_size=16, num_pages=40)
        for rid in x:
            close(out[rid], expected[rid], torch.bfloat16)
    assert calls and all(calls)


def gla_part(dtype, heads, d, e, rank, tau, hidden=48, seed=2):
    from qwen_inference_lab_b200.parts import GatedLinearAttention
    from qwen_inference_lab_b200.models.virulix import BARE
    names = {k: "m." + k for k in ("q", "k", "v", "g", "o", "a1", "a2", "norm")}
    part = GatedLinearAttention(hidden, heads, d, e, rank, tau=tau, norm_eps=1e-5, names=names, suffixes=BARE, norm_suffix="")
    w = fill(part, seed, dtype, scales={"a2": 1.0, "b": 1.5, "norm": 1.0})
    return part, w, dict(heads=heads, dim=d, vdim=e, tau=tau)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("shape", [dict(heads=2, d=32, e=48, rank=12, tau=9.0), dict(heads=3, d=24, e=40, rank=4, tau=1.0),
                                   dict(heads=1, d=72, e=16, rank=7, tau=5.0), dict(heads=1, d=8, e=320, rank=2, tau=3.0),
                                   dict(heads=2, d=130, e=72, rank=9, tau=8.0)])
def test_gla_mixer_whole_cut_and_side_by_side(dtype, shape):
    """States that one block holds (alone in a thread, or split over 2, 4 and 8 threads a column) and one whose
    value columns are spread over blocks; portions down to one token beside another request's."""
    part, w, mixer = gla_part(dtype, **shape)
    x = {"a": rows(50, 48, 20), "b": rows(23, 48, 21)}
    expected = {rid: plain.gla_mixer(v, w, "m.", mixer, 1e-5, low=low_of(dtype)) for rid, v in x.items()}
    body = lambda ctx, h, view: part.forward(ctx, h, view)
    whole = harness.run_part(part, 48, dtype, body, x, {"a": [50], "b": [23]})
    cut = harness.run_part(part, 48, dtype, body, x, {"a": [9, 2, 1, 1, 17, 8, 12], "b": [1, 1, 2, 19]})
    for rid in x:
        close(whole[rid], expected[rid], dtype, scale=0.3)
        close(cut[rid], expected[rid], dtype, scale=0.3)
        if dtype == torch.float32:
            assert torch.equal(whole[rid], cut[rid]), "the scan takes tokens one by one: a cut must not change a bit"


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("shape", [dict(heads=2, d=32, e=48, rank=12, tau=9.0), dict(heads=1, d=40, e=300, rank=3, tau=4.0)])
def test_gla_long_portions_run_as_chunks_side_by_side(dtype, shape):
    """Portions of more than 128 tokens are cut into chunks of 64 whose states are carried over: 129 tokens (a last
    chunk of one token), 300 after a cached prefix, a long portion beside a short one and a single token; against
    the plain recurrence, and against the token-by-token path in float32 to rounding."""
    part, w, mixer = gla_part(dtype, **shape)
    x = {"a": rows(480, 48, 22), "b": rows(200, 48, 23)}
    expected = {rid: plain.gla_mixer(v, w, "m.", mixer, 1e-5, low=low_of(dtype)) for rid, v in x.items()}
    body = lambda ctx, h, view: part.forward(ctx, h, view)
    chunked = harness.run_part(part, 48, dtype, body, x, {"a": [129, 300, 1, 50], "b": [7, 192, 1]}, num_pages=200)
    stepwise = harness.run_part(part, 48, dtype, body, x, {"a": [120] * 4, "b": [100, 100]}, num_pages=200)
    for rid in x:
        close(chunked[rid], expected[rid], dtype, scale=0.3)
        close(stepwise[rid], expected[rid], dtype, scale=0.3)
        if dtype == torch.float32:
            torch.testing.assert_close(chunked[rid], stepwise[rid], atol=2e-5, rtol=2e-5)


def test_gla_state_decays_as_the_product_of_its_decays():
    """A first token with a large key and value, then tokens with keys of zero: what is read later is the first
    token's outer product times the product of the decays since, channel by channel."""
    from qwen_inference_lab_b200.kernels import ops
    heads, d, e, rank, T = 1, 4, 3, 2, 40
    g = torch.Generator().manual_seed(4)
    width = 2 * d + 2 * e + rank
    projected = torch.zeros(T, width)
    projected[:, :d] = 1.0                                   # q: reads every channel
    projected[0, d:2 * d] = torch.tensor([1.0, 2.0, 3.0, 4.0])   # k of the first token only
    projected[0, 2 * d:2 * d + e] = torch.tensor([1.0, -1.0, 0.5])
    projected[:, 2 * d + e:2 * d + 2 * e] = 30.0             # gate: silu(30) = 30
    projected[:, -rank:] = torch.randn(T, rank, generator=g)
    a2, bias = torch.randn(d, rank, generator=g), torch.randn(d, generator=g) + 2
    alpha = torch.sigmoid(projected[:, -rank:] @ a2.t() + bias) ** (1 / 3.0)
    state = torch.zeros(2, heads, d, e, device="cuda")
    out = torch.empty(T, e, device="cuda")
    seg = lambda *v: torch.tensor(v, dtype=torch.int32, device="cuda")
    decays = ops.gla_decay(projected.cuda(), 2 * d + 2 * e, a2.cuda(), bias.cuda(), 3.0)
    torch.testing.assert_close(decays.cpu(), alpha, atol=1e-6, rtol=1e-5)
    ops.gla_scan(projected.cuda(), (0, d, 2 * d, 2 * d + e), decays, 1.0, torch.ones(e, device="cuda"), 0.0, state,
                 seg(0), seg(T), seg(1), 1, heads, d, e, out)
    decay = torch.cumprod(alpha[1:], dim=0)
    for t in (1, 7, T - 1):
        o = (decay[t - 1] * projected[0, d:2 * d]).sum() * projected[0, 2 * d:2 * d + e]
        expected = o / o.pow(2).mean().sqrt() * 30.0
        torch.testing.assert_close(out[t].cpu(), expected, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(state[1, 0].cpu(), (decay[-1] * projected[0, d:2 * d])[:, None] * projected[0, 2 * d:2 * d + e][None, :],
                               atol=1e-5, rtol=1e-4)
    assert state[0].abs().max() == 0


def experts_part(dtype, experts, top, shared, hidden=40, ff=24, seed=3):
    from qwen_inference_lab_b200.parts import GatedMLP, RoutedExperts
    from qwen_inference_lab_b200.models.virulix import BARE, SWISH_ALPHA
    shared_part = GatedMLP(hidden, 16, names={k: f"f.shared.{k}" for k in ("gate", "up", "down")}, activation="clamped_swish",
                           limit=0.8, alpha=SWISH_ALPHA, suffixes=BARE) if shared else None
    part = RoutedExperts(hidden, ff, experts, top, names=dict(router="f.router", router_bias="f.router.b",
                                                               expert=lambda i, which: f"f.e{i}.{which}"),
                         activation="clamped_swish", limit=1.1, alpha=SWISH_ALPHA, shared=shared_part)
    w = fill(part, seed, dtype, scales={"router": 0.7, "b": 0.7})
    mlp = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=1.1))
    if shared:
        mlp["shared"] = dict(ff=16, limit=0.8)
    return part, w, mlp


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("experts,top,shared", [(5, 2, True), (3, 1, False), (11, 3, True), (4, 4, False), (70, 5, False)])
def test_routed_experts_alone_and_in_a_batch(dtype, experts, top, shared):
    from qwen_inference_lab_b200.kernels import ops
    part, w, mlp = experts_part(dtype, experts, top, shared)
    x = rows(150, 40, 30)
    chosen, weights = ops.moe_route(x.to(dtype).cuda(), part.router.data, part.router_bias.data, top)
    want_chosen, want_weights = plain.route(x, w, "f.", top)
    assert torch.equal(chosen.cpu().long(), want_chosen), "the router's choice (no close calls among these logits)"
    torch.testing.assert_close(weights.cpu(), want_weights, atol=1e-5, rtol=1e-5)
    assert len(set(want_chosen.flatten().tolist())) >= min(experts, 11), "most experts should be in use"
    expected = plain.routed_feed_forward(x, w, "f.", mlp, low=low_of(dtype))
    body = lambda ctx, h, view: part.forward(ctx, h)
    together = harness.run_part(part, 40, dtype, body, {"a": x[:99], "b": x[99:]}, {"a": [99], "b": [51]})
    close(torch.cat((together["a"], together["b"])), expected, dtype, scale=0.3)
    alone = harness.run_part(part, 40, dtype, body, {"b": x[99:]}, {"b": [3, 1, 47]})
    if dtype == torch.float32:
        assert torch.equal(alone["b"], together["b"]), "a token's experts do not depend on the rest of the batch"
    else:       # the shared expert's products take another kernel for three rows than for a hundred: rounding only
        close(alone["b"], together["b"], dtype)


def test_routed_experts_group_many_pairs():
    """More pairs than the one-block grouping takes: the placement by atomic cursors gives the same sums."""
    part, w, mlp = experts_part(torch.float32, 6, 3, False)
    x = rows(1500, 40, 31)
    body = lambda ctx, h, view: part.forward(ctx, h)
    many = harness.run_part(part, 40, torch.float32, body, {"a": x}, {"a": [1500]}, num_pages=400)["a"]
    few = harness.run_part(part, 40, torch.float32, body, {"a": x}, {"a": [500, 500, 500]}, num_pages=400)["a"]
    assert torch.equal(many, few)
    close(many[:40], plain.routed_feed_forward(x[:40], w, "f.", mlp), torch.float32, scale=0.3)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_dense_feed_forward_with_biases(dtype):
    from qwen_inference_lab_b200.parts import GatedMLP
    from qwen_inference_lab_b200.models.virulix import BARE
    part = GatedMLP(40, 56, names={k: "f." + k for k in ("gate", "up", "down")}, activation="gelu_tanh", bias=True, suffixes=BARE)
    w = fill(part, 7, dtype)
    x = rows(33, 40, 32)
    out = harness.run_part(part, 40, dtype, lambda ctx, h, view: part.forward(ctx, h), {"a": x}, {"a": [20, 13]})["a"]
    close(out, plain.dense_feed_forward(x, w, "f.", low=low_of(dtype)), dtype, scale=0.3)


def test_a_float32_residual_under_bfloat16_products():
    """The stream stays float32: what a projection adds is not rounded to bfloat16 on its way in."""
    from qwen_inference_lab_b200.parts import Linear
    part = Linear(64, 48, name="p", bias=True)
    w = fill(part, 8, torch.bfloat16)
    for count in (5, 40):                      # the weight-streaming kernel and the library product
        x = rows(count, 64, 33)
        stream = torch.randn(count, 48, generator=torch.Generator().manual_seed(1)) * 50
        out = part.forward(None, x.to(torch.bfloat16).cuda(), residual=stream.cuda().clone())
        assert out.dtype == torch.float32
        expected = stream + x @ w["p.weight"].t() + w["p.bias"]
        torch.testing.assert_close(out.cpu(), expected, atol=2e-4, rtol=1e-5)


# ------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    result = {}
    for name, case in cases.CASES.items():
        folder = tmp_path_factory.mktemp(f"virulix{name}")
        weights = cases.write_folder(case["config"], case["seed"], folder)
        requests = {f"r{i}": cases.random_tokens(case["config"], n, 60 + i) for i, n in enumerate(case["lengths"])}
        result[name] = (folder, weights, requests)
    return result


@pytest.fixture(scope="module")
def truth(folders):
    """The plain rows of every case, float32 and with bfloat16 roundings: computed once."""
    return {name: (cases.plain_rows(requests, weights, cases.CASES[name]["config"]),
                   cases.plain_rows(requests, weights, cases.CASES[name]["config"], torch.bfloat16))
            for name, (folder, weights, requests) in folders.items()}


SCHEDULES = {"whole": harness.whole_schedule, "tail_decode": harness.tail_decode_schedule,
             "chunks": harness.chunk_schedule, "mixed": harness.mixed_schedule}


def replay(folders, case, schedule_name, dtype):
    folder, weights, requests = folders[case]
    page_size = cases.CASES[case]["page_size"]
    schedule = SCHEDULES[schedule_name](requests)
    num_pages = harness.peak_pages(schedule, page_size) + 1
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=num_pages, page_size=page_size)
    for _, _, tensor in cache.state_groups:
        tensor.fill_(float("nan"))             # a slot that is not zeroed at admission shows
    ledger = harness.PageLedger(cache)
    actual = harness.run_schedule(runner, cache, schedule, ledger)
    assert cache.free_pages() == num_pages and not cache.owners()
    assert ledger.handovers > 0, "no page was used again by another request: the pool is too large"
    return actual


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("case", list(cases.CASES))
def test_replay_matches_plain(folders, truth, case, schedule, dtype):
    actual = replay(folders, case, schedule, dtype)
    expected, low = truth[case]
    harness.assert_rows_close(actual, expected, dtype, f"virulix {case} {schedule} {dtype}",
                              low if dtype == torch.bfloat16 else None)


@pytest.mark.parametrize("case", list(cases.CASES))
def test_float32_rows_are_the_same_bits_under_every_schedule(folders, case):
    """Requests of up to 128 tokens take the recurrence token by token under every schedule: not a bit may differ.
    A longer prompt in one piece runs its recurrence as chunks side by side, which rounds differently."""
    runs = {name: replay(folders, case, name, torch.float32) for name in SCHEDULES}
    lengths = {rid: len(tokens) for rid, tokens in folders[case][2].items()}
    for name, got in runs.items():
        exact = [key for key in sorted(got) if lengths[key[0]] <= 128]
        different = [key for key in exact if not torch.equal(got[key], runs["whole"][key])]
        assert exact and not different, \
            f"virulix {case}: {len(different)} rows of schedule {name} differ from the whole run, first {different[0]}"
        for key in sorted(got):
            torch.testing.assert_close(got[key], runs["whole"][key], atol=5e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_and_the_first_tokens(folders, dtype):
    """Three tokens as a prompt, then 300 single tokens (recorded graphs, two context buckets would need more:
    here the state and the pages carry everything), every position judged."""
    folder, weights, _ = folders["B"]
    config = cases.CASE_B
    tokens = cases.random_tokens(config, 303, 99)
    schedule = [([("r", tokens[:3], [0, 1, 2])], [])]
    schedule += [([("r", [tokens[i]], [0])], ["r"] if i == 302 else []) for i in range(3, 303)]
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=20, page_size=16)
    actual = harness.run_schedule(runner, cache, schedule)
    assert runner._graphs, "single-token steps should have been recorded"
    expected = cases.plain_rows({"r": tokens}, weights, config)
    low = cases.plain_rows({"r": tokens}, weights, config, torch.bfloat16) if dtype == torch.bfloat16 else None
    harness.assert_rows_close(actual, expected, dtype, f"virulix long decoding {dtype}", low)


def test_a_state_slot_and_pages_that_another_request_used_before(folders):
    """"x" runs and ends; "y" takes its slot and its pages: its logits are those of "y" in a fresh cache, bit for bit."""
    folder, weights, _ = folders["A"]
    config = cases.CASE_A
    x, y = cases.random_tokens(config, 37, 1), cases.random_tokens(config, 29, 2)
    def run(first):
        _, cache, runner = harness.build_engine_parts(folder, torch.float32, num_pages=12, page_size=4, max_requests=1)
        schedule = []
        if first:
            schedule += [([("x", x[:30], [])], [])] + [([("x", [t], [0])], []) for t in x[30:]]
            schedule[-1] = (schedule[-1][0], ["x"])
        schedule += [([("y", y[:11], list(range(11)))], []), ([("y", y[11:13], [0, 1])], [])]
        schedule += [([("y", [t], [0])], []) for t in y[13:]]
        schedule[-1] = (schedule[-1][0], ["y"])
        got = harness.run_schedule(runner, cache, schedule)
        return torch.stack([got[("y", p)] for p in range(len(y))])
    assert torch.equal(run(first=True), run(first=False))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_greedy_generation_through_the_engine(folders, dtype):
    """Prompts of unequal length through ``Engine.generate`` (scheduler, chunked prompts, sampler): every token is
    the plain implementation's best one, or in bfloat16 inside what bfloat16 costs the plain implementation."""
    from qwen_inference_lab_b200 import Engine, load_model
    folder, weights, _ = folders["A"]
    config = cases.CASE_A
    model = load_model(folder, device="cuda", dtype=dtype)
    engine = Engine(model, num_pages=48, page_size=4, token_budget=24, prefill_chunk=10, max_active=3)
    prompts = [cases.random_tokens(config, n, 40 + n) for n in (2, 31, 17, 5)]
    results = engine.generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert engine.idle and engine.cache.free_pages() == 48
    for prompt, row in zip(prompts, results):
        assert len(row["token_ids"]) == 12
        sequence = list(prompt)
        for token in row["token_ids"]:
            logits = plain.forward(sequence, weights, config)[-1]
            best = int(logits.argmax())
            if token != best:
                assert dtype == torch.bfloat16, f"token {token} instead of {best} after {len(sequence)} tokens"
                noise = (plain.forward(sequence, weights, config, low=torch.bfloat16)[-1] - logits).abs().max().item()
                assert float(logits[best] - logits[token]) < 4 * noise
            sequence.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_replays_a_mixed_schedule(folders, truth, tmp_path, dtype):
    folder, weights, requests = folders["B"]
    schedule = harness.mixed_schedule(requests)
    peak = harness.peak_pages(schedule, 64, round_to=64) * 64
    process = subprocess.Popen([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                                "--out", str(tmp_path / "out"), "--max-tokens", str(peak), "--max-live", "4"],
                               stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    got, position = {}, {}
    for number, (entries, ended) in enumerate(schedule):
        step = dict(step=number, entries=[dict(id=rid, tokens=tokens, want=want) for rid, tokens, want in entries], end=ended)
        process.stdin.write(json.dumps(step) + "\n")
        process.stdin.flush()
        assert process.stdout.readline().strip() == f"done {number}"
        wanted = [(rid, position.get(rid, 0) + w) for rid, tokens, want in entries for w in want]
        data = np.fromfile(tmp_path / "out" / f"{number}.f32", dtype="<f4").reshape(len(wanted), cases.CASE_B["vocab"])
        for key, row in zip(wanted, data):
            got[key] = torch.from_numpy(row.copy())
        for rid, tokens, _ in entries:
            position[rid] = position.get(rid, 0) + len(tokens)
    process.stdin.close()
    assert process.wait(timeout=60) == 0
    expected, low = truth["B"]
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    harness.assert_rows_close(got, expected, torch_dtype, f"virulix trace_run {dtype}", low if dtype == "bfloat16" else None)


def test_command_line_generates_with_written_and_with_random_weights(folders, tmp_path):
    """``python -m qwen_inference_lab_b200`` on a Virulix folder: greedy tokens as the plain implementation's; and
    ``--random-weights`` on a folder that holds only config.json (the sizes that only tensors give take their defaults)."""
    folder, weights, _ = folders["A"]
    prompt = cases.random_tokens(cases.CASE_B, 9, 77)          # ids that both vocabularies hold
    run = lambda model, *extra: subprocess.run(
        [sys.executable, "-m", "qwen_inference_lab_b200", "--model", str(model), "--token-ids", json.dumps(prompt),
         "--dtype", "float32", "--max-new-tokens", "4", "--pages", "16", "--page-size", "4", "--chunk-size", "5",
         "--ignore-eos", *extra], capture_output=True, text=True, cwd=str(ROOT))
    done = run(folder)
    assert done.returncode == 0, done.stderr
    tokens = json.loads(done.stdout)["token_ids"]
    sequence = list(prompt)
    for token in tokens:
        assert token == int(plain.forward(sequence, weights, cases.CASE_A)[-1].argmax())
        sequence.append(token)
    bare = tmp_path / "bare"
    bare.mkdir()
    (bare / "config.json").write_text(json.dumps(cases.CASE_B))
    done = run(bare, "--random-weights", "3")
    assert done.returncode == 0, done.stderr
    assert len(json.loads(done.stdout)["token_ids"]) == 4 and (bare / "model.safetensors").is_file()


def test_a_checkpoint_may_leave_out_the_second_norm_of_a_layer_without_feed_forward(folders, tmp_path):
    from qwen_inference_lab_b200.weights import SafetensorsFile, write_safetensors
    folder, weights, requests = folders["A"]
    with SafetensorsFile(folder / "model.safetensors") as f:
        tensors = {name: f.tensor(name).clone() for name in f.keys() if name != "l2.norm2"}
    (tmp_path / "config.json").write_text((folder / "config.json").read_text())
    write_safetensors(tmp_path / "model.safetensors", tensors)
    rows_of = {}
    for source in (folder, tmp_path):
        _, cache, runner = harness.build_engine_parts(source, torch.float32, num_pages=40, page_size=4)
        rows_of[source] = harness.run_schedule(runner, cache, harness.whole_schedule({"r1": requests["r1"], "r2": requests["r2"]}))
    assert all(torch.equal(rows_of[folder][key], rows_of[tmp_path][key]) for key in rows_of[folder])
