"""Debisun on the GPU: every mechanism alone against its plain function, then whole models under four ways of
cutting the work, long decoding, slots and pages used again, generation through the engine and the replay program."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import debisun_cases as cases
from tests import harness
from tests.plain import debisun_plain as plain

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
    assert difference.pow(2).mean().sqrt() <= 0.01 * expected.pow(2).mean().sqrt() + 1e-6, \
        f"rms difference {difference.pow(2).mean().sqrt():.3e} against rows of {expected.pow(2).mean().sqrt():.3e}"
    assert difference.abs().max() <= 0.05 * expected.abs().max() + 1e-6, \
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


def rows(count, width, seed, scale=1.0):
    return (torch.randn(count, width, generator=torch.Generator().manual_seed(seed)) * scale).to(torch.bfloat16).float()


class Ctx:
    """The little of a step's context that parts without a cache read."""
    def __init__(self, dtype, token_ids=None, stream_dtype=torch.float32):
        self.dtype, self.device, self.stream_dtype = dtype, torch.device("cuda"), stream_dtype
        self.token_ids = token_ids

    def empty(self, shape, dtype=None):
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width", [80, 257, 1024])
def test_layer_norm_of_a_float32_stream(dtype, width):
    from qwen_inference_lab_b200.parts import LayerNorm
    norm = LayerNorm(width, 1e-5, name="n", suffixes=("", ".b"))
    w = fill(norm, 3, dtype)
    x = torch.randn(9, width, generator=torch.Generator().manual_seed(4)) * 3 + 1.5
    out = norm.forward(Ctx(dtype), x.cuda())
    assert out.dtype == dtype
    close(out, plain.layer_norm(x.double(), w["n"], w["n.b"], 1e-5), dtype)
    picked = norm.forward(Ctx(dtype), x.cuda(), rows=torch.tensor([7, 0, 7], dtype=torch.int32, device="cuda"))
    assert torch.equal(picked, out[[7, 0, 7]])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_plain_activations_and_the_table_slice(dtype):
    from qwen_inference_lab_b200.kernels import ops
    z = rows(7, 24, 5, 2.0)
    for kind, f in (("relu2", plain.squared_relu), ("gelu_tanh", plain.gelu_tanh), ("silu", lambda t: t * torch.sigmoid(t))):
        close(ops.activation(z.to(dtype).cuda(), kind), f(z.double()), dtype)
    table = rows(11, 60, 6)
    ids = torch.tensor([3, 10, 0, 3, 7, 7, 1], dtype=torch.int32)
    out = ops.activation(z.to(dtype).cuda(), "gelu_tanh", table=table.to(dtype).cuda(), ids=ids.cuda(), first_col=30)
    close(out, plain.gelu_tanh(z.double()) * table[ids.long(), 30:54].double(), dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_scaled_add_and_normed_add_on_a_float32_stream(dtype):
    from qwen_inference_lab_b200.kernels import ops
    stream, branch = rows(5, 72, 7, 4.0), rows(5, 72, 8)
    scale, weight = rows(1, 72, 9)[0], (1 + 0.1 * rows(1, 72, 10)[0]).to(torch.bfloat16).float()
    out = ops.scaled_add(stream.clone().cuda(), branch.to(dtype).cuda(), scale.cuda())
    torch.testing.assert_close(out.cpu(), stream + scale * branch, atol=1e-5, rtol=1e-6)
    out = ops.rms_scale_add(stream.clone().cuda(), branch.cuda(), weight.to(dtype).cuda(), 1e-6)
    torch.testing.assert_close(out.cpu(), (stream.double() + plain.rms_norm(branch.double(), weight, 1e-6)).float(), atol=1e-5, rtol=1e-6)


def attention_part(dtype, heads=6, kv_heads=2, dim=24, vdim=40, hidden=64, taps=4, softcap=15.0, table=(16, 100), chunk=48,
                   scale=0.21, seed=1):
    from qwen_inference_lab_b200.parts import GroupedQueryAttention
    part = GroupedQueryAttention(hidden, heads, kv_heads, dim, names=dict(q="m.q", k="m.k", v="m.v", o="m.o", distance_bias="m.rel"),
                                 scale=scale, v_head_dim=vdim, suffixes=("", ".b"), conv_taps=taps, softcap=softcap,
                                 distance_bias=table, chunk=chunk, sink=True)
    w = fill(part, seed, dtype, scales=dict(rel=1.0, conv=0.6))
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, softcap=softcap, bias_max=table[1], mask=dict(size=chunk))
    return part, w, m


SHAPES = [dict(), dict(heads=3, kv_heads=3, dim=16, vdim=16, taps=2, chunk=5, table=(8, 64)),
          dict(heads=4, kv_heads=1, dim=40, vdim=8, taps=1, chunk=33, softcap=6.0, table=(10, 30)),
          dict(heads=2, kv_heads=1, dim=64, vdim=64, taps=7, chunk=96, table=(28, 310), scale=0.125)]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("shape", SHAPES, ids=["a", "b", "c", "d"])
def test_attention_mixer_whole_cut_and_side_by_side(dtype, shape):
    """The mixer over whole sequences, over portions down to one and two tokens, and with two requests in every
    step, against the plain mixer (the convolution reaches back over the cuts, the chunks' edges fall inside portions)."""
    part, w, m = attention_part(dtype, **shape)
    inputs = {"a": rows(75, 64, 11), "b": rows(41, 64, 12)}
    expected = {rid: plain.attention_mixer(x.double(), w, "m.", m, low_of(dtype)) for rid, x in inputs.items()}
    body = lambda ctx, x, view: part.forward(ctx, x, view)
    for cuts in ({"a": [75], "b": [41]}, {"a": [3, 1, 1, 2, 30, 1, 5, 2, 30], "b": [1] * 9 + [2] * 6 + [20]},
                 {"a": [1] * 75, "b": [17, 24]}):
        got = harness.run_part(part, 64, dtype, body, inputs, cuts, page_size=4, num_pages=40)
        for rid in inputs:
            close(got[rid], expected[rid], dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("taps", [1, 2, 3, 6])
def test_short_convolution_with_state_under_every_cut(dtype, taps):
    """The kernel alone: queries, and keys and values read back from the pages, for a sequence cut in many ways
    beside a neighbour; in float32 every cut gives the same bits."""
    from qwen_inference_lab_b200.kernels import ops
    heads, kv_heads, d, e, page = 3, 1, 8, 24, 4
    channels = heads * d + kv_heads * (d + e)
    T = 23
    u = {"a": rows(T, channels, 20 + taps), "b": rows(9, channels, 30)}
    weight = rows(channels, taps, 21)
    expected = {rid: plain.short_convolution(x.double(), weight, low_of(dtype)) for rid, x in u.items()}
    results = []
    for cuts in ({"a": [T], "b": [9]}, {"a": [1] * T, "b": [1] * 9}, {"a": [2, 1, 3, 1, 1, 7, 2, 6], "b": [4, 1, 4]}):
        state = torch.full((2, max(taps - 1, 0), channels), float("nan"), device="cuda")
        state[:] = 0 if taps > 1 else state
        pages = torch.full((16, kv_heads * page * (d + e)), float("nan"), dtype=dtype, device="cuda")
        table = torch.tensor([[5, 2, 9, 0, 7, 11], [3, 8, 1, -1, -1, -1]], dtype=torch.int32, device="cuda")
        done = {"a": 0, "b": 0}
        queues = {rid: list(c) for rid, c in cuts.items()}
        q_all = {rid: [] for rid in u}
        while any(queues.values()):
            batch = [(rid, queues[rid].pop(0)) for rid in ("b", "a") if queues[rid]]
            x = torch.cat([u[rid][done[rid]:done[rid] + n] for rid, n in batch]).to(dtype).cuda()
            positions = torch.tensor([done[rid] + i for rid, n in batch for i in range(n)], dtype=torch.int32, device="cuda")
            token_row = torch.tensor([0 if rid == "a" else 1 for rid, n in batch for _ in range(n)], dtype=torch.int32, device="cuda")
            seg_len = torch.tensor([n for _, n in batch], dtype=torch.int32, device="cuda")
            seg_start = torch.tensor(np.cumsum([0] + [n for _, n in batch])[:-1], dtype=torch.int32, device="cuda")
            seg_row = torch.tensor([0 if rid == "a" else 1 for rid, _ in batch], dtype=torch.int32, device="cuda")
            q = torch.empty((x.shape[0], heads * d), dtype=dtype, device="cuda")
            ops.short_conv_store(x, weight.t().contiguous().to(dtype).cuda(), state, q, pages, positions, token_row, table, seg_row, seg_start,
                                 seg_len, len(batch), heads, kv_heads, d, e, page)
            at = 0
            for rid, n in batch:
                q_all[rid].append(q[at:at + n].float().cpu())
                at += n
                done[rid] += n
        for rid, row in (("a", 0), ("b", 1)):
            n = u[rid].shape[0]
            close(torch.cat(q_all[rid]), expected[rid][:, :heads * d], dtype)
            flat = pages[table[row, :(n + page - 1) // page].long()].float().cpu()
            keys = flat[:, :kv_heads * page * d].reshape(-1, d)[:n]
            values = flat[:, kv_heads * page * d:].reshape(-1, e)[:n]
            close(keys, expected[rid][:, heads * d:heads * d + d], dtype)
            close(values, expected[rid][:, heads * d + d:], dtype)
        results.append(torch.cat(q_all["a"]))
    if dtype == torch.float32:
        assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])


def _scores_case(dtype, n_tokens, first_position, far, chunk, heads=2, kv_heads=1, d=32, e=16, page=8):
    """Queries at consecutive positions whose first channel is large, all keys zero but the one at ``far``."""
    T = first_position + n_tokens
    q = torch.zeros(n_tokens, heads, d); q[:, :, 0] = 30.0
    k = torch.zeros(T, kv_heads, d); k[far, :, 0] = 30.0
    v = rows(T, kv_heads * e, 40).view(T, kv_heads, e)
    return q, k, v, T


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("single", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("chunk,query,far", [(64, 127, 64), (64, 128, 127), (64, 128, 64), (192, 383, 192), (192, 384, 383),
                                             (7, 13, 7), (7, 14, 13), (128, 127, 0), (128, 128, 0), (33, 65, 33), (33, 66, 65)])
def test_a_key_just_inside_and_just_outside_the_chunk(dtype, single, chunk, query, far):
    """One key stands out (its score sits at the cap, every other at zero).  From inside its chunk the query's
    output is that key's value; from the first position of the next chunk the key is not seen at all.  The
    query comes as the last token of a portion and as a single token; pages are shuffled and of 8."""
    from qwen_inference_lab_b200.kernels import ops
    heads, kv_heads, d, e, page, cap = 2, 1, 32, 16, 8, 18.0
    n_tokens = 1 if single else 5
    first = query - n_tokens + 1
    q, k, v, T = _scores_case(dtype, n_tokens, first, far, chunk)
    n_pages = (T + page - 1) // page
    order = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(chunk))[:n_pages]
    pages = torch.full((n_pages + 3, kv_heads * page * (d + e)), float("nan"), dtype=dtype)
    for p in range(n_pages):
        span = slice(p * page, min(T, (p + 1) * page))
        kk = torch.zeros(page, d); kk[:span.stop - span.start] = k[span, 0]
        vv = torch.zeros(page, e); vv[:span.stop - span.start] = v[span, 0]
        pages[order[p]] = torch.cat([kk.flatten(), vv.flatten()]).to(dtype)
    table = torch.full((2, n_pages + 2), -1, dtype=torch.int32); table[1, :n_pages] = order.int()
    bias = torch.zeros(heads, 4)
    out = torch.empty((n_tokens, heads * e), dtype=dtype, device="cuda")
    ops.attention_generic(q.view(n_tokens, -1).to(dtype).cuda(), pages.cuda(), out,
                          torch.arange(first, query + 1, dtype=torch.int32, device="cuda"),
                          torch.ones(n_tokens, dtype=torch.int32, device="cuda"), table.cuda(), heads, kv_heads, d, page, 0, 1.0,
                          v_dim=e, softcap=cap, distance_bias=bias.cuda(), chunk=chunk, sink=True)
    m = dict(scale=1.0, softcap=cap, bias_max=30, mask=dict(size=chunk))
    full_q = torch.zeros(T, heads, d); full_q[first:] = q
    expected = plain.chunk_attention(full_q.double(), k.double(), v.double(), m, torch.zeros(8, heads, dtype=torch.float64))[query]
    close(out[-1].view(heads, e), expected, dtype)
    inside = far // chunk == query // chunk
    got = out[-1].view(heads, e).float().cpu()
    if inside:
        close(got, v[far].expand(heads, e), dtype)
    else:
        assert (got - v[far]).abs().max() > 0.05


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_the_distance_table_and_the_sink_alone(dtype):
    """Zero queries: the scores are the table's entries alone, the weights exp(b) / (1 + sum exp(b)); a table with
    one large entry picks the key at that distance; distances beyond the table read its last entry."""
    from qwen_inference_lab_b200.kernels import ops
    heads, d, e, page, T = 3, 16, 16, 4, 40
    v = rows(T, e, 50)
    pages = torch.zeros((10, page * (d + e)), dtype=dtype)
    for p in range(10):
        pages[p, page * d:] = v[p * page:(p + 1) * page].flatten().to(dtype)
    table = torch.arange(10, dtype=torch.int32).view(1, 10)
    bias = rows(heads, 6, 51)
    bias[1, 3] = 25.0                       # head 1: the key three positions back
    bias[2, 5] = 25.0                       # head 2: the last entry: every key five or more positions back
    out = torch.empty((1, heads * e), dtype=dtype, device="cuda")
    ops.attention_generic(torch.zeros((1, heads * d), dtype=dtype, device="cuda"), pages.cuda(), out,
                          torch.tensor([T - 1], dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda"),
                          table.cuda(), heads, 1, d, page, 0, 0.5, v_dim=e, distance_bias=bias.cuda(), sink=True)
    distance = torch.arange(T - 1, -1, -1).clamp(max=5)
    for h in range(heads):
        weights = plain.sink_softmax(bias[h, distance].double())
        close(out[0].view(heads, e)[h], weights @ v.double(), dtype)
    close(out[0].view(heads, e)[1], v[T - 4], dtype)
    close(out[0].view(heads, e)[2], v[:T - 5].double().mean(0), dtype)
    assert float(plain.sink_softmax(bias[0, distance].double()).sum()) < 1.0


def paged_pool(keys, values, page, seed):
    """keys, values: lists of [T, G, d] per request -> (pages [P, 2, G, page, d] bfloat16 with NaN where nothing was
    written, block table int32 [requests, width]); page ids are shuffled."""
    G, d = keys[0].shape[1:]
    counts = [(k.shape[0] + page - 1) // page for k in keys]
    total = sum(counts) + 3
    order = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    pages = torch.full((total, 2, G, page, d), float("nan"), dtype=torch.bfloat16)
    table = torch.full((len(keys), max(counts) + 1), -1, dtype=torch.int32)
    for r, (k, v) in enumerate(zip(keys, values)):
        for i in range(counts[r]):
            pid = order.pop()
            table[r, i] = pid
            n = min(page, k.shape[0] - i * page)
            pages[pid, 0, :, :n] = k[i * page:i * page + n].transpose(0, 1).to(torch.bfloat16)
            pages[pid, 1, :, :n] = v[i * page:i * page + n].transpose(0, 1).to(torch.bfloat16)
    return pages, table


def run_tensor_core_attention(q_rows, positions, request, pages, table, heads, kv_heads, d, page, scale, options, span_len=None,
                              tickets=False):
    """Consecutive positions of one request through the tiled kernel (``span_len`` None) or, every row a single
    token of its own, through the span kernel (its merge kernel, or the ticket form)."""
    from qwen_inference_lab_b200.kernels import attention_mma
    n = q_rows.shape[0]
    as_int = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
    out = torch.full((n, heads * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    q = q_rows.reshape(n, heads * d).to(torch.bfloat16).cuda()
    if span_len is None:
        info = [v for first in range(0, n, 64) for v in (first, positions[first], min(64, n - first), request)]
        attention_mma.prefill(q, pages.cuda(), out, as_int(info), len(info) // 4, table.cuda(), heads, kv_heads, d, page, 0,
                              scale, None, options)
        return out
    longest = max(positions) + 1
    n_spans = (longest + span_len - 1) // span_len
    info = [v for i in range(n) for v in (i, positions[i], request, longest)]
    part_o = torch.full((n * heads * n_spans * d,), float("nan"), device="cuda")
    part_ml = torch.full((n * heads * n_spans * 2,), float("nan"), device="cuda")
    counters = torch.zeros(n * heads, dtype=torch.int32, device="cuda") if tickets else None
    attention_mma.decode(q, pages.cuda(), out, as_int(info), n, part_o, part_ml, n_spans, span_len, table.cuda(), heads,
                         kv_heads, d, page, 0, scale, counters, None, options)
    return out


@pytest.mark.parametrize("heads,kv_heads,d,chunk,cap,rows_,farthest,page", [
    (4, 1, 96, 176, 25.0, 28, 310, 16), (6, 2, 32, 48, 15.0, 16, 100, 4), (2, 1, 80, 128, 50.0, 32, 500, 16),
    (3, 3, 16, 7, 8.0, 10, 30, 8), (8, 2, 64, 33, 10.0, 10, 40, 16), (20, 1, 48, 150, 0.0, 8, 64, 8)])
def test_tensor_core_attention_with_score_options(heads, kv_heads, d, chunk, cap, rows_, farthest, page):
    """The tiled kernel and the span kernel (short and long spans, merged by a second kernel and by tickets: the same
    bits) with cap, distance table, chunks and sink, on shuffled pages beside another request's, against the plain
    attention; the prompt's tiles and the single tokens straddle chunk edges."""
    from qwen_inference_lab_b200.kernels import attention_mma
    from qwen_inference_lab_b200.parts.attention import distance_rows
    T = 331
    generator = torch.Generator().manual_seed(d + chunk)
    q = (torch.randn(T, heads, d, generator=generator) * 1.5).to(torch.bfloat16).float()
    k = (torch.randn(T, kv_heads, d, generator=generator) * 1.5).to(torch.bfloat16).float()
    v = torch.randn(T, kv_heads, d, generator=generator).to(torch.bfloat16).float()
    other = torch.randn(70, kv_heads, d, generator=generator)
    pages, table = paged_pool([other, k], [other, v], page, seed=chunk)
    learned = torch.randn(rows_, heads, generator=generator).to(torch.bfloat16).float()
    scale = d ** -0.5
    m = dict(scale=scale, softcap=cap, bias_max=farthest, mask=dict(size=chunk))
    expected = plain.chunk_attention(q.double(), k.double(), v.double(), m, learned.double()).reshape(T, heads * d)
    by_distance = learned[torch.tensor(distance_rows(rows_, farthest, farthest + 1))].t().contiguous().cuda()
    options = attention_mma.ScoreOptions(cap, by_distance, chunk, True)
    out = run_tensor_core_attention(q, list(range(T)), 1, pages, table, heads, kv_heads, d, page, scale, options)
    close(out, expected, torch.bfloat16)
    late = run_tensor_core_attention(q[150:], list(range(150, T)), 1, pages, table, heads, kv_heads, d, page, scale, options)
    close(late, expected[150:], torch.bfloat16)
    singles = sorted({0, 1, chunk - 1, chunk, chunk + 1, 2 * chunk - 1, 2 * chunk, 63, 64, 65, 127, 128, 255, 256, 300, T - 1} & set(range(T)))
    for span_len in (64, 128, 2048):
        merged = run_tensor_core_attention(q[singles], singles, 1, pages, table, heads, kv_heads, d, page, scale, options, span_len)
        close(merged, expected[singles], torch.bfloat16)
        by_tickets = run_tensor_core_attention(q[singles], singles, 1, pages, table, heads, kv_heads, d, page, scale, options,
                                               span_len, tickets=True)
        assert torch.equal(merged, by_tickets)


@pytest.mark.parametrize("single", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("chunk,query,far", [(64, 127, 64), (64, 128, 127), (64, 128, 64), (192, 383, 192), (192, 384, 383),
                                             (7, 13, 7), (7, 14, 13), (128, 127, 0), (128, 128, 0), (33, 65, 33), (33, 66, 65)])
def test_a_key_at_the_chunks_edge_through_the_tensor_core_kernels(single, chunk, query, far):
    """The standing-out key of the test above through the tiled kernel (the query is the last row of a five-token
    portion) and the span kernel: seen from inside its chunk, not from the first position of the next."""
    from qwen_inference_lab_b200.kernels import attention_mma
    heads, kv_heads, d, page, cap = 2, 1, 32, 8, 18.0
    n_tokens = 1 if single else 5
    first = query - n_tokens + 1
    q, k, _, T = _scores_case(torch.bfloat16, n_tokens, first, far, chunk)
    v = rows(T, kv_heads * d, 41).view(T, kv_heads, d)
    pages, table = paged_pool([k], [v], page, seed=query)
    options = attention_mma.ScoreOptions(cap, torch.zeros(heads, 4, device="cuda"), chunk, True)
    positions = list(range(first, query + 1))
    out = run_tensor_core_attention(q, positions, 0, pages, table, heads, kv_heads, d, page, 1.0, options,
                                    span_len=64 if single else None, tickets=single)
    got = out[-1].view(heads, d).float().cpu()
    if far // chunk == query // chunk:
        close(got, v[far].expand(heads, d), torch.bfloat16)
    else:
        assert (got - v[far]).abs().max() > 0.05
        own = v[query // chunk * chunk:query + 1, 0].double()
        close(got, (own.sum(0) / (own.shape[0] + 1)).expand(heads, d), torch.bfloat16)      # equal weights, and the sink's


def experts_part(dtype, experts, identity, top, shared, hidden=40, ff=24, scale=1.7, seed=3):
    from qwen_inference_lab_b200.parts import PlainMLP, RoutedExperts
    shared_part = PlainMLP(hidden, shared, names=dict(up="f.shared.up", down="f.shared.down"), suffixes=("", ".b")) if shared else None
    part = RoutedExperts(hidden, ff, experts, top, names=dict(router="f.router", correction="f.correction",
                                                              expert=lambda i, which: f"f.e{i}.{which}"),
                         activation="relu2", gated=False, routing="softmax_all", weight_scale=scale, identity=identity,
                         shared=shared_part, shared_gate="f.shared.sg" if shared else None)
    w = fill(part, seed, dtype, scales=dict(router=0.5, correction=0.05, sg=0.3))
    mlp = dict(kind="moe", router=dict(experts=experts, identity=identity, top=top, scale=scale), expert=dict(ff=ff))
    if shared:
        mlp["shared"] = dict(ff=shared)
    return part, w, mlp


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("experts,identity,top,shared", [(5, 2, 3, 40), (3, 0, 1, 0), (8, 4, 4, 16), (4, 1, 5, 0), (70, 3, 6, 8), (1, 1, 1, 8)])
def test_routed_experts_alone_and_in_a_batch(dtype, experts, identity, top, shared):
    """Choice, weights, identity outputs, the gated shared expert and the output scale, against the plain
    feed-forward; a token alone gives the same result as among ninety others, which the many-token form of the router's kernel
    takes (float32: the same bits)."""
    from qwen_inference_lab_b200.kernels import ops
    part, w, mlp = experts_part(dtype, experts, identity, top, shared)
    x = rows(91, 40, 13)
    chosen, weights = ops.moe_route(x.to(dtype).cuda(), part.router.data, None, top, softmax_all=True,
                                    correction=part.correction.data, weight_scale=mlp["router"]["scale"])
    want_chosen, want_weights = plain.route(x.double(), w, "f.", mlp["router"])
    assert torch.equal(chosen.cpu().long().sort(1).values, want_chosen.sort(1).values)
    torch.testing.assert_close(weights.cpu().double().sort(1).values, want_weights.sort(1).values, atol=1e-5, rtol=1e-5)
    assert identity == 0 or bool((want_chosen >= experts).any()), "no token chose an identity output: use other weights"
    scale = (0.7 + 0.2 * rows(1, 40, 14)[0]).to(torch.bfloat16).float()
    stream = rows(91, 40, 15, 3.0)
    expected = stream.double() + plain.moe_ff(x.double(), w, "f.", mlp, low_of(dtype)) * scale.double()
    ctx = Ctx(dtype)
    together = part.forward(ctx, x.to(dtype).cuda(), residual=stream.clone().cuda(), out_scale=scale.cuda())
    close(together, expected, dtype)
    alone = part.forward(ctx, x[17:18].to(dtype).cuda(), residual=stream[17:18].clone().cuda(), out_scale=scale.cuda())
    close(alone, expected[17:18], dtype)
    if dtype == torch.float32:
        assert torch.equal(alone[0], together[17])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("n", [1, 9, 300])
def test_plain_feed_forward_with_an_output_scale(dtype, n):
    from qwen_inference_lab_b200.parts import PlainMLP
    part = PlainMLP(48, 72, names=dict(up="f.up", down="f.down"), suffixes=("", ".b"))
    w = fill(part, 5, dtype)
    x, stream = rows(n, 48, 16), rows(n, 48, 17, 3.0)
    scale = (0.7 + 0.2 * rows(1, 48, 18)[0]).to(torch.bfloat16).float()
    out = part.forward(Ctx(dtype), x.to(dtype).cuda(), residual=stream.clone().cuda(), out_scale=scale.cuda())
    assert out.dtype == torch.float32
    close(out, stream.double() + plain.dense_ff(x.double(), w, "f.", low_of(dtype)) * scale.double(), dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("dim,index", [(8, 2), (5, 0), (16, 3)])
def test_token_side_input(dtype, dim, index):
    from qwen_inference_lab_b200.parts import Param, TokenSideInput
    table = Param((31, 4 * dim))
    part = TokenSideInput(56, dim, index, 1e-6, table=table, suffixes=("", ".b"), norm_suffix="",
                          names=dict(table="side.embed", gate="s.gate", proj="s.proj", norm="s.norm"))
    w = fill(part, 6, dtype, scales=dict(embed=1.0, norm=0.2))
    for n in (1, 12, 40):
        tokens = torch.randint(0, 31, (n,), generator=torch.Generator().manual_seed(n))
        x = rows(n, 56, 19 + n, 2.0)
        out = part.forward(Ctx(dtype, tokens.int().cuda()), x.clone().cuda())
        w_plain = {"side.embed": w["side.embed"], "p.side.gate": w["s.gate"], "p.side.proj": w["s.proj"], "p.side.norm": w["s.norm"]}
        expected = x.double() + plain.token_side(x.double(), tokens, w_plain, "p.", index, dim, 1e-6, low_of(dtype))
        close(out, expected, dtype)


# ------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    result = {}
    for name, case in cases.CASES.items():
        folder = tmp_path_factory.mktemp(f"debisun{name}")
        weights = cases.write_folder(case["config"], case["seed"], folder)
        requests = {f"r{i}": cases.random_tokens(case["config"], n, 60 + i) for i, n in enumerate(case["lengths"])}
        result[name] = (folder, weights, requests)
    return result


@pytest.fixture(scope="module")
def truth(folders):
    """The plain rows of every case, in float64 and with bfloat16 roundings, and the close calls: computed once."""
    return {name: (cases.plain_rows(requests, weights, cases.CASES[name]["config"]),
                   cases.plain_rows(requests, weights, cases.CASES[name]["config"], torch.bfloat16),
                   cases.close_calls(requests, weights, cases.CASES[name]["config"]))
            for name, (folder, weights, requests) in folders.items()}


def judge(actual, expected, low, skip, dtype, what):
    """float32: every row, element by element, against the float64 rows (5e-5: what float32 sums of this depth cost).

    bfloat16: the yardstick is what bfloat16 costs the plain implementation itself (``low``), on the rows whose
    choice of experts is no close call.  The mean row error may be 1.5 times the yardstick's; no row's largest
    error may pass twice the yardstick's largest (the largest of a few hundred rows is itself a draw); a row's own error may be 1.5 times the yardstick's in that row
    or 2.25 times its mean, which one row in twenty-five may pass, by a factor of two at most (a branch normed by its own
    root mean square makes single rows sensitive, and the engine does not round where the plain code does); and
    wherever the float64 row's best logit leads by four times the yardstick's largest error in that row, the
    engine's best token is the same."""
    assert set(actual) == set(expected), f"{what}: different (request, position) sets"
    if dtype == torch.float32:
        bad = [k for k in sorted(expected) if not torch.allclose(actual[k], expected[k], atol=5e-5, rtol=1e-5)]
        assert not bad, f"{what}: {len(bad)} rows differ, first {bad[0]} by {(actual[bad[0]] - expected[bad[0]]).abs().max():.3e}"
        return
    assert len(skip) < len(expected) // 4, f"{what}: {len(skip)} of {len(expected)} rows are close calls; use other weights"
    keys = [k for k in sorted(expected) if k not in skip]
    assert all(torch.isfinite(actual[k]).all() for k in sorted(expected)), f"{what}: non-finite logits"
    rms = lambda rows, k: (rows[k] - expected[k]).pow(2).mean().sqrt().item()
    peak = lambda rows, k: (rows[k] - expected[k]).abs().max().item()
    mean_bar = 1.5 * sum(rms(low, k) for k in keys) / len(keys)
    peak_bar = 2.0 * max(peak(low, k) for k in keys)
    mean_rms = sum(rms(actual, k) for k in keys) / len(keys)
    assert mean_rms <= mean_bar, f"{what}: mean row error {mean_rms:.3e} against a bar of {mean_bar:.3e}"
    worst = max(keys, key=lambda k: peak(actual, k))
    assert peak(actual, worst) <= peak_bar, f"{what}: row {worst} is off by {peak(actual, worst):.3e}, the bar is {peak_bar:.3e}"
    row_bar = lambda k: max(1.5 * mean_bar, 1.5 * rms(low, k))
    over = [k for k in keys if rms(actual, k) > row_bar(k)]
    assert len(over) <= max(1, len(keys) // 25) and all(rms(actual, k) <= 2 * row_bar(k) for k in over), \
        f"{what}: {len(over)} of {len(keys)} rows are further off than their bar, first {over[0]}: " \
        f"{rms(actual, over[0]):.3e} against {row_bar(over[0]):.3e}"
    judged = 0
    for k in keys:
        best = expected[k].topk(2).values
        if (best[0] - best[1]).item() > 4 * peak(low, k):
            judged += 1
            assert actual[k].argmax().item() == expected[k].argmax().item(), f"{what}: another best token at {k}"
    assert judged > len(keys) // 4, f"{what}: only {judged} of {len(keys)} rows have a clear best token; use other weights"


SCHEDULES = {"whole": harness.whole_schedule, "tail_decode": harness.tail_decode_schedule,
             "chunks": harness.chunk_schedule, "mixed": harness.mixed_schedule}


def peak_live_pages(schedule, config, page_size):
    """The most pages the schedule holds at once when chunks that are over give their pages back: found by
    walking the schedule through a cache manager on the CPU."""
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.parts import KVCacheSpec
    specs = [KVCacheSpec(1, 1, chunk=layer["mixer"]["mask"]["size"]) for layer in config["layers"]]
    cache = CacheManager(specs, num_pages=4096, page_size=page_size, max_requests=8, max_context=1 << 20,
                         dtype=torch.float32, device="cpu")
    peak = 0
    for entries, ended in schedule:
        for rid, tokens, _ in entries:
            if rid not in cache.rows:
                assert cache.admit(rid)
            cache.ensure(rid, cache.written(rid) + len(tokens))
        peak = max(peak, max(g.capacity - len(g.free) for g in cache.kv_groups))
        for rid, tokens, _ in entries:
            cache.advance(rid, cache.written(rid) + len(tokens))
        for rid in ended:
            cache.release(rid)
    return peak


def replay(folders, case, schedule_name, dtype):
    folder, weights, requests = folders[case]
    page_size = cases.CASES[case]["page_size"]
    schedule = SCHEDULES[schedule_name](requests)
    num_pages = peak_live_pages(schedule, cases.CASES[case]["config"], page_size) + 1
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
    expected, low, skip = truth[case]
    judge(actual, expected, low, skip, dtype, f"debisun {case} {schedule} {dtype}")


@pytest.mark.parametrize("case", list(cases.CASES))
def test_float32_rows_are_the_same_bits_under_every_schedule(folders, case):
    runs = {name: replay(folders, case, name, torch.float32) for name in SCHEDULES}
    for name, got in runs.items():
        different = [key for key in sorted(got) if not torch.equal(got[key], runs["whole"][key])]
        assert not different, \
            f"debisun {case}: {len(different)} rows of schedule {name} differ from the whole run, first {different[0]}"


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_and_the_first_tokens(folders, dtype):
    """Three tokens as a prompt, then 300 single tokens (recorded graphs) across many chunk edges, every position
    judged; the pool holds far fewer pages than the positions, because chunks that are over give theirs back."""
    folder, weights, _ = folders["B"]
    config = cases.CASE_B
    tokens = cases.random_tokens(config, 303, 99)
    schedule = [([("r", tokens[:3], [0, 1, 2])], [])]
    schedule += [([("r", [tokens[i]], [0])], ["r"] if i == 302 else []) for i in range(3, 303)]
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=10, page_size=16)
    actual = harness.run_schedule(runner, cache, schedule)
    assert runner._graphs, "single-token steps should have been recorded"
    expected = cases.plain_rows({"r": tokens}, weights, config)
    low = cases.plain_rows({"r": tokens}, weights, config, torch.bfloat16) if dtype == torch.bfloat16 else None
    judge(actual, expected, low, cases.close_calls({"r": tokens}, weights, config), dtype, f"debisun long decoding {dtype}")


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
            logits = plain.forward(config, weights, sequence, torch.float32)[-1]
            best = int(logits.argmax())
            if token != best:
                assert dtype == torch.bfloat16, f"token {token} instead of {best} after {len(sequence)} tokens"
                noise = (plain.forward(config, weights, sequence, torch.float32, torch.bfloat16)[-1] - logits).abs().max().item()
                assert float(logits[best] - logits[token]) < 4 * noise
            sequence.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_replays_a_mixed_schedule(folders, truth, tmp_path, dtype):
    folder, weights, requests = folders["B"]
    schedule = harness.mixed_schedule(requests)
    peak = harness.peak_pages(schedule, 64, round_to=64) * 64
    process = subprocess.Popen([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                                "--out", str(tmp_path / "out"), "--max-tokens", str(peak)],
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
    expected, low, skip = truth["B"]
    judge(got, expected, low, skip, torch.float32 if dtype == "float32" else torch.bfloat16, f"debisun trace_run {dtype}")


def test_command_line_generates_with_written_and_with_random_weights(folders, tmp_path):
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
        assert token == int(plain.forward(cases.CASE_A, weights, sequence, torch.float32)[-1].argmax())
        sequence.append(token)
    bare = tmp_path / "bare"
    bare.mkdir()
    (bare / "config.json").write_text(json.dumps(cases.CASE_B))
    done = run(bare, "--random-weights", "3")
    assert done.returncode == 0, done.stderr
    assert len(json.loads(done.stdout)["token_ids"]) == 4 and (bare / "model.safetensors").is_file()


def test_a_checkpoint_may_leave_out_the_second_norm_and_scale_of_a_layer_without_feed_forward(folders, tmp_path):
    from qwen_inference_lab_b200.weights import SafetensorsFile, write_safetensors
    folder, weights, requests = folders["A"]
    with SafetensorsFile(folder / "model.safetensors") as f:
        tensors = {name: f.tensor(name).clone() for name in f.keys() if name not in ("l2.norm2", "l2.norm2.b", "l2.ls2")}
    (tmp_path / "config.json").write_text((folder / "config.json").read_text())
    write_safetensors(tmp_path / "model.safetensors", tensors)
    rows_of = {}
    for source in (folder, tmp_path):
        _, cache, runner = harness.build_engine_parts(source, torch.float32, num_pages=40, page_size=4)
        rows_of[source] = harness.run_schedule(runner, cache, harness.whole_schedule({"r1": requests["r1"], "r2": requests["r2"]}))
    assert all(torch.equal(rows_of[folder][key], rows_of[tmp_path][key]) for key in rows_of[folder])
