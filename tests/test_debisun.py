"""Debisun without a GPU: configuration and refusals, tensor names, distance rows, the plain functions against
closed forms, the cache manager's chunked groups and paired specs."""
import math

import pytest
import torch

from qwen_inference_lab_b200.cache import CacheManager
from qwen_inference_lab_b200.config import registry
from qwen_inference_lab_b200.config.model_config import ConfigError, DebisunConfig
from qwen_inference_lab_b200.parts import KVCacheSpec, StateSpec
from qwen_inference_lab_b200.parts.attention import distance_rows
from tests import debisun_cases as cases
from tests.plain import debisun_plain as plain


def test_the_registry_builds_the_model_with_the_design_names():
    entry = registry.lookup(cases.CASE_A)
    assert entry.config_class is DebisunConfig
    model = entry.build(DebisunConfig.from_dict(cases.CASE_A))
    names = set(model.all_named_params())
    for expected in ("embed", "side.embed", "l0.norm1", "l0.norm1.b", "l0.mix.q", "l0.mix.q.conv", "l0.mix.v.conv",
                     "l0.mix.rel", "l0.mix.o", "l0.ls1", "l0.ls2", "l0.mlp.e4.up", "l0.mlp.e4.down", "l0.mlp.router",
                     "l0.mlp.correction", "l0.mlp.shared.up", "l0.mlp.shared.sg", "l0.side.gate", "l0.side.proj",
                     "l0.side.norm", "l1.mlp.up", "l1.mlp.down", "final.norm", "final.norm.b", "head"):
        assert expected in names, expected
    assert "l0.mlp.e5.up" not in names and "l0.mlp.e0.gate" not in names      # identity outputs own no tensors
    assert "l3.mix.q.conv" in names and "l3.mlp.shared.up" not in names
    params = model.all_named_params()
    assert params["l0.mlp.router"].shape == (7, 80) and params["l0.mlp.correction"].shape == (7,)
    assert params["l0.mix.rel"].shape == (16, 6) and params["l0.mix.k.conv"].shape == (48, 4)
    assert params["side.embed"].shape == (211, 4 * 8) and params["l2.norm2"].optional
    # the table's rows come from the checkpoint's tensor when there is one
    model = entry.build(DebisunConfig.from_dict(cases.CASE_A), tensor_shapes={"l0.mix.rel": (12, 6)})
    assert model.all_named_params()["l0.mix.rel"].shape == (12, 6)
    specs = model.cache_specs()
    assert specs[0] == (KVCacheSpec(2, 24, 0, 40, chunk=48), StateSpec((3, 6 * 24 + 2 * 24 + 2 * 40), torch.float32))
    assert specs[3] == KVCacheSpec(2, 16, 0, 24, chunk=7)             # one tap keeps no state


@pytest.mark.parametrize("change", [
    lambda c: c.update(vocab=0), lambda c: c["norm"].update(eps=0), lambda c: c.update(layers=[]),
    lambda c: c["layers"][0].update(type="gla"), lambda c: c["layers"][0]["mixer"].update(kv_heads=4),
    lambda c: c["layers"][0]["mixer"].update(scale=-1.0), lambda c: c["layers"][0]["mixer"].update(conv=0),
    lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), lambda c: c["layers"][0]["mixer"].pop("bias_max"),
    lambda c: c["layers"][0]["mlp"]["router"].update(top=8), lambda c: c["layers"][0]["mlp"]["router"].update(identity=-1),
    lambda c: c["layers"][1]["mlp"].update(kind="gated"), lambda c: c["layers"][0]["mlp"]["shared"].pop("ff"),
    lambda c: c["token_side"].update(dim=0), lambda c: c.update(architecture="Other"),
])
def test_configurations_that_are_refused(change):
    data = DebisunConfig.from_dict(cases.CASE_A).to_dict()
    change(data)
    with pytest.raises(ConfigError):
        DebisunConfig.from_dict(data)


def test_configuration_round_trip_and_optional_keys():
    config = DebisunConfig.from_dict(cases.CASE_B)
    assert DebisunConfig.from_dict(config.to_dict()) == config and config.side_dim == 0
    assert DebisunConfig.from_dict(cases.CASE_A).side_dim == 8


def test_distance_rows_follow_the_logarithm():
    # below half the rows a distance is its own row; from `farthest` on everything is the last row
    rows = distance_rows(28, 310, 400)
    assert rows[:14] == list(range(14)) and rows[14] == 14 and rows[309] == 27 and rows[310] == 27 and rows[399] == 27
    assert all(b >= a for a, b in zip(rows, rows[1:]))
    for n in (15, 27, 28, 29, 100, 200, 309):
        assert rows[n] == min(27, 14 + math.floor(math.log(n / 14) / math.log(310 / 14) * 14))
    for table, farthest in ((8, 64), (10, 30), (24, 300), (16, 100)):
        ours = distance_rows(table, farthest, farthest + 5)
        assert ours == [plain.distance_bucket(n, table, farthest) for n in range(farthest + 5)]
    with pytest.raises(ValueError):
        distance_rows(32, 16, 4)


def test_plain_functions_against_closed_forms():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    y = plain.layer_norm(x, torch.ones(4), torch.zeros(4), 0.0)
    assert torch.allclose(y.mean(), torch.tensor(0.0, dtype=torch.float64)) and torch.allclose(y.pow(2).mean(), torch.tensor(1.0, dtype=torch.float64))
    assert torch.allclose(plain.squared_relu(torch.tensor([-2.0, 3.0])), torch.tensor([0.0, 9.0]))
    # the sink: one key of score s gets e^s / (1 + e^s)
    assert torch.allclose(plain.sink_softmax(torch.tensor([0.0], dtype=torch.float64)), torch.tensor([0.5], dtype=torch.float64))
    assert torch.allclose(plain.sink_softmax(torch.tensor([-200.0, -200.0], dtype=torch.float64)).sum(), torch.tensor(0.0, dtype=torch.float64))
    # the convolution: taps (1, 10, 100) on the sequence 1, 2, 3 reach back two positions, zeros before the start
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    assert plain.short_convolution(u, torch.tensor([[1.0, 10.0, 100.0]])).flatten().tolist() == [100.0, 210.0, 321.0]
    # routing: the correction moves the choice, not the weight
    w = {"r.router": torch.eye(3, dtype=torch.float64), "r.correction": torch.tensor([0.0, 0.0, 5.0])}
    chosen, weights = plain.route(torch.tensor([[3.0, 1.0, 0.0]], dtype=torch.float64), w, "r.", dict(top=2, scale=2.0))
    assert chosen.tolist() == [[2, 0]]
    scores = torch.softmax(torch.tensor([3.0, 1.0, 0.0], dtype=torch.float64), 0)
    assert torch.allclose(weights[0], torch.stack([scores[2], scores[0]]) / (scores[2] + scores[0]) * 2.0)


def test_chunk_attention_sees_its_own_chunk_only():
    """A key that would dominate is seen from inside its chunk and not from the chunk after it."""
    m = dict(scale=1.0, softcap=18.0, bias_max=30, mask=dict(size=5))
    table = torch.zeros(8, 1, dtype=torch.float64)
    T = 12
    q = torch.zeros(T, 1, 4, dtype=torch.float64); k = torch.zeros(T, 1, 4, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64).view(T, 1, 1) + 1.0
    k[4, 0, 0] = 100.0                       # the last position of chunk 0
    q[:, 0, 0] = 100.0
    out = plain.chunk_attention(q, k, v, m, table).flatten()
    assert abs(out[4].item() - 5.0) < 1e-6    # position 4 sees key 4 at the cap: exp(18) outweighs everything
    assert out[5].item() < 6.0 / 2 + 1e-9 and abs(out[5].item() - 6.0 / 2) < 1e-9     # position 5 sees itself and the sink only
    assert abs(out[9].item() - (6 + 7 + 8 + 9 + 10) / 6.0) < 1e-9


def test_the_cache_manager_pairs_pages_with_a_state_slot_and_gives_chunks_back():
    pages, state = KVCacheSpec(1, 4, chunk=8), StateSpec((2, 6), torch.float32)
    cache = CacheManager([(pages, state), (pages, state), KVCacheSpec(1, 4)], num_pages=12, page_size=4, max_requests=2,
                         max_context=64, dtype=torch.float32, device="cpu")
    views = cache.views()
    assert isinstance(views[0], tuple) and views[0][0].pages.shape[0] == 12 and views[0][1].slots.shape == (2, 2, 6)
    assert views[0][1].slots.data_ptr() != views[1][1].slots.data_ptr() and not isinstance(views[2], tuple)
    chunked, full = cache.kv_groups
    assert chunked.members == [0, 1] and full.members == [2]
    views[0][1].slots.fill_(7.0)
    assert cache.admit("a")
    assert float(views[0][1].slots[cache.row("a")].abs().max()) == 0.0          # zeroed at admission
    cache.ensure("a", 7); cache.advance("a", 7)
    assert [p >= 0 for p in chunked.tables["a"]] == [True, True]
    cache.ensure("a", 8); cache.advance("a", 8)          # the next position opens chunk 1: chunk 0's pages go back
    assert [p >= 0 for p in chunked.tables["a"]] == [False, False] and [p >= 0 for p in full.tables["a"]] == [True, True]
    cache.ensure("a", 21); cache.advance("a", 21)        # position 21 reads from 16 on
    assert [p >= 0 for p in chunked.tables["a"]] == [False, False, False, False, True, True]
    cache.check_invariants()
    cache.release("a")
    assert len(chunked.free) == 12 and len(full.free) == 12
    cache.check_invariants()
