"""Virulix without a GPU: configuration, registry, tensor names, and the plain implementation against itself."""
import json

import pytest
import torch

from qwen_inference_lab_b200.config import ConfigError, VirulixConfig, registry
from qwen_inference_lab_b200.loading import tensor_shapes
from tests import virulix_cases as cases
from tests.plain import virulix_plain as plain


def test_config_json_names_the_architecture_in_a_single_string(tmp_path):
    cases.write_folder(cases.CASE_A, 1, tmp_path)
    entry, config = registry.read_model_config(tmp_path)
    assert entry.name == "Virulix" and isinstance(config, VirulixConfig) and entry.shape_aware
    assert config.vocab_size == 211 and config.width == 80 and config.eps == 1e-5
    assert VirulixConfig.from_dict(config.to_dict()) == config
    assert registry.lookup(config.to_dict()) is entry


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "divide"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "shape of keys"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "experts"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "neither"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c.update(vocab=0), "vocab"),
    (lambda c: c["layers"][3]["mixer"].pop("tau"), "lacks"),
])
def test_configurations_that_are_refused(change, message):
    data = json.loads(json.dumps(cases.CASE_A))
    change(data)
    with pytest.raises(ConfigError, match=message):
        VirulixConfig.from_dict(data)


def test_tensor_names_sizes_and_what_a_layer_leaves_out(tmp_path):
    weights = cases.write_folder(cases.CASE_A, 2, tmp_path)
    shapes = tensor_shapes(tmp_path)
    entry, config = registry.read_model_config(tmp_path)
    model = entry.build(config, tensor_shapes=shapes)
    expected = {name: param.shape for name, param in model.all_named_params().items()}
    assert expected == {name: tuple(shape) for name, shape in shapes.items()}
    assert "l2.mix.k" not in weights and "l2.mix.q.b" in weights and "l2.mix.o.b" not in weights
    assert "l2.norm2" in weights and model.all_named_params()["l2.norm2"].optional     # no feed-forward: may be left out
    assert weights["l3.mix.a1"].shape == (5, 80) and weights["l0.mix.a1"].shape == (16, 80)
    assert weights["l1.mlp.gate.b"].shape == (56,) and "l0.mlp.shared.gate.b" not in weights
    assert "l3.mlp.shared.gate" not in weights and weights["l0.mlp.e4.down"].shape == (80, 24)
    specs = model.cache_specs()
    assert specs[2] is None and specs[1].v_head_dim == 40 and specs[4].v_head_dim == 0
    assert specs[0].shape == (3, 24, 40) and specs[0].dtype == torch.float32
    assert model.order[2].reads_cache_of == 1 and model.stream_dtype == torch.float32


def test_the_decay_rank_comes_from_the_tensor(tmp_path):
    weights = cases.make_weights(cases.CASE_B, 3)
    entry = registry.lookup(cases.CASE_B)
    config = entry.config_class.from_dict(cases.CASE_B)
    model = entry.build(config, tensor_shapes={"l1.mix.a1": (11, 64)})
    assert model.all_named_params()["l1.mix.a1"].shape == (11, 64)
    assert model.all_named_params()["l1.mix.a2"].shape == (8, 11)
    assert weights["l1.mix.a1"].shape == (3, 64)


def test_plain_recurrence_carries_its_state_across_a_cut():
    torch.manual_seed(0)
    T, H, d, e = 23, 2, 5, 7
    q, k, alpha = torch.randn(T, H, d), torch.randn(T, H, d), torch.rand(T, H, d)
    v = torch.randn(T, H, e)
    whole, final = plain.gated_linear_recurrence(q, k, v, alpha)
    first, state = plain.gated_linear_recurrence(q[:9], k[:9], v[:9], alpha[:9])
    second, end = plain.gated_linear_recurrence(q[9:], k[9:], v[9:], alpha[9:], state)
    torch.testing.assert_close(torch.cat((first, second)), whole)
    torch.testing.assert_close(end, final)
    # the closed form of one output: o_t = sum_s (prod_{s < r <= t} alpha_r) . k_s . q_t  v_s
    t = 6
    expected = sum((alpha[s + 1:t + 1, 0].prod(dim=0) * k[s, 0] * q[t, 0]).sum() * v[s, 0] for s in range(t + 1))
    torch.testing.assert_close(whole[t, 0], expected)


def test_plain_attention_bias_and_temperature():
    slopes = plain.distance_slopes(4)
    assert slopes.tolist() == [2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8]
    temperature = plain.query_temperature(torch.arange(12), 0.5, 4)
    assert temperature[2] == 1.0 and temperature[3] == pytest.approx(1 + 0.5 * 0.6931471805599453)
    assert temperature[11] == pytest.approx(1 + 0.5 * 1.3862943611198906)
    # with equal keys the weights fall off with distance as exp(-slope * distance)
    q, k, v = torch.ones(5, 1, 3), torch.ones(5, 1, 3), torch.eye(5)[:, None, :]
    out = plain.biased_attention(q, k, v, 1.0)[4, 0]
    torch.testing.assert_close(out[3] / out[4], torch.exp(torch.tensor(-2.0 ** -8)))


def test_plain_router_weights_are_a_softmax_over_the_chosen_alone():
    w = {"r.router": torch.eye(4), "r.router.b": torch.tensor([0.0, 0.5, 0.0, 0.0])}
    chosen, weights = plain.route(torch.tensor([[3.0, 1.0, 2.0, -5.0]]), w, "r.", 2)
    assert chosen.tolist() == [[0, 2]]
    torch.testing.assert_close(weights, torch.softmax(torch.tensor([[3.0, 2.0]]), dim=-1))


def test_scan_planner_cuts_long_segments_into_chunks():
    import numpy as np
    from qwen_inference_lab_b200.parts import Segments
    from qwen_inference_lab_b200.parts.linear_attention import CHUNK, LONG_SEGMENT, ScanPlanner
    lens = np.array([1, LONG_SEGMENT, LONG_SEGMENT + 1, 7, 3 * CHUNK])
    first = np.concatenate(([0], np.cumsum(lens[:-1])))
    plan = ScanPlanner().plan(Segments(rows=np.array([3, 0, 2, 1, 5]), first=first, lens=lens,
                                       starts=np.array([9, 0, 40, 0, 1000]), n_tokens=int(lens.sum())))
    assert plan["short_start"].tolist() == [0, 1, 1 + LONG_SEGMENT + LONG_SEGMENT + 1]
    assert plan["short_len"].tolist() == [1, LONG_SEGMENT, 7] and plan["short_row"].tolist() == [3, 0, 1]
    assert plan["chunk_len"].tolist() == [CHUNK, CHUNK, 1, CHUNK, CHUNK, CHUNK]
    assert plan["chunk_index"].tolist() == list(range(6))
    assert plan["chunk_start"].tolist()[:3] == [129, 129 + CHUNK, 129 + 2 * CHUNK]
    assert plan["carry"].tolist() == [2, 0, 3, 5, 3, 3]
    singles = ScanPlanner().plan(Segments(rows=np.arange(4), first=np.arange(4), lens=np.ones(4, dtype=np.int64),
                                          starts=np.array([5, 6, 7, 8]), n_tokens=4))
    assert singles["chunk_start"].size == 0 and singles["carry"].size == 0 and singles["short_len"].tolist() == [1] * 4
