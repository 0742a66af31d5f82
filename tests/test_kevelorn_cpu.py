"""Kevelorn without a GPU: the configuration's round trip and errors, the plan, the tensors the parts expect against an
independent list, what the cache is asked for, and the plain implementation's mechanisms on cases worked out by hand."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_kevelorn as plain
from kevelorn_models import CONFIGS, RANKS, make_weights, tensor_shapes


def build(name):
    from pico_engine.config.kevelorn import KevelornConfig
    from pico_engine.parts.model import DecoderModel
    cfg = CONFIGS[name]
    c = KevelornConfig.from_dict(cfg, tensor_shapes(cfg, RANKS[name]))
    return c, DecoderModel(c.plan(), torch.float32, "meta")


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_expected_tensors(name):
    from pico_engine.config.registry import config_from_dict
    c, model = build(name)
    again = type(c).from_dict(c.to_dict())
    assert again.to_dict() == c.to_dict()
    assert type(config_from_dict(CONFIGS[name])) is type(c)
    expected = {n: tuple(s.shape) for n, s in model.expected_tensors().items()}
    assert expected == {n: tuple(s) for n, s in tensor_shapes(CONFIGS[name], RANKS[name]).items()}


def test_rank_comes_from_the_stored_tensor(tmp_path):
    from conftest import write_model
    from pico_engine.config.registry import read_config
    cfg = CONFIGS["K2"]
    folder = write_model(tmp_path / "m", cfg, make_weights(cfg, 0, RANKS["K2"]))
    assert read_config(folder).layers[0].decay_rank == RANKS["K2"]


def test_schedule_of_a_loop():
    c, model = build("K1")
    sched = model.plan.schedule
    assert [e.layer for e in sched] == [0, 1, 0, 1, 0, 1, 2]
    assert [e.add_vector for e in sched] == [("loop.step", 0), None, ("loop.step", 1), None, ("loop.step", 2), None, None]
    assert [e.add_embedding for e in sched] == [False, False, True, False, True, False, False]
    assert all(e.cache_of is None for e in sched)                      # every pass keeps its own keys, values and states
    c, model = build("K2")
    assert [e.layer for e in model.plan.schedule] == [0, 1, 2] and not model.plan.stream_vectors
    c, model = build("K4")
    assert [e.layer for e in model.plan.schedule] == [0, 1, 1]


def test_cache_needs():
    c, model = build("K1")
    needs = model.cache_needs()
    left = CONFIGS["K1"]["layers"][0]["mixer"]
    assert needs[0].kv.window == 40 and needs[0].kv.n_kv_heads == 2 and needs[0].kv.head_dim == 32
    assert needs[0].state_elems == 2 * 16 * 24 and needs[1].state_elems == 3 * 24 * 16 and needs[1].kv is None
    assert needs[6].state_elems == 3 * 40 * 8
    c, model = build("K2")
    assert model.cache_needs()[1].kv.value_shape == (4, 40) and model.cache_needs()[1].kv.window == 70
    c, model = build("K3")
    assert model.cache_needs()[1].kv.window is None


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda d: d["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 4), "evenly"),
    (lambda d: d["layers"][2]["mixer"].__setitem__("decay", [0.5]), "decay"),
    (lambda d: d["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda d: d["loop"].__setitem__("stop", 7), "loop"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_errors_name_the_key(change, word):
    from pico_engine.config.kevelorn import KevelornConfig
    from pico_engine.config.specs import ConfigError
    d = copy.deepcopy(CONFIGS["K1"])
    change(d)
    with pytest.raises(ConfigError, match=word):
        KevelornConfig.from_dict(d)


# ------------------------------------------------------------------ the plain implementation on cases worked by hand

def test_rotation_by_hand():
    u = torch.zeros(3, 1, 6, dtype=torch.float64)
    u[:, 0] = torch.tensor([1.0, 0.0, 0.0, 2.0, 5.0, 7.0])
    out = plain.rotate_pairs(u, 2, 4, 100.0, 2.0)              # pairs (0,1), (2,3) turn; entries 4, 5 stay
    for t in range(3):
        p = 2 + t
        a0, a1 = p * 1.0 / 2.0, p * 100.0 ** -0.5 / 2.0
        assert torch.allclose(out[t, 0], torch.tensor([math.cos(a0), math.sin(a0), -2 * math.sin(a1), 2 * math.cos(a1), 5.0, 7.0], dtype=torch.float64))


def test_window_by_hand():
    n = 6
    q = torch.zeros(n, 2, 2, dtype=torch.float64)
    k = torch.zeros(n, 1, 2, dtype=torch.float64)
    v = torch.arange(n, dtype=torch.float64).view(n, 1, 1)
    out = plain.window_attention(q, k, v, 1.0, 3)              # equal scores: the mean of the visible values
    assert torch.allclose(out[:, 0, 0], torch.tensor([0.0, 0.5, 1.0, 2.0, 3.0, 4.0], dtype=torch.float64))
    assert torch.allclose(plain.window_attention(q, k, v, 1.0, 1)[:, 1, 0], v.view(-1))
    assert torch.allclose(plain.window_attention(q, k, v, 1.0, None)[:, 0, 0], torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 2.5], dtype=torch.float64))


def test_recurrence_by_hand():
    q = torch.ones(3, 1, 1, dtype=torch.float64)
    k = torch.ones(3, 1, 1, dtype=torch.float64)
    v = torch.tensor([1.0, 10.0, 100.0], dtype=torch.float64).view(3, 1, 1)
    o, S = plain.linear_recurrence(q, k, v, torch.full((3, 1, 1), 0.5, dtype=torch.float64))
    assert o.view(-1).tolist() == [1.0, 10.5, 105.25] and float(S) == 105.25
    o2, _ = plain.linear_recurrence(q[2:], k[2:], v[2:], torch.full((1, 1, 1), 0.5, dtype=torch.float64), state=torch.tensor([[[10.5]]], dtype=torch.float64))
    assert float(o2) == 105.25


def test_mixture_by_hand():
    W = 2
    w = {"r.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [-1.0, -1.0]], dtype=torch.float64)}
    for e in range(3):
        w[f"r.e{e}.gate"] = torch.full((1, W), 50.0, dtype=torch.float64)       # silu(large) = itself
        w[f"r.e{e}.up"] = torch.full((1, W), float(e + 1), dtype=torch.float64)
        w[f"r.e{e}.down"] = torch.ones(W, 1, dtype=torch.float64)
    h = torch.tensor([[2.0, 1.0]], dtype=torch.float64)
    out = plain.mixture(h, w, "r.", {"router": {"experts": 3, "top": 2}})
    p0 = math.exp(2) / (math.exp(2) + math.exp(1))
    gate = 150.0                                                                 # 50 * (2 + 1)
    assert torch.allclose(out, torch.full((1, W), gate * (p0 * 3.0 + (1 - p0) * 6.0), dtype=torch.float64))


def test_layer_runs():
    assert plain.layer_runs({"layers": [0] * 4, "loop": {"start": 1, "stop": 3, "times": 2}}) == \
        [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert plain.layer_runs({"layers": [0] * 2}) == [(0, None), (1, None)]
