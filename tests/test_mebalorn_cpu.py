"""Mebalorn without a GPU: the configuration reader, the plan it makes, the tensors it expects, the random-weights
writer, and properties of the plain implementation that the GPU tests lean on."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_mebalorn as plain
from mebalorn_models import CONFIGS, make_weights, tensor_shapes

from pico_engine.config import ConfigError, config_from_dict, read_config
from pico_engine.config.mebalorn import MebalornConfig
from pico_engine.config.specs import CausalConvAddSpec, DenseMLPSpec, HeadMixAttentionSpec, LayerNormSpec, MinGRUSpec


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_config_round_trip_and_expected_tensors(name):
    d = CONFIGS[name]
    cfg = config_from_dict(d)
    assert isinstance(cfg, MebalornConfig) and cfg.to_dict() == d
    from pico_engine.config.registry import architecture
    model = architecture(cfg.ARCHITECTURE).build_model(cfg, torch.bfloat16, "meta")
    assert {n: tuple(s.shape) for n, s in model.expected_tensors().items()} == tensor_shapes(d)


def test_plan_follows_the_layer_list():
    d = CONFIGS["M1"]
    plan = config_from_dict(d).plan()
    assert [type(l.mixer) for l in plan.layers] == [HeadMixAttentionSpec, MinGRUSpec, HeadMixAttentionSpec, MinGRUSpec]
    a = plan.layers[0].mixer
    assert (a.n_heads, a.n_kv_heads, a.head_dim, a.v_head_dim, a.scale) == (6, 2, 32, 16, 0.21)
    assert plan.layers[1].feed_forward is None and plan.layers[1].feed_forward_norm is None
    assert isinstance(plan.layers[3].feed_forward, DenseMLPSpec) and plan.layers[3].feed_forward.intermediate == 200
    assert all(l.arrangement == "parallel" and isinstance(l.mixer_norm, LayerNormSpec) for l in plan.layers)
    assert all(isinstance(l.mixer_input, CausalConvAddSpec) and l.mixer_input.taps == 4 for l in plan.layers)
    assert plan.logit_softcap == 9.0 and config_from_dict(CONFIGS["M2"]).plan().logit_softcap is None


def test_state_a_layer_keeps():
    """The recurrence's state, then taps - 1 rows of the model's width for every sublayer that has a convolution."""
    from pico_engine.config.registry import architecture
    cfg = config_from_dict(CONFIGS["M1"])
    model = architecture(cfg.ARCHITECTURE).build_model(cfg, torch.float32, "meta")
    needs = model.cache_needs()
    assert [n.state_elems for n in needs] == [2 * 3 * 72, 40 + 3 * 72, 2 * 3 * 72, 96 + 2 * 3 * 72]
    assert needs[0].kv.value_shape == (2, 16) and needs[2].kv.value_shape == (4, 48) and needs[1].kv is None
    one_tap = config_from_dict(CONFIGS["M2"])
    needs = architecture(one_tap.ARCHITECTURE).build_model(one_tap, torch.float32, "meta").cache_needs()
    assert [n.state_elems for n in needs] == [48, 0]


@pytest.mark.parametrize("change, word", [
    (lambda d: d["layers"][0].update(type="mamba"), "type"),
    (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=4), "evenly"),
    (lambda d: d["layers"][1]["mixer"].pop("width"), "width"),
    (lambda d: d.pop("canon"), "canon"),
    (lambda d: d["norm"].update(eps=0), "eps"),
])
def test_config_errors_name_the_key(change, word):
    d = copy.deepcopy(CONFIGS["M1"])
    change(d)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_random_model_folder_loads(tmp_path):
    from pico_engine.weights import write_random_model
    from pico_engine.weights.safetensors_io import Checkpoint
    cfg = config_from_dict(CONFIGS["M3"])
    write_random_model(cfg, 5, str(tmp_path))
    assert read_config(str(tmp_path)) == cfg
    ck = Checkpoint(str(tmp_path))
    assert {n: tuple(e.shape) for n, e in ck.entries.items()} == tensor_shapes(CONFIGS["M3"])
    talk = ck.read("l0.mix.talk").float()
    assert (talk.diagonal() - 1).abs().max() < 0.2 and (talk - torch.eye(2)).abs().max() < 0.2


# ------------------------------------------------------------------ the plain implementation

def test_plain_is_causal_and_positions_count_from_zero():
    cfg = CONFIGS["M1"]
    w = make_weights(cfg, 1)
    toks = torch.randint(0, cfg["vocab"], (19,), generator=torch.Generator().manual_seed(3)).tolist()
    full = plain.logits(toks, w, cfg)
    assert torch.allclose(plain.logits(toks[:11], w, cfg), full[:11], atol=1e-10)
    assert not torch.allclose(plain.logits(toks[1:12], w, cfg)[:-1], full[1:11], atol=1e-3)      # positions matter


def test_plain_convolution_by_hand():
    h = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 0.25, 2.0], [0.0, 1.0, 0.0]], dtype=torch.float64)        # [width, taps], the last tap is the token itself
    out = plain.input_conv(h, w)
    assert out[0].tolist() == [1 + 2 * 1, 10.0]
    assert out[1].tolist() == [2 + 0.25 * 1 + 2 * 2, 20 + 10.0]
    assert out[2].tolist() == [3 + 0.5 * 1 + 0.25 * 2 + 2 * 3, 30 + 20.0]


def test_plain_sink_and_mixing_by_hand():
    """One key, two heads: the softmax weight is e^s / (e^s + e^sink); mixing swaps or sums the heads' weights."""
    q = torch.tensor([[[1.0], [2.0]]], dtype=torch.float64)      # [n=1, H=2, D=1]
    k = torch.tensor([[[3.0]]], dtype=torch.float64)             # G = 1
    v = torch.tensor([[[1.0, -1.0]]], dtype=torch.float64)
    sink = torch.tensor([0.0, 6.0], dtype=torch.float64)
    w0 = 1 / (1 + torch.exp(torch.tensor(-3.0, dtype=torch.float64)))
    w1 = torch.tensor(0.5, dtype=torch.float64)
    out = plain.mixed_attention(q, k, v, 1.0, sink, None)
    assert torch.allclose(out[0, :, 0], torch.stack([w0, w1]))
    swap = torch.tensor([[0.0, 1.0], [1.0, 0.0]], dtype=torch.float64)
    assert torch.allclose(plain.mixed_attention(q, k, v, 1.0, sink, swap)[0, :, 0], torch.stack([w1, w0]))
    both = torch.tensor([[1.0, 1.0], [0.0, -2.0]], dtype=torch.float64)
    assert torch.allclose(plain.mixed_attention(q, k, v, 1.0, sink, both)[0, :, 1], -torch.stack([w0 + w1, -2 * w1]))


def test_plain_recurrence_by_hand():
    pz = torch.tensor([[0.0], [0.0]], dtype=torch.float64)        # z = 1/2
    pu = torch.tensor([[1.5], [-30.0]], dtype=torch.float64)      # candidates 2 and ~0
    pg = torch.tensor([[50.0], [50.0]], dtype=torch.float64)      # silu(50) = 50
    y, S = plain.mingru_recurrence(pz, pu, pg)
    assert torch.allclose(y[:, 0] / 50, torch.tensor([1.0, 0.5], dtype=torch.float64), atol=1e-9) and abs(float(S) - 0.5) < 1e-9
    assert plain.mingru_candidate(torch.tensor([0.0, -0.0, 1e-30])).tolist() == [0.5, 0.5, 0.5]
