"""Dizepel on the host: registry, configuration keys and errors, the order of looped layers, which cache and state
every run gets, the tensors the model asks for, and the plain functions against closed forms."""
import copy
import math

import numpy as np
import pytest
import torch

from lgml_b200.cache import FixedState, PagedKV
from lgml_b200.config import ConfigError, DizepelConfig, architectures, config_from_dict
from lgml_b200.models import build_model
from tests import dizepel_helpers as L
from tests.plain import dizepel_plain as P


def test_registered_by_name():
    assert "Dizepel" in architectures()
    cfg = config_from_dict(L.LOOPED)
    assert isinstance(cfg, DizepelConfig) and cfg.vocab_size == 97 and cfg.hidden_size == 64 and cfg.num_hidden_layers == 4
    assert cfg.embed_scale == 2.5 and cfg.canon_taps == 3 and cfg.loop == (1, 3, 3)
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    plain = config_from_dict(L.ODD)
    assert plain.embed_scale == 1.0 and plain.loop is None and plain.canon_taps == 4
    assert config_from_dict(L.WIDE_HEADS).canon_taps == 0


@pytest.mark.parametrize("edit,key", [
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["norm"].pop("eps"), "norm"),
    (lambda d: d["layers"][0].__setitem__("type", "serial"), "layers[0].type"),
    (lambda d: d["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 2), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["left"].__setitem__("vdim", 40), "vdim"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda d: d["layers"][2]["mixer"]["right"].__setitem__("groups", 3), "groups"),
    (lambda d: d["layers"][2]["mixer"]["right"].__setitem__("norm_groups", 3), "norm_groups"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "moe"), "mlp.kind"),
    (lambda d: d["loop"].__setitem__("stop", 9), "loop"),
    (lambda d: d["canon"].__setitem__("taps", 0), "canon.taps"),
])
def test_a_bad_key_is_named(edit, key):
    d = copy.deepcopy(L.LOOPED)
    edit(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert key.split(".")[-1] in str(e.value)


def test_order_of_looped_layers_and_their_pass_vectors():
    assert config_from_dict(L.LOOPED).layer_runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert config_from_dict(L.WIDE_HEADS).layer_runs() == [(0, 0), (1, None), (0, 1), (1, None)]
    assert config_from_dict(L.TAIL_LOOP).layer_runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None)]
    assert config_from_dict(L.ODD).layer_runs() == [(0, None), (1, None)]
    assert P.layer_runs(L.LOOPED) == config_from_dict(L.LOOPED).layer_runs()


def test_every_run_has_its_own_cache_and_state():
    model = build_model(config_from_dict(L.LOOPED))
    layout = model.cache_layout()
    assert sorted(layout) == list(range(8))
    E = 64
    for ci, call in enumerate(model.schedule):
        layer = L.LOOPED["layers"][call.block]
        l, r = layer["mixer"]["left"], layer["mixer"]["right"]
        pages, state = layout[ci]
        assert pages == PagedKV(l["kv_heads"], l["dim"], None, l["vdim"])
        convs = 2 * E * (2 if layer["mlp"] else 1)
        left_state = (l["conv"] - 1) * (l["heads"] + l["kv_heads"]) * l["dim"]
        inner = r["heads"] * r["vdim"]
        right_state = inner * r["state"] + (r["conv"] - 1) * (inner + 2 * r["groups"] * r["state"])
        assert state == FixedState((convs + left_state + right_state,), torch.float32)
    assert [c.add_row for c in model.schedule] == [None, 0, None, 1, None, 2, None, None]
    assert model.graph_safe


def test_tensors_the_model_asks_for():
    for cfg in L.CONFIGS.values():
        names = {s.name: tuple(s.shape) for s in build_model(config_from_dict(cfg)).tensor_specs()}
        made = L.random_weights(cfg, 1)
        assert {n: tuple(t.shape) for n, t in made.items()} == names


def test_plain_functions_against_closed_forms():
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    assert np.allclose(P.layer_norm(x, np.ones(4), 0.0), (x - 3.0) / math.sqrt(3.5))
    assert np.allclose(P.rms_unit(x, 0.0), x / math.sqrt(12.5))
    u = np.arange(1.0, 6.0)[:, None]
    w = np.array([[0.5, 0.0, 2.0]])                         # the last column weighs the current row
    assert np.allclose(P.causal_conv(u, w)[:, 0], [2.0, 4.0, 6.5, 9.0, 11.5])
    f, mag = P.stretched_frequencies(100.0, 4, None)
    assert np.allclose(f, [1.0, 0.1]) and mag == 1.0
    f, mag = P.stretched_frequencies(100.0, 4, {"factor": 4.0, "original": 8, "fast": 1e9, "slow": 1e-9})
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    q = np.zeros((2, 1, 4)); q[:, 0, 0] = 1.0
    turned = P.rotate_halves(q, {"base": 100.0, "dims": 2}, [0, 1])
    assert np.allclose(turned[1, 0], [math.cos(1.0), math.sin(1.0), 0.0, 0.0])
    # one key, a sink of equal weight: half the value comes through; a cap far below the score replaces it
    o = P.capped_sink_attention(np.ones((1, 1, 2)), np.ones((1, 1, 2)), np.full((1, 1, 3), 4.0), 1.0, None, [2.0])
    assert np.allclose(o, 2.0)
    o = P.capped_sink_attention(np.ones((1, 1, 2)) * 50, np.ones((1, 1, 2)), np.full((1, 1, 3), 4.0), 1.0, 1.0, [1.0])
    assert np.allclose(o, 4.0 * math.e ** math.tanh(100.0) / (math.e ** math.tanh(100.0) + math.e))
    # a state that only decays: y_t = C . (B x_0) exp(-a dt)^t after the first token
    T = 5
    x = np.zeros((T, 1, 1)); x[0] = 1.0
    y = P.state_space_scan(x, np.full((T, 1), 0.5), np.array([2.0]), np.ones((T, 1, 3)), np.ones((T, 1, 3)), np.array([0.0]))
    assert np.allclose(y[:, 0, 0], [0.5 * 3 * math.exp(-1.0 * t) for t in range(T)])
    z = np.array([[1.0, -2.0]])
    want = 2.0 * z / math.sqrt(2.5) + 3.0 * z ** 2 / math.sqrt(8.5) + 0.5 * z ** 3 / math.sqrt(32.5) + 0.25
    assert np.allclose(P.poly_norm(z, [2.0, 3.0, 0.5, 0.25], 0.0), want)
