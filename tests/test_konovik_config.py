"""Konovik on the host: the registry, the configuration's keys and errors, the order in which looped
layers run and which cache and state each run gets, the loader's report, a random-weights folder, the
stretched rotary frequencies, and the plain functions against closed forms."""
import copy
import math

import numpy as np
import pytest
import torch

from lgml_b200.cache import FixedState, PagedKV
from lgml_b200.config import ConfigError, KonovikConfig, architectures, config_from_dict, load_config
from lgml_b200.models import build_model
from lgml_b200.parts.latent_attention import scaled_frequencies
from lgml_b200.weights import WeightError, index_folder, write_random_model
from lgml_b200.weights.loader import check_index
from tests import konovik_helpers as L
from tests.plain import konovik_plain as P


def test_registered_and_read_from_its_own_keys():
    assert "Konovik" in architectures()
    cfg = config_from_dict(copy.deepcopy(L.LOOPED))
    assert isinstance(cfg, KonovikConfig)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers, cfg.residual_mult, cfg.side_dim, cfg.loop) == (97, 64, 5, 0.5, 12, (1, 3, 3))
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    plain = config_from_dict(copy.deepcopy(L.ODD))
    assert (plain.residual_mult, plain.loop, plain.side_dim) == (1.0, None, 5)
    assert config_from_dict(copy.deepcopy(L.NO_SIDE)).side_dim == 0


@pytest.mark.parametrize("edit,word", [
    (lambda d: d.pop("width"), "width"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["layers"][0].update(type="conv"), "layers[0].type"),
    (lambda d: d["layers"][0]["mixer"].pop("width"), "width"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0.0), "factor"),
    (lambda d: d["layers"][1]["mixer"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda d: d["layers"][1]["mlp"]["shared"].pop("ff"), "ff"),
    (lambda d: d["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda d: d["loop"].update(stop=6), "loop"),
    (lambda d: d["loop"].update(start=3), "loop"),
    (lambda d: d["loop"].update(times=0), "loop"),
    (lambda d: d["loop"].pop("times"), "loop.times"),
    (lambda d: d["token_side"].update(dim=0), "dim"),
])
def test_errors_name_the_key(edit, word):
    d = copy.deepcopy(L.LOOPED)
    edit(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_looped_layers_run_in_order_and_every_run_has_its_own_cache_and_state():
    cfg = config_from_dict(copy.deepcopy(L.LOOPED))
    runs = cfg.layer_runs()
    assert [i for i, _ in runs] == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert [again for _, again in runs] == [False, False, False, True, False, True, False, False, False]
    assert runs == P.layer_runs(L.LOOPED)
    model = build_model(cfg)
    assert [(c.block, c.add_input, c.cache) for c in model.schedule] == [(i, again, None) for i, again in runs]
    layout = model.cache_layout()
    assert sorted(layout) == list(range(9))                            # one entry per run, not per layer
    assert layout[0] == FixedState((64 + 48,), torch.float32)         # the shifted row, then the recurrence
    for run in (1, 3, 5):
        assert layout[run] == (PagedKV(1, 24 + 8, 20, 24, v_in_k=True), FixedState((64,), torch.float32))
    for run in (2, 4, 6):
        assert layout[run] == FixedState((64 + 64,), torch.float32)
    assert layout[7] == (PagedKV(1, 40 + 12, 70, 40, v_in_k=True), FixedState((64,), torch.float32))
    assert layout[8] == FixedState((64 + 80,), torch.float32)
    # a loop over all layers, and none
    assert [i for i, _ in config_from_dict(copy.deepcopy(L.NO_SIDE)).layer_runs()] == [0, 1, 2, 0, 1, 2]
    assert [i for i, _ in config_from_dict(copy.deepcopy(L.ODD)).layer_runs()] == [0, 1, 2, 3]
    free = build_model(config_from_dict(copy.deepcopy(L.NO_SIDE))).cache_layout()
    assert free[0][0].window is None and free[2][0].window == 64


def test_which_parts_a_configuration_asks_for():
    model = build_model(config_from_dict(copy.deepcopy(L.LOOPED)))
    b0, b1, b2, b3 = model.blocks[:4]
    assert b0.residual_scale == 0.5 and b0.shift is not None and b0.side.col0 == 0 and b3.side.col0 == 36 and b3.side.table_cols == 60
    assert (b0.mixer.width, b0.mixer.inner) == (64, 48)
    m = b1.mixer
    assert (m.n_heads, m.head_dim, m.rot_dim, m.v_head_dim, m.rank, m.window, m.out_gate, m.scale) == (3, 16, 8, 12, 24, 20, True, 0.2)
    assert m.rope_scaling == {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0} and b3.mixer.rope_scaling is None
    f = b1.ffn
    assert (f.n_experts, f.top, f.router, f.route_scale, f.gated, f.shared_inner, f.inner) == (5, 2, "sigmoid", 1.5, False, 40, 24)
    assert b2.ffn.route_scale == 1.0 and b3.ffn is None and b3.ffn_norm is None
    assert model.blocks[4].ffn.inner == 48
    bare = build_model(config_from_dict(copy.deepcopy(L.NO_SIDE)))
    assert all(b.side is None for b in bare.blocks) and bare.blocks[0].ffn.shared_inner == 0


def test_folder_of_random_weights_and_the_loaders_report(tmp_path):
    cfg = config_from_dict(copy.deepcopy(L.ODD))
    folder = write_random_model(tmp_path / "m", cfg, seed=3)
    loaded = load_config(folder)
    assert loaded.to_dict() == cfg.to_dict()
    specs = build_model(loaded).tensor_specs()
    index = index_folder(folder)
    check_index(index, specs)
    names = set(index)
    assert {"embed", "embed.norm", "side.embed", "final.norm", "head", "l0.norm1", "l0.shift", "l0.mix.dkv.norm", "l0.mix.g", "l0.mlp.e0.down",
            "l0.mlp.router", "l0.mlp.correction", "l0.side.gate", "l0.side.norm", "l2.mix.z.b", "l2.mlp.shared.sg", "l3.mix.x"} <= names
    assert "l3.norm2" not in names and "l0.mlp.e0.gate" not in names and "l0.mlp.shared.up" not in names and "l0.mlp.e1.up" not in names
    assert tuple(index["embed.norm"].shape) == () and tuple(index["l1.norm2"].shape) == ()
    assert tuple(index["side.embed"].shape) == (61, 4 * 5) and tuple(index["l2.mlp.shared.sg"].shape) == (1, 36)
    index.pop("l2.mlp.correction")
    with pytest.raises(WeightError) as e:
        check_index(index, specs)
    assert "l2.mlp.correction" in e.value.missing


@pytest.mark.parametrize("base,dims,scaling", [(10000.0, 16, (8.0, 2048, 32.0, 1.0)), (5000.0, 8, (4.0, 64, 8.0, 1.0)), (50.0, 4, (2.0, 32, 4.0, 2.0)),
                                               (20000.0, 4, (8.0, 128, 16.0, 1.0)), (30000.0, 32, (4.0, 256, 32.0, 1.0)), (300.0, 12, None)])
def test_stretched_frequencies(base, dims, scaling):
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    got, mag = scaled_frequencies(base, dims, sc)
    want, want_mag = P.yarn_frequencies(base, dims, sc)
    assert np.allclose(got, want, rtol=1e-14, atol=0) and mag == pytest.approx(want_mag, rel=1e-14)
    plain = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    if sc is None:
        assert np.array_equal(want, plain) and want_mag == 1.0
        return
    # the fastest pair keeps its frequency unless the ramp starts at it; the slowest is divided by the factor once the ramp has ended
    ratio = want / plain
    assert np.all(ratio <= 1.0 + 1e-15) and np.all(ratio >= 1.0 / sc["factor"] - 1e-15) and np.all(np.diff(ratio) <= 1e-15)
    assert want_mag == pytest.approx(0.1 * math.log(sc["factor"]) + 1.0)


def test_the_ramp_of_the_stretched_frequencies_by_hand():
    # base 100, 8 rotated entries, original 100: n(t) = 8 ln(100 / (2 pi t)) / (2 ln 100); n(4) = 1.2 -> lo 1; n(0.5) = 3.005 -> hi min(4, 7) = 4
    f, mag = P.yarn_frequencies(100.0, 8, {"factor": 10.0, "original": 100, "fast": 4.0, "slow": 0.5})
    plain = np.array([1.0, 100.0 ** -0.25, 100.0 ** -0.5, 100.0 ** -0.75])
    r = np.array([0.0, 0.0, 1.0 / 3.0, 2.0 / 3.0])
    assert np.allclose(f, plain / 10.0 * r + plain * (1.0 - r)) and mag == pytest.approx(0.1 * math.log(10.0) + 1.0)


def test_plain_functions_against_closed_forms():
    # the shift: row t moves towards the unshifted row t - 1, the first towards zeros
    h = np.array([[2.0, 4.0], [6.0, 8.0], [10.0, 0.0]])
    assert np.allclose(P.token_shift(h, np.array([0.5, 0.0])), [[1.0, 4.0], [4.0, 8.0], [8.0, 0.0]])
    assert np.allclose(P.token_shift(h, np.array([1.0, 1.0])), [[0.0, 0.0], [2.0, 4.0], [6.0, 8.0]])
    # the norm with one number
    assert np.allclose(P.scalar_norm(np.array([[3.0, 4.0]]), 2.0, 0.0), [[6.0 / math.sqrt(12.5), 8.0 / math.sqrt(12.5)]])
    # the recurrence: z = 1/2 throughout (logit 0); u = 1 -> candidate 1.5, then u = -inf-ish -> candidate sigmoid(-30) ~ 0
    eye = np.eye(1)
    W = {"m.z": np.zeros((1, 1)), "m.z.b": np.zeros(1), "m.x": eye, "m.x.b": np.zeros(1), "m.g": np.zeros((1, 1)), "m.o": eye}
    hh = np.array([[1.0], [1.0], [-30.0]])
    W["m.g"] = np.array([[0.0]])
    assert np.allclose(P.min_gru(hh, W, "m"), 0.0)                     # silu(0) = 0 closes the output
    W["m.g"] = np.array([[1.0]])
    silu = lambda v: v / (1.0 + math.exp(-v))
    S = [0.75, 0.375 + 0.75, 0.5 * 1.125 + 0.5 / (1.0 + math.exp(30.0))]
    assert np.allclose(P.min_gru(hh, W, "m")[:, 0], [S[0] * silu(1.0), S[1] * silu(1.0), S[2] * silu(-30.0)])
    # the candidate's two branches meet at u = 0 (both 1/2)
    W["m.z.b"] = np.array([60.0])                                       # z = 1: the state is the candidate
    W["m.g"], W["m.x"], W["m.x.b"] = np.zeros((1, 1)), np.zeros((1, 1)), np.array([0.0])
    W["m.o"] = np.array([[1.0]])
    for ub, cand in ((0.0, 0.5), (-1e-12, 0.5), (2.0, 2.5), (-2.0, 1.0 / (1.0 + math.exp(2.0)))):
        Wc = {**W, "m.x.b": np.array([ub]), "m.g": np.array([[1.0]])}
        assert np.allclose(P.min_gru(np.array([[1.0]]), Wc, "m"), [[cand * silu(1.0)]])
    # the window: position 10 with a window of 3 sees 8, 9, 10; a window of 1 only itself
    assert list(np.nonzero(P.visible(12, 3)[10])[0]) == [8, 9, 10] and list(np.nonzero(P.visible(5, 1)[4])[0]) == [4]
    assert list(np.nonzero(P.visible(5, None)[3])[0]) == [0, 1, 2, 3]
    # rotation: pairs (2i, 2i + 1) turn by p f_i, both parts times the factor; entries past dims pass
    v = np.zeros((3, 6)); v[:, 0] = 1.0; v[:, 2] = 1.0; v[:, 4] = 7.0
    r = P.rotate_interleaved(v, {"base": 100.0, "dims": 4}, [0, 1, 2])
    assert np.allclose(r[2], [np.cos(2.0), np.sin(2.0), np.cos(0.2), np.sin(0.2), 7.0, 0.0])
    # the router: scores sigmoid(0, 2, 1); the correction (3, 0, 0) brings expert 0 in; top 2 = experts 0 and 1 with weights from the scores alone
    Wf = {"f.router": np.array([[0.0], [2.0], [1.0]]), "f.correction": np.array([3.0, 0.0, 0.0])}
    for e in range(3):
        Wf[f"f.e{e}.up"], Wf[f"f.e{e}.down"] = np.array([[2.0]]), np.array([[float(10 ** e)]])
    f = {"router": {"experts": 3, "top": 2, "scale": 3.0}}
    s0, s1 = 0.5, 1.0 / (1.0 + math.exp(-2.0))
    y = P.routed_ff(np.array([[1.0]]), Wf, "f", f)
    assert np.allclose(y, [[3.0 * 4.0 * (s0 * 1.0 + s1 * 10.0) / (s0 + s1)]])
    assert np.allclose(P.routed_ff(np.array([[-1.0]]), Wf, "f", f), 0.0)           # relu closes a negative input
    # a shared expert behind its own gate
    Wf.update({"f.shared.up": np.array([[1.0]]), "f.shared.down": np.array([[100.0]]), "f.shared.sg": np.array([[0.0]])})
    y2 = P.routed_ff(np.array([[1.0]]), Wf, "f", {**f, "shared": {"ff": 1}})
    assert np.allclose(y2 - y, [[0.5 * 100.0]])
    # the token input: y = proj (gelu(gate x) e), unit root mean square, times the weight
    Ws = {"s.gate": np.array([[1.0, 0.0]]), "s.proj": np.array([[1.0], [-1.0]]), "s.norm": np.array([2.0, 3.0])}
    out = P.side_input(np.array([[1.5, 9.0]]), Ws, "s", np.array([[0.7]]), 0.0)
    assert np.allclose(out, [[2.0, -3.0]])
    assert np.allclose(P.gelu_tanh(np.array([0.0, 10.0, -10.0])), [0.0, 10.0, 0.0], atol=1e-9)
