"""Dizepel in the engine against the plain implementation: every mechanism alone, then whole models under every
way of cutting the work.

The models are small and differ from each other in every size and option (one to six heads of 8 to 128 entries,
values shorter than keys, 2 to all entries of a head rotated, stretched and plain frequencies, capped and uncapped
scores, states of 5 to 128 numbers, convolutions of 1 to 5 taps, loops at the start, in the middle and at the end,
layers without a feed-forward).  Where random numbers would hide a fault, the inputs are made so that it shows: one
far key carries the largest score, the sink outweighs the keys, scores lie far beyond the cap, the recurrence decays
so slowly that a state from hundreds of tokens back still decides the output.
"""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import dizepel_helpers as L
from tests import helpers as H
from tests.plain import dizepel_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": dict(atol=3e-5, rtol=2e-4), "bfloat16": dict(atol=3e-2, rtol=0.12)}


def i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def f32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV)


def batch_of(lens):
    """(request index of every token, first token row of every request) of a step with these portions."""
    seq_of = [r for r, n in enumerate(lens) for _ in range(n)]
    return i32(seq_of), i32(np.concatenate([[0], np.cumsum(lens)]))


def portions_of(total, cuts):
    out, a, i = [], 0, 0
    while a < total:
        b = min(total, a + cuts[i % len(cuts)])
        out.append((a, b))
        a, i = b, i + 1
    return out


# ---------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E", [36, 64, 321, 1030])
def test_norm_of_what_is_read_and_of_what_is_added(out_dtype, E):
    from lgml_b200 import ops

    rng = np.random.default_rng(E)
    n, eps = 7, 1e-5
    x, a, b = rng.normal(size=(n, E)) * 3 + 1.5, rng.normal(size=(n, E)) * 2 + 0.7, rng.normal(size=(n, E)) * 0.1
    ua, ub, wpost, wpre, row = (rng.normal(size=E) * 0.3 + 1 for _ in range(5))
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    # two results, each over its own root mean square, the norm on their half sum, one more row, the norm on x
    xd, out = f32(x), torch.empty((n, E), dtype=out_dtype, device=DEV)
    ops.sandwich_norm(xd, f32(wpre), eps, out, delta=(f32(a), f32(b)), units=(f32(ua), f32(ub)), w_post=f32(wpost), row_add=f32(row))
    m = 0.5 * (P.rms_unit(a, eps) * ua + P.rms_unit(b, eps) * ub)
    want_x = x + P.layer_norm(m, wpost, eps) + row
    assert np.abs(xd.cpu().numpy() - want_x).max() < 1e-5
    assert np.abs(out.float().cpu().numpy() - P.layer_norm(want_x, wpre, eps)).max() < tol * 4
    # one result, chosen rows only: x stays as it was
    xd, rows = f32(x), i32([5, 0, 5])
    out = torch.empty((3, E), dtype=out_dtype, device=DEV)
    ops.sandwich_norm(xd, f32(wpre), eps, out, delta=f32(a), w_post=f32(wpost), rows=rows)
    assert torch.equal(xd, f32(x))
    want = P.layer_norm(x + P.layer_norm(a, wpost, eps), wpre, eps)[[5, 0, 5]]
    assert np.abs(out.float().cpu().numpy() - want).max() < tol * 4
    # nothing pending but a row; then nothing at all; then a delta that is added as it is and no output
    xd = f32(x)
    ops.sandwich_norm(xd, f32(wpre), eps, out := torch.empty((n, E), dtype=out_dtype, device=DEV), row_add=f32(row))
    assert np.abs(xd.cpu().numpy() - (x + row)).max() < 1e-6
    assert np.abs(out.float().cpu().numpy() - P.layer_norm(x + row, wpre, eps)).max() < tol * 4
    xd = f32(x)
    ops.sandwich_norm(xd, None, eps, None, delta=f32(a))
    assert np.abs(xd.cpu().numpy() - (x + a)).max() < 1e-6


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,C,act,residual", [(1, 20, "none", True), (2, 33, "silu", False), (3, 64, "none", True), (4, 130, "silu", False),
                                                 (5, 8, "none", False), (8, 12, "silu", True)])
def test_short_convolution_across_steps_requests_and_reused_slots(out_dtype, taps, C, act, residual):
    """Three requests in slots 2, 0, 3 of 4, their tokens cut into steps of 1, 2, 5 ... tokens (fewer than the taps
    reach back, more, hundreds, and none for a request in some steps); then the slots are cleared and used again."""
    from lgml_b200 import ops

    rng = np.random.default_rng(taps * 100 + C)
    w, bias = rng.normal(size=(C, taps)), rng.normal(size=C) if act == "silu" else None
    lens, slots = [23, 9, 340], [2, 0, 3]
    state = torch.full((4, (taps - 1) * C + 3), 7.0, device=DEV)
    for round_ in range(2):
        us = [rng.normal(size=(n, C + 5)) for n in lens]
        state[slots, :(taps - 1) * C] = 0.0
        done = [0, 0, 0]
        cuts = [[1, 1, 2, 1, 5, 64], [2, 1, 1, 64], [3, 1, 1, 1, 17, 290, 64]]      # (a step of 256 tokens or more: four tokens a thread)
        got = [np.zeros((n, C)) for n in lens]
        step = 0
        while any(d < n for d, n in zip(done, lens)):
            who = [r for r in range(3) if done[r] < lens[r] and (step + r) % 4 != 3]
            take = [min(cuts[r][min(step, len(cuts[r]) - 1)], lens[r] - done[r]) for r in who]
            step += 1
            if not who:
                continue
            u = np.concatenate([us[r][done[r]:done[r] + k] for r, k in zip(who, take)])
            seq_of, starts = batch_of(take)
            out = torch.empty((u.shape[0], C), dtype=out_dtype, device=DEV)
            ops.short_conv(f32(u)[:, 2:2 + C], f32(w.T.copy()), f32(bias) if bias is not None else None, state[:, :max((taps - 1) * C, 1)] if taps > 1 else None,
                           seq_of, starts, i32([slots[r] for r in who]), out, act=act, residual=residual)
            o = out.float().cpu().numpy()
            at = 0
            for r, k in zip(who, take):
                got[r][done[r]:done[r] + k] = o[at:at + k]
                at += k
                done[r] += k
        for r in range(3):
            u = us[r][:, 2:2 + C]
            want = P.causal_conv(u, w, bias)
            if act == "silu":
                want = P.silu(want)
            if residual:
                want = want + u
            tol = 2e-5 if out_dtype == torch.float32 else 3e-2
            assert np.abs(got[r] - want).max() < tol * (1 + np.abs(want).max()), f"round {round_} request {r}"
        assert bool((state[1] == 7.0).all()) and bool((state[:, (taps - 1) * C:] == 7.0).all() or taps == 1)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("F", [20, 64, 333, 1500])
def test_polynomial_of_normed_powers(out_dtype, F):
    from lgml_b200 import ops

    rng = np.random.default_rng(F)
    z = rng.normal(size=(5, F)) * 1.7
    coef = np.array([0.9, -0.6, 0.3, 0.2])
    out = torch.empty((5, F), dtype=out_dtype, device=DEV)
    ops.poly_norm(f32(z), f32(coef), 1e-6, out)
    want = P.poly_norm(z, coef, 1e-6)
    assert np.abs(out.float().cpu().numpy() - want).max() < (2e-5 if out_dtype == torch.float32 else 3e-2) * (1 + np.abs(want).max())


@pytest.mark.parametrize("Hs,G,Pd,N", [(1, 1, 20, 5), (4, 2, 8, 12), (6, 3, 12, 20), (2, 1, 40, 33), (3, 3, 32, 48), (3, 1, 32, 128), (2, 2, 64, 100),
                                      (8, 8, 4, 8), (2, 1, 16, 300)])
def test_state_space_scan_whole_in_pieces_and_token_by_token_with_slow_decay(Hs, G, Pd, N):
    """Decays of exp(-0.002) a token: what the first tokens wrote still makes up much of the output 300 tokens on.  Two
    requests of unequal length in slots 3 and 1, whole, in portions and one token a step."""
    from lgml_b200 import ops

    rng = np.random.default_rng(Hs * 1000 + N)
    inner, lens, slots = Hs * Pd, [300, 41], [3, 1]
    a_log, dt_bias, dskip = rng.normal(size=Hs) * 0.3 - 3.0, rng.normal(size=Hs) * 0.3 - 2.5, rng.normal(size=Hs) + 1
    xs = [rng.normal(size=(n, inner + 2 * G * N + 3)) for n in lens]       # x | B | C with three spare columns behind
    dts = [rng.normal(size=(n, Hs)) * 0.5 for n in lens]
    xs[0][:3] *= 6.0                                                        # the first tokens write the most
    want = []
    for x, dt in zip(xs, dts):
        n = x.shape[0]
        y = P.state_space_scan(x[:, :inner].reshape(n, Hs, Pd), P.softplus(dt + dt_bias), np.exp(a_log), x[:, inner:inner + G * N].reshape(n, G, N),
                               x[:, inner + G * N:inner + 2 * G * N].reshape(n, G, N), dskip)
        want.append(y.reshape(n, inner))
    share = np.abs(want[0][-1]).max()
    for cuts in ([400], [7, 2, 19, 3, 64, 2, 33, 5, 2, 70], [1]):
        state = torch.zeros((4, inner * N + 5), device=DEV)
        got = [np.zeros_like(w) for w in want]
        done = [0, 0]
        k = 0
        while any(d < n for d, n in zip(done, lens)):
            who = [r for r in range(2) if done[r] < lens[r]]
            take = [min(cuts[k % len(cuts)], lens[r] - done[r]) for r in who]
            k += 1
            x = np.concatenate([xs[r][done[r]:done[r] + t] for r, t in zip(who, take)])
            dt = np.concatenate([dts[r][done[r]:done[r] + t] for r, t in zip(who, take)])
            _, starts = batch_of(take)
            y = ops.ssd_scan(f32(x)[:, :inner + 2 * G * N], f32(dt), f32(dt_bias), f32(a_log), f32(dskip), state, starts, i32([slots[r] for r in who]),
                             Hs, G, Pd, N).cpu().numpy()
            at = 0
            for r, t in zip(who, take):
                got[r][done[r]:done[r] + t] = y[at:at + t]
                at += t
                done[r] += t
        for r in range(2):
            assert np.abs(got[r] - want[r]).max() < 2e-4 * (1 + np.abs(want[r]).max()), f"cuts {cuts[:3]} request {r}"
        assert bool((state[[0, 2]] == 0).all()) and bool((state[:, inner * N:] == 0).all())
    assert share > 0.05
    # in pieces that run side by side: first 100 tokens of both requests in pieces of 16, then the rest in pieces of 64 beside each other
    state = torch.zeros((4, inner * N + 5), device=DEV)
    for (a0, b0), (a1, b1), size in (((0, 100), (0, 30), 16), ((100, 300), (30, 41), 64)):
        x = np.concatenate([xs[0][a0:b0], xs[1][a1:b1]])
        dt = np.concatenate([dts[0][a0:b0], dts[1][a1:b1]])
        rows, first, at = [], [0], 0
        for n in (b0 - a0, b1 - a1):
            rows += [(at + t, at + min(t + size, n)) for t in range(0, n, size)]
            first.append(len(rows))
            at += n
        pieces = (torch.tensor(rows, dtype=torch.int32, device=DEV), i32(first))
        y = ops.ssd_scan(f32(x)[:, :inner + 2 * G * N], f32(dt), f32(dt_bias), f32(a_log), f32(dskip), state, i32([0, b0 - a0, b0 - a0 + b1 - a1]),
                         i32(slots), Hs, G, Pd, N, pieces=pieces).cpu().numpy()
        for got_rows, w in ((y[:b0 - a0], want[0][a0:b0]), (y[b0 - a0:], want[1][a1:b1])):
            assert np.abs(got_rows - w).max() < 2e-4 * (1 + np.abs(w).max()), f"pieces of {size}"


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,groups", [(20, 1), (48, 3), (96, 2), (640, 5)])
def test_gate_then_norm_in_parts(out_dtype, inner, groups):
    from lgml_b200 import ops

    rng = np.random.default_rng(inner)
    y, z, w = rng.normal(size=(6, inner)) * 2, rng.normal(size=(6, inner + 4)) * 2, rng.normal(size=inner) * 0.3 + 1
    out = ops.ssd_gate_norm(f32(y), f32(z)[:, 1:1 + inner], f32(w), groups, 1e-5, out_dtype)
    want = P.grouped_rms(y * P.silu(z[:, 1:1 + inner]), groups, 1e-5) * w
    assert np.abs(out.float().cpu().numpy() - want).max() < (2e-5 if out_dtype == torch.float32 else 3e-2) * (1 + np.abs(want).max())


def attention_case(H, G, D, Dv, taps, dims, scaling, softcap, T, seed, loud):
    """Projected q and k rows of T tokens such that, after the convolution and the turn, the last token's queries find
    the key at position ``loud`` with a score far above the cap's linear range, and a sink that outweighs the rest."""
    rng = np.random.default_rng(seed)
    C = (H + G) * D
    proj = rng.normal(size=(T, C + 6)) * 0.5
    w = rng.normal(size=(C, taps)) * 0.3
    w[:, -1] += 1.0
    sink = rng.normal(size=H) + 1.0
    rot = {"base": 3000.0, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    # the unrotated entries of the loud key and of the last queries point the same way
    proj[loud, H * D:C] *= 0.2
    proj[T - 1, :H * D] *= 0.2
    for g in range(G):
        proj[loud, H * D + g * D + dims:H * D + (g + 1) * D] += 3.0
    for h in range(H):
        proj[T - 1, h * D + dims:(h + 1) * D] += 3.0
    return proj, w, sink, rot


@pytest.mark.parametrize("dtype,form", [(torch.float32, "general"), (torch.bfloat16, "general"), (torch.bfloat16, "split"), (torch.bfloat16, "tensor")])
@pytest.mark.parametrize("shape", [(4, 2, 16, 16, 4, 8, (4.0, 64, 8.0, 1.0), 8.0), (3, 3, 24, 20, 2, 24, None, 30.0), (1, 1, 12, 12, 1, 4, None, None),
                                   (4, 2, 64, 64, 4, 48, (6.0, 128, 24.0, 1.0), 25.0), (2, 1, 128, 128, 3, 64, None, 15.0),
                                   (2, 2, 48, 16, 3, 24, None, 10.0), (6, 2, 8, 4, 4, 2, None, 3.0)])
@pytest.mark.parametrize("T,loud", [(150, 0), (150, 63), (150, 64), (131, 100), (70, 69)])
def test_convolved_rotated_keys_as_values_under_a_cap_with_a_sink(dtype, form, shape, T, loud):
    """The convolution, the values taken from the keys, the turn, the cache write and attention in all kernel forms,
    with the tokens cut into steps that end inside, at and past pages; a loud key far back, at a page's edge, next to it."""
    from lgml_b200 import ops
    from lgml_b200.engine.runtime import Runtime
    from lgml_b200.parts.latent_attention import scaled_frequencies

    H, G, D, Dv, taps, dims, scaling, softcap = shape
    if form == "tensor" and D > 128:
        pytest.skip("no tensor-core form for this head size")
    proj, w, sink, rot = attention_case(H, G, D, Dv, taps, dims, scaling, softcap, T, seed=T + loud + D, loud=loud)
    scale = 1.0 / D ** 0.5 * 1.5
    C = (H + G) * D
    qk = P.causal_conv(proj[:, :C], w)
    q, k = qk[:, :H * D].reshape(T, H, D), qk[:, H * D:].reshape(T, G, D)
    v = k[..., :Dv].copy()
    pos = np.arange(T)
    want = P.capped_sink_attention(P.rotate_halves(q, rot, pos), P.rotate_halves(k, rot, pos), v, scale, softcap, sink).reshape(T, H * Dv)
    if softcap and dims < D:
        raw = np.einsum("hd,hd->h", P.rotate_halves(q, rot, pos)[T - 1], P.rotate_halves(k, rot, pos)[loud][np.arange(H) // (H // G)]) * scale
        assert np.abs(raw).max() > softcap * 0.8, "the loud score does not reach the cap"
    # a cap that is ignored (where the loud score reaches it), a sink that is left out, or values taken after the turn must show
    qr, kr = P.rotate_halves(q, rot, pos), P.rotate_halves(k, rot, pos)
    others = [P.capped_sink_attention(qr, kr, v, scale, softcap, sink - 30.0), P.capped_sink_attention(qr, kr, kr[..., :Dv], scale, softcap, sink)]
    if softcap and dims < D:
        others.append(P.capped_sink_attention(qr, kr, v, scale, None, sink))
    for other in others:
        assert np.abs(other.reshape(T, -1) - want).max() > 3e-4 * (1 + np.abs(want).max())        # ten times the float32 bound below

    rt = Runtime(DEV, dtype)
    freq, mag = scaled_frequencies(rot["base"], dims, rot.get("scaling"))
    exact = torch.tensor(freq, dtype=torch.float64)
    hi = exact.float()
    inv_freq = torch.stack([hi, (exact - hi.double()).float()]).contiguous().to(DEV)
    n_pages, page = 4, 64
    k_pages = torch.zeros((n_pages, G, page, D), dtype=dtype, device=DEV)
    v_pages = torch.zeros((n_pages, G, page, Dv), dtype=dtype, device=DEV)
    table = i32([2, 0, 3, 1]).view(1, 4)
    state = torch.zeros((2, (taps - 1) * C + 1), device=DEV)
    got = np.zeros((T, H * Dv))
    cuts = {"general": [T], "split": [60, 3, 1, 2, 8, 5], "tensor": [50, 14, 64, 9, 100]}[form] if dtype == torch.bfloat16 else [37, 1, 2, 64, 27, 5]
    for a, b in portions_of(T, cuts):
        n = b - a
        qd = ops.conv_rope_store(f32(proj[a:b])[:, :C], f32(w.T.copy()), state[:, :max((taps - 1) * C, 1)] if taps > 1 else None, i32(range(a, b)), i32([0] * n),
                                 i32([0, n]), i32([1]), table, inv_freq, mag, dims, k_pages, v_pages, H, rt.status)
        out = torch.empty((n, H * Dv), dtype=dtype, device=DEV)
        args = (qd, i32(range(a, b)), i32([0] * n), table, k_pages, v_pages, out, H, scale, 0, rt.status)
        kw = dict(sinks=f32(sink), softcap=softcap or 0.0)
        if form == "general":
            ops.sink_attention(*args, **kw)
        elif form == "split":
            ops.sink_decode(*args, 3 if b > 128 else 1, **kw)
        else:
            tiles_of = lambda tt: torch.tensor([[0, t0, min(tt, n - t0), 0] for t0 in range(0, n, tt)], dtype=torch.int32, device=DEV)
            if D in (64, 128) and Dv == D:
                ops.sink_attention_twin(qd, i32(range(a, b)), tiles_of(ops.prefill_twin_tile_tokens(H, G)), table, k_pages, v_pages, out, H, scale, 0,
                                        rt.status, **kw)
            else:
                ops.sink_attention_mma(qd, i32(range(a, b)), tiles_of(ops.SINK_TILE_TOKENS), table, k_pages, v_pages, out, H, scale, 0, rt.status, **kw)
        got[a:b] = out.float().cpu().numpy()
    rt.check_status()
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    err = np.abs(got - want).max(axis=1)
    assert err.max() < tol * (1 + np.abs(want).max()), f"token {int(err.argmax())}: {err.max():.3g}"


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------

def make_runner(folder, dtype, n_pages, slots=4, **kw):
    from lgml_b200.engine.engine import parse_dtype
    from lgml_b200.engine.runner import ModelRunner

    return ModelRunner.from_folder(folder, parse_dtype(dtype), DEV, n_pages=n_pages, max_slots=slots, max_step_tokens=n_pages * 64, **kw)


def sequences(cfg, lens, seed=50):
    return {f"r{i}": H.random_ids(n, cfg["vocab"], seed + i) for i, n in enumerate(lens)}


# one mechanism at a time: a model of one layer that has as little else as the design allows
ALONE = {
    "no_feed_forward": L.config(53, 40, [L.parallel(L.left(2, 1, 8, 8, 1, 0.4, dims=2), L.right(2, 4, 6, 1, 1, 1))], eps=1e-5),
    "attention_far": L.config(53, 40, [L.parallel(L.left(2, 2, 16, 16, 3, 0.4, base=9000.0, dims=6, scaling=(16.0, 48, 6.0, 0.5), softcap=6.0),
                                                 L.right(1, 4, 4, 1, 2, 1), ff=24)], eps=1e-5, scale=3.0),
    "recurrence_wide": L.config(53, 40, [L.parallel(L.left(1, 1, 8, 8, 2, 0.3, dims=4), L.right(5, 16, 24, 5, 4, 5), ff=24)], eps=1e-5),
    "input_convolution": L.config(53, 40, [L.parallel(L.left(2, 1, 8, 6, 2, 0.3, dims=8), L.right(2, 4, 6, 2, 2, 2), ff=72)], eps=1e-5, taps=5),
    "one_tap_everywhere": L.config(53, 40, [L.parallel(L.left(2, 1, 8, 8, 1, 0.3, dims=4), L.right(2, 4, 6, 1, 1, 2), ff=24)], eps=1e-5, taps=1),
    "odd_width": L.config(51, 35, [L.parallel(L.left(3, 1, 10, 7, 3, 0.3, dims=6, softcap=7.0), L.right(3, 5, 9, 3, 2, 3), ff=33)], eps=1e-5, scale=1.5, taps=2,
                          loop=(0, 1, 2)),
    "loop_of_one": L.config(53, 40, [L.parallel(L.left(2, 1, 8, 8, 2, 0.3, dims=4), L.right(2, 4, 6, 1, 2, 1), ff=24),
                                     L.parallel(L.left(1, 1, 16, 8, 4, 0.3, dims=16, softcap=4.0), L.right(4, 6, 10, 2, 3, 4))], eps=1e-5, taps=2,
                            loop=(1, 2, 4)),
    "loop_from_the_start": L.config(53, 40, [L.parallel(L.left(2, 2, 8, 8, 2, 0.3, dims=4), L.right(2, 4, 6, 1, 2, 1), ff=24)], eps=1e-5, taps=3,
                                    loop=(0, 1, 3)),
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_mechanism_at_a_time(name, tmp_path):
    """Models of one or two layers, in float32: whole, in portions down to two tokens, token by token."""
    cfg = ALONE[name]
    weights = L.random_weights(cfg, seed=21, sharpen=2.0)
    folder = L.write_folder(tmp_path / name, cfg, weights)
    seqs = sequences(cfg, [1, 2, 70, 150], seed=30)
    for trace in (H.trace_whole(seqs), H.trace_portions(seqs), H.trace_tail(seqs, tail=40)):
        runner = make_runner(folder, "float32", n_pages=4)
        L.compare(H.run_trace(runner, trace), cfg, weights, seqs, **TOL["float32"])
    if name == "odd_width":
        # bfloat16 at a width no 16-byte access or tensor-memory copy takes: the products fall to the library, the rest to scalar accesses
        weights = L.random_weights(cfg, seed=21)
        folder = L.write_folder(tmp_path / (name + "_bf16"), cfg, weights)
        runner = make_runner(folder, "bfloat16", n_pages=4)
        L.compare(H.run_trace(runner, H.trace_portions(seqs)), cfg, weights, seqs, **TOL["bfloat16"])


@pytest.fixture(scope="module", params=sorted(L.CONFIGS))
def model(request, tmp_path_factory):
    cfg = L.CONFIGS[request.param]
    made = {}
    # float32 runs see attention sharpened (a wrong key moves the logits far past the tolerance);
    # bfloat16's own rounding of q and k would be amplified alike, so its models are left as drawn
    for dtype, sharpen in (("float32", 2.0), ("bfloat16", 1.0)):
        weights = L.random_weights(cfg, seed=11, sharpen=sharpen)
        made[dtype] = (weights, L.write_folder(tmp_path_factory.mktemp(f"{request.param}_{dtype}"), cfg, weights))
    return request.param, cfg, made


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_cuttings_match_the_plain_model(model, dtype):
    """Whole; the last 32 tokens one by one; portions down to two tokens; and up to three live requests with so few
    pages and slots that both are used again."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [1, 5, 23, 64, 65, 97, 150, 201])
    results = {}
    for kind, trace in (("whole", H.trace_whole(seqs)), ("tail", H.trace_tail(seqs)), ("portions", H.trace_portions(seqs))):
        runner = make_runner(folder, dtype, n_pages=4)
        results[kind] = H.run_trace(runner, trace)
        assert all(g.pool.n_held == 0 for g in runner.cache.groups)
    trace = H.trace_mixed(seqs, max_tokens=64 * 7, seed=5, max_live=3)
    assert max(len(st["entries"]) for st in trace) >= 3
    runner = make_runner(folder, dtype, n_pages=7, slots=3)
    results["mixed"] = H.run_trace(runner, trace)
    assert all(g.pool.taken_total > g.pool.n_pages for g in runner.cache.groups), "no page was used twice"
    for kind, got in results.items():
        worst = L.compare(got, cfg, weights, seqs, **TOL[dtype])
        print(f"{name} {dtype} {kind}: max |diff| {worst:.3g}")
    if dtype == "float32":
        for kind in ("tail", "portions", "mixed"):
            for key, row in results["whole"].items():
                assert float((row - results[kind][key]).abs().max()) < 2e-5 * (1.0 + float(row.abs().max())), f"float32 {kind} differs from whole at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_then_long_decoding(model, dtype):
    """Three tokens of prompt, then 230 tokens one by one (through captured steps): the states are carried 230 times,
    every convolution starts inside its first taps, and the keys cross three pages."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [233], seed=70)
    runner = make_runner(folder, dtype, n_pages=4)
    got = H.run_trace(runner, H.trace_tail(seqs, tail=230))
    assert runner.graph_replays > 100
    L.compare(got, cfg, weights, seqs, **TOL[dtype])


def test_a_slot_that_is_used_again_starts_from_nothing(model):
    name, cfg, made = model
    weights, folder = made["float32"]
    seqs = sequences(cfg, [130, 75], seed=90)
    fresh = make_runner(folder, "float32", n_pages=3, slots=1)
    want = H.run_trace(fresh, H.trace_portions({"r1": seqs["r1"]}))
    used = make_runner(folder, "float32", n_pages=3, slots=1)
    H.run_trace(used, H.trace_portions({"r0": seqs["r0"]}))
    got = H.run_trace(used, H.trace_portions({"r1": seqs["r1"]}))
    for key, row in want.items():
        assert torch.equal(row, got[key]), f"position {key[1]} differs after the slot was used before"
    L.compare(got, cfg, weights, {"r1": seqs["r1"]}, **TOL["float32"])


def test_batch_of_unequal_requests_equals_each_alone(model):
    name, cfg, made = model
    weights, folder = made["float32"]
    seqs = sequences(cfg, [90, 3, 41, 1], seed=120)
    runner = make_runner(folder, "float32", n_pages=8)
    alone = H.run_trace(runner, H.trace_whole(seqs))
    together = H.run_trace(runner, [{"step": 0, "entries": [{"id": r, "tokens": ids, "want": list(range(len(ids)))} for r, ids in seqs.items()],
                                     "end": list(seqs)}])
    for key, row in alone.items():
        assert torch.equal(row, together[key])
    L.compare(together, cfg, weights, seqs, **TOL["float32"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_tokens_in_a_step_beside_decoded_ones(model, dtype):
    """A portion of 290 tokens beside a decoded token (attention on tensor cores where the sizes allow, in bfloat16);
    then the same request goes on token by token from the states and pages that step left."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [320, 80], seed=140)
    runner = make_runner(folder, dtype, n_pages=16)
    a, b = runner.open("r0"), runner.open("r1")
    got = {}
    rows = runner.step([(b, seqs["r1"][:70], [69])]).float().cpu()
    got[("r1", 69)] = rows[0]
    rows = runner.step([(a, seqs["r0"][:290], list(range(0, 290, 7))), (b, seqs["r1"][70:71], [0])]).float().cpu()
    for i, p in enumerate(range(0, 290, 7)):
        got[("r0", p)] = rows[i]
    got[("r1", 70)] = rows[-1]
    for p in range(290, 320):
        q = 71 + p - 290
        entries = [(a, [seqs["r0"][p]], [0])] + ([(b, [seqs["r1"][q]], [0])] if q < 80 else [])
        rows = runner.step(entries).float().cpu()
        got[("r0", p)] = rows[0]
        if len(entries) > 1:
            got[("r1", q)] = rows[1]
    runner.rt.check_status()
    L.compare(got, cfg, weights, seqs, **TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(model, dtype):
    """Engine.generate (scheduler, portions of 16 prompt tokens, sampling on the device, steps run ahead) and
    Engine.greedy against greedy decoding with the plain model."""
    import lgml_b200

    name, cfg, made = model
    weights, folder = made[dtype]
    prompts = [H.random_ids(n, cfg["vocab"], 200 + n) for n in (37, 5, 70)]
    eng = lgml_b200.Engine(str(folder), dtype=dtype, n_ctx=256, slots=2, ubatch=16)
    outs = eng.generate(prompts, max_tokens=10, temperature=0.0, stop=[])
    solo, _ = eng.greedy(prompts[0], 10)
    for prompt, got in zip(prompts, outs):
        assert len(got) == 10
        for i, tok in enumerate(got):
            row = L.oracle_logits(cfg, weights, prompt + got[:i])[-1]
            gap = float(row.max() - row[tok])
            bound = 0.0 if dtype == "float32" and gap > 1e-4 else (1e-4 if dtype == "float32" else 5e-2 * float(row.abs().max()))
            assert gap <= bound, f"{dtype}: token {i} is {tok}, the plain model prefers {int(row.argmax())} by {gap:.3g}"
    if dtype == "float32":
        assert solo == outs[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_process(model, tmp_path, dtype):
    """bin/trace_run as a process on a mixed trace with two live requests and four pages."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [70, 20, 131], seed=310)
    trace = H.trace_mixed(seqs, max_tokens=64 * 4, seed=2, max_live=2)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                           "--max-tokens", str(64 * 4)], input="\n".join(json.dumps(s) for s in trace) + "\n", text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")]
    assert done == [f"done {s['step']}" for s in trace]
    got, fed = {}, {r: 0 for r in seqs}
    for st in trace:
        if not any(e["want"] for e in st["entries"]):
            continue
        rows = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        r = 0
        for e in st["entries"]:
            for i in e["want"]:
                got[(e["id"], fed[e["id"]] + i)] = torch.from_numpy(rows[r].copy())
                r += 1
        assert r == rows.shape[0]
        for e in st["entries"]:
            fed[e["id"]] += len(e["tokens"])
    # (steps without wanted rows still advance their requests)
    got2, fed = {}, {r: 0 for r in seqs}
    for st in trace:
        rows = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"]) if any(e["want"] for e in st["entries"]) else None
        r = 0
        for e in st["entries"]:
            for i in e["want"]:
                got2[(e["id"], fed[e["id"]] + i)] = torch.from_numpy(rows[r].copy())
                r += 1
            fed[e["id"]] += len(e["tokens"])
    L.compare(got2, cfg, weights, seqs, **TOL[dtype])


def test_command_line_generates_with_the_folders_architecture(model):
    name, cfg, made = model
    weights, folder = made["float32"]
    prompt = H.random_ids(19, cfg["vocab"], 400)
    proc = subprocess.run([sys.executable, "-m", "lgml_b200", "-m", str(folder), "--dtype", "float32", "-c", "128", "--prompt-ids", ",".join(map(str, prompt)),
                           "-n", "5", "--temperature", "0", "--repeat-stop", "0"], capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(t) for t in proc.stdout.strip().splitlines()[-1].split(",")]
    assert len(got) == 5
    for i, tok in enumerate(got):
        row = L.oracle_logits(cfg, weights, prompt + got[:i])[-1]
        assert float(row.max() - row[tok]) <= 1e-4


def test_random_weights_mode_runs_the_design():
    """A configuration alone is enough: the engine draws weights of the shapes and kinds the parts ask for."""
    from lgml_b200.config import config_from_dict
    from lgml_b200.engine.runner import ModelRunner

    runner = ModelRunner.from_config(config_from_dict(L.TAIL_LOOP), seed=3, dtype=torch.bfloat16, n_pages=4, max_slots=2)
    req = runner.open("a")
    rows = runner.step([(req, H.random_ids(70, 83, 1), [0, 69])])
    runner.rt.check_status()
    assert rows.shape == (2, 83) and bool(torch.isfinite(rows).all())
