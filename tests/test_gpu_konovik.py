"""Konovik in the engine against the plain implementation: every mechanism alone, then whole models
under every way of cutting the work.

The models are small and differ from each other in every size and option (recurrences narrower and
wider than the model, one to five heads, windows of 1 to 100 and none, stretched and plain rotary
frequencies, loops at the start, in the middle and at the end, one to eight experts with one to all
of them chosen, with and without a shared expert, with and without per-layer token inputs, layers
without a feed-forward).  Where random numbers would hide a fault, the inputs are made so that it
shows: the keys at a window's edge carry the largest scores, the recurrence's gates are nearly shut
so that a state from hundreds of tokens back still decides the output.
"""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests import konovik_helpers as L
from tests.plain import konovik_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent
F64 = torch.float64
TOL = {"float32": dict(atol=3e-5, rtol=2e-4), "bfloat16": dict(atol=3e-2, rtol=8e-2)}


def bf(t):
    return t.to(torch.bfloat16).double()


def i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def batch_of(lens):
    """(request index of every token, first token row of every request) of a step with these portions."""
    seq_of = [r for r, n in enumerate(lens) for _ in range(n)]
    starts = np.concatenate([[0], np.cumsum(lens)])
    return i32(seq_of), i32(starts)


def portions_of(total, cuts):
    """[(a, b)] covering 0 .. total with the sizes ``cuts`` in turn."""
    out, a, i = [], 0, 0
    while a < total:
        b = min(total, a + cuts[i % len(cuts)])
        out.append((a, b))
        a, i = b, i + 1
    return out


# ---------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [36, 64, 321])
def test_norm_with_one_weight(dtype, W):
    """x over its root mean square times ONE number, with the residual sum ahead of it and a float32 result."""
    from lgml_b200 import ops

    torch.manual_seed(1)
    x = torch.randn(70, W, dtype=F64) * 3.0
    d = torch.randn(70, W, dtype=F64)
    g, eps, m = 1.3125, 1e-5, 0.3
    want = torch.from_numpy(P.scalar_norm((x + m * d).numpy(), g, eps))
    from lgml_b200.parts import make_part

    xd, dd = x.float().to(DEV), d.float().to(DEV)
    norm = make_part("norm", "rmsnorm", width=W, eps=eps, suffix="", single=True)
    assert [tuple(s.shape) for s in norm.tensor_specs("n")] == [()]
    norm.bind("n", {"n": torch.tensor(g, dtype=torch.float32, device=DEV)}, None)
    out = norm.forward(None, xd, dtype, delta=dd, delta_scale=m)
    tol = 3e-6 if dtype == torch.float32 else 2e-2
    assert float((out.double().cpu() - want).abs().max()) < tol * (1.0 + float(want.abs().max()))
    assert float((xd.double().cpu() - (x.float().double() + m * d.float().double())).abs().max()) < 1e-5, "the sum was not left in the stream"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [20, 64, 130])
def test_token_shift_carries_the_last_row_between_steps(dtype, W):
    """Three requests of unequal length in steps of unequal portions (one of them left out of a step), slots in
    another order than the requests: every row but a request's very first mixes with the row before it, whichever
    step that row came in."""
    from lgml_b200 import ops

    torch.manual_seed(2)
    lens = {"a": 41, "b": 7, "c": 1}
    h = {r: torch.randn(n, W, dtype=F64).float().double() for r, n in lens.items()}
    mu = torch.rand(W, dtype=F64).float().double()
    mu[0], mu[1] = 0.0, 1.0
    want = {r: torch.from_numpy(P.token_shift(t.numpy(), mu.numpy())) for r, t in h.items()}
    slot = {"a": 2, "b": 0, "c": 3}
    state = torch.full((5, W + 3), 7.0, dtype=torch.float32, device=DEV)       # rows wider than the part's
    state[:, :W] = 0.0
    steps = [{"a": (0, 5), "b": (0, 2)}, {"a": (5, 6), "c": (0, 1)}, {"b": (2, 7), "a": (6, 40)}, {"a": (40, 41)}]
    got = {r: torch.zeros(n, W, dtype=F64) for r, n in lens.items()}
    for st in steps:
        rows = torch.cat([h[r][a:b] for r, (a, b) in st.items()]).float().to(DEV)
        seq_of, starts = batch_of([b - a for a, b in st.values()])
        out = torch.empty(rows.shape, dtype=dtype, device=DEV)
        ops.token_shift(rows, mu.float().to(DEV), state[:, :W], seq_of, starts, i32(slot[r] for r in st), out)
        at = 0
        for r, (a, b) in st.items():
            got[r][a:b] = out[at:at + b - a].double().cpu()
            at += b - a
    tol = 1e-6 if dtype == torch.float32 else 2e-2
    for r in lens:
        assert float((got[r] - want[r]).abs().max()) < tol * (1.0 + float(want[r].abs().max())), r
    assert float(state[:, W:].min()) == 7.0 and float(state[1, :W].abs().max()) == 0.0, "the kernel wrote outside its rows"
    assert torch.equal(state[2, :W].cpu().double(), h["a"][-1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,E", [(24, 16), (64, 40), (321, 32)])
def test_mingru_in_sequence_and_in_pieces_with_gates_nearly_shut(dtype, W, E):
    """The recurrence over two requests, in one step and in steps of 2 to 300 tokens, token by token at the end,
    both as one scan and in pieces side by side.  Half of the channels have gates near 0.002: their state at token 600
    still holds most of what the first tokens wrote, so a state that is lost or reset at any cut shows."""
    from lgml_b200 import ops

    torch.manual_seed(3)
    T = {"a": 700, "b": 130}
    Wm = {"m.z": bf(torch.randn(W, E, dtype=F64) * 0.4), "m.z.b": bf(torch.randn(W, dtype=F64)), "m.x": bf(torch.randn(W, E, dtype=F64)),
          "m.x.b": bf(torch.randn(W, dtype=F64) * 0.5), "m.g": bf(torch.randn(W, E, dtype=F64) * 0.5), "m.o": torch.eye(W, dtype=F64)}
    Wm["m.z.b"][: W // 2] = -6.25
    Wm["m.z"][: W // 2] *= 0.125
    h = {r: bf(torch.randn(n, E, dtype=F64)) for r, n in T.items()}
    npW = {n: t.numpy() for n, t in Wm.items()}
    want = {r: torch.from_numpy(P.min_gru(t.numpy(), npW, "m")) for r, t in h.items()}
    w_in = torch.cat([Wm["m.z"], Wm["m.x"], Wm["m.g"]])
    b_in = torch.cat([Wm["m.z.b"], Wm["m.x.b"], torch.zeros(W, dtype=F64)])
    piece = ops.mingru_chunk_tokens()

    def run(cuts, in_pieces):
        state = torch.zeros(4, W, dtype=torch.float32, device=DEV)
        got = {r: torch.zeros(n, W, dtype=F64) for r, n in T.items()}
        todo = {r: portions_of(n, cuts[r]) for r, n in T.items()}
        while any(todo.values()):
            st = {r: p.pop(0) for r, p in todo.items() if p}
            proj = torch.cat([(h[r][a:b] @ w_in.T + b_in) for r, (a, b) in st.items()]).float().to(DEV).contiguous()
            lens = [b - a for a, b in st.values()]
            _, starts = batch_of(lens)
            out = torch.empty(proj.shape[0], W, dtype=dtype, device=DEV)
            chunks = first = None
            if in_pieces:
                rows, firsts, at = [], [0], 0
                for n in lens:
                    rows += [(at + t0, at + min(t0 + piece, n)) for t0 in range(0, n, piece)]
                    firsts.append(len(rows))
                    at += n
                chunks, first = torch.tensor(rows, dtype=torch.int32, device=DEV), i32(firsts)
            ops.mingru_scan(proj, state, starts, i32({"a": 3, "b": 1}[r] for r in st), out, chunks, first)
            at = 0
            for r, (a, b) in st.items():
                got[r][a:b] = out[at:at + b - a].double().cpu()
                at += b - a
        return got

    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for cuts in ({"a": [700], "b": [130]}, {"a": [300, 2, 129, 64, 1, 1, 1, 200, 1, 1], "b": [2, 100, 1]}, {"a": [1, 699], "b": [129, 1]}):
        for in_pieces in (False, True):
            got = run(cuts, in_pieces)
            for r in T:
                err = (got[r] - want[r]).abs().max(dim=1).values
                bad = torch.nonzero(err > tol * (1.0 + float(want[r].abs().max())))
                assert bad.numel() == 0, f"request {r}, cuts {cuts[r]}, pieces {in_pieces}: first wrong token {int(bad[0])}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,dim,cols,col0", [(36, 5, 20, 10), (64, 12, 36, 24), (136, 24, 24, 0), (48, 1, 3, 2), (264, 64, 131, 67), (72, 264, 272, 8),
                                            (520, 8, 40, 16)])
@pytest.mark.parametrize("n", [70, 3, 25, 150])
def test_token_input_in_one_kernel_and_as_products(dtype, E, dim, cols, col0, n):
    """x += m delta; x += m rms_unit(W_proj (gelu_tanh(W_gate x) * table[token, col0 : col0 + dim])) * w, in the form
    for few tokens (one kernel, the fewer the tokens the more blocks share one) and in the form for many (two
    products with small kernels between)."""
    from lgml_b200 import ops

    torch.manual_seed(4)
    vocab, m, eps = 33, 0.4, 1e-5
    x = (torch.randn(n, E, dtype=F64) * 2.0).float().double()
    delta = torch.randn(n, E, dtype=F64).float().double()
    ids = torch.randint(0, vocab, (n,))
    ids[0], ids[1] = 0, vocab - 1
    W = {"s.gate": bf(torch.randn(dim, E, dtype=F64) * 0.3), "s.proj": bf(torch.randn(E, dim, dtype=F64)), "s.norm": bf(1.0 + 0.3 * torch.randn(E, dtype=F64))}
    table = bf(torch.randn(vocab, cols, dtype=F64))
    x1 = x + m * delta
    want = x1 + m * torch.from_numpy(P.side_input(x1.numpy(), {k: t.numpy() for k, t in W.items()}, "s", table[ids, col0:col0 + dim].numpy(), eps))
    dev = lambda t, ty=dtype: t.to(ty).to(DEV).contiguous()
    tol = (1e-5 if dtype == torch.float32 else 4e-2) * (1.0 + float(want.abs().max()))
    # rows whose y all but vanishes before it is divided by its root mean square are a unit vector made of rounding
    # (with one number per token: a sign); bfloat16 is compared on the others
    sizes = []
    P.side_input(x1.numpy(), {k: t.numpy() for k, t in W.items()}, "s", table[ids, col0:col0 + dim].numpy(), eps, sizes)
    sound = torch.from_numpy(sizes[0] >= (0.0 if dtype == torch.float32 else 0.1) * np.median(sizes[0]))
    assert int(sound.sum()) >= (n + 1) // 2
    want = want[sound]
    # one kernel
    xd = dev(x, torch.float32)
    ops.token_side(xd, dev(delta, torch.float32), m, ids.to(torch.int32).to(DEV), dev(table), col0, dev(W["s.gate"]), dev(W["s.proj"]),
                   dev(W["s.norm"], torch.float32), eps, m)
    assert float((xd.double().cpu()[sound] - want).abs().max()) < tol
    # two products
    xd = dev(x, torch.float32)
    xb = ops.residual_fold(xd, dev(delta, torch.float32), m, copy_dtype=dtype if dtype != torch.float32 else None)
    assert float((xd.double().cpu() - x1).abs().max()) < 1e-5
    gate = ((xd if xb is None else xb).float() @ dev(W["s.gate"], torch.float32).T).contiguous()
    g = ops.side_gate(gate, ids.to(torch.int32).to(DEV), dev(table), col0, dtype)
    y = (g.float() @ dev(W["s.proj"], torch.float32).T).contiguous()
    ops.side_add(xd, y, dev(W["s.norm"], torch.float32), eps, m)
    assert float((xd.double().cpu()[sound] - want).abs().max()) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("X,top,E,F,Fs,scale", [(5, 2, 64, 24, 40, 1.5), (1, 1, 36, 20, 0, 0.7), (4, 4, 40, 12, 8, 1.0), (16, 3, 96, 40, 56, 2.0),
                                                (40, 6, 128, 64, 0, 2.5), (3, 2, 256, 520, 264, 1.0)])
def test_sigmoid_router_with_a_correction_and_experts_without_a_gate(dtype, X, top, E, F, Fs, scale):
    """The correction decides which experts are chosen but not their weights (it is made large: most choices differ
    from those of the scores alone); the weights are the chosen scores over their sum, times the scale; the experts
    square a relu; a shared expert joins behind its own sigmoid.  300 tokens (the grouped form) and 2 (a block a row)."""
    from lgml_b200 import ops

    torch.manual_seed(8)
    T = 300
    W = {"f.router": bf(torch.randn(X, E, dtype=F64) * 0.3), "f.correction": bf(torch.randn(X, dtype=F64) * 0.5)}
    for e in range(X):
        W[f"f.e{e}.up"], W[f"f.e{e}.down"] = bf(torch.randn(F, E, dtype=F64) * 0.3), bf(torch.randn(E, F, dtype=F64) * 0.3)
    f = {"router": {"experts": X, "top": top, "scale": scale}}
    if Fs:
        f["shared"] = {"ff": Fs}
        W["f.shared.up"], W["f.shared.down"], W["f.shared.sg"] = (bf(torch.randn(Fs, E, dtype=F64) * 0.3), bf(torch.randn(E, Fs, dtype=F64) * 0.3),
                                                                bf(torch.randn(1, E, dtype=F64) * 0.3))
    h = bf(torch.randn(T, E, dtype=F64))
    npW = {n: t.numpy() for n, t in W.items()}
    want = torch.from_numpy(P.routed_ff(h.numpy(), npW, "f", f))
    hd = h.to(dtype).to(DEV)
    w_router = torch.cat([W["f.router"]] + ([W["f.shared.sg"]] if Fs else [])).float().to(DEV).contiguous()
    res = ops.moe_router(hd, w_router, W["f.correction"].float().to(DEV), top, "sigmoid", scale, n_extra=1 if Fs else 0)
    ids, wts = res[0], res[1]
    s = torch.sigmoid(h @ W["f.router"].T)
    chosen = torch.argsort(-(s + W["f.correction"]), dim=1, stable=True)[:, :top]
    assert torch.equal(ids.cpu().long(), chosen)
    if top < X:
        assert not torch.equal(chosen, torch.argsort(-s, dim=1, stable=True)[:, :top]), "the correction changes nothing here"
    picked = torch.gather(s, 1, chosen)
    assert float((wts.double().cpu() - picked / (picked.sum(1, keepdim=True) + 1e-20) * scale).abs().max()) < 1e-5
    also = also_w = None
    if Fs:
        also_w = res[2].reshape(-1).contiguous()
        assert float((also_w.double().cpu() - torch.sigmoid(h @ W["f.shared.sg"].T).reshape(-1)).abs().max()) < 1e-5
        also = torch.from_numpy(P.relu2_expert(h.numpy(), npW, "f.shared")).float().to(DEV).contiguous()
    w_up = torch.stack([W[f"f.e{e}.up"] for e in range(X)]).to(dtype).to(DEV)
    w_down = torch.stack([W[f"f.e{e}.down"] for e in range(X)]).to(dtype).to(DEV)
    tol = (3e-5 if dtype == torch.float32 else 2e-2) * (1.0 + float(want.abs().max()))
    out = ops.moe_experts_rows(hd, ids, wts, w_up, w_down, gated=False, also=also, also_w=also_w)
    assert float((out.double().cpu() - want).abs().max()) < tol
    two = ops.moe_experts_rows(hd[:2], ids[:2].contiguous(), wts[:2].contiguous(), w_up, w_down, gated=False,
                               also=None if also is None else also[:2].contiguous(), also_w=None if also is None else also_w[:2].contiguous())
    assert float((two.double().cpu() - want[:2]).abs().max()) < tol
    if dtype == torch.bfloat16 and ops.moe_grouped_supports(hd, w_up, False):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out3 = ops.moe_experts_tcgen05(hd, ids, wts, w_up, w_down, status, gated=False, also=also, also_w=also_w)
        assert int(status.item()) == 0
        assert float((out3.double().cpu() - want).abs().max()) < tol
    # equal choice scores go to the lower index, and equal scores share the scale equally
    tie = ops.moe_router(torch.zeros(3, E, dtype=dtype, device=DEV), W["f.router"].float().to(DEV).contiguous(), None, top, "sigmoid", scale)
    assert torch.equal(tie[0].cpu(), torch.arange(top, dtype=torch.int32).expand(3, top))
    assert float((tie[1] - scale / top).abs().max()) < 1e-6


def latent_pages(T, width, dtype, seed):
    """Empty cells for one request of T tokens behind a shuffled block table."""
    n_blocks = -(-T // 64)
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_blocks + 3, generator=g)[:n_blocks]
    cells = torch.zeros(n_blocks + 3, 1, 64, width, dtype=dtype, device=DEV)
    return cells, order.to(torch.int32).view(1, -1).contiguous().to(DEV)


@pytest.mark.parametrize("dtype,form", [(torch.float32, "general"), (torch.bfloat16, "general"), (torch.bfloat16, "split"), (torch.bfloat16, "mma")])
@pytest.mark.parametrize("window", [None, 1, 2, 40, 64, 65, 129])
@pytest.mark.parametrize("shape", [(3, 16, 8, 12, 24, 8, None), (1, 12, 2, 20, 10, 2, (4.0, 16, 2.0, 0.5)), (2, 24, 12, 20, 40, 8, (8.0, 64, 8.0, 1.0)),
                                   (4, 32, 32, 32, 96, 32, (2.0, 32, 4.0, 1.0))])
def test_latent_attention_at_the_windows_edge(dtype, form, window, shape):
    """The latent's norm, the rotation (plain and stretched frequencies, fewer rotated pairs than the rotated part
    holds), both products per head, the window, the output gate.  The rotated key part is not normed, so the rows of h
    at some positions are scaled up: those keys carry the largest scores, and a query that sees one key more or less
    than its window holds gets another result.  Whole and in portions that end inside, at and past pages."""
    from lgml_b200 import ops
    from lgml_b200.parts.latent_attention import scaled_frequencies

    Hh, D, Dr, Dv, R, dims, scaling = shape
    torch.manual_seed(5)
    E, T, scale, eps = 48, 200, 0.3, 1e-5
    rot = {"base": 1000.0, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": Hh, "dim": D, "rot_dim": Dr, "vdim": Dv, "kv_rank": R, "scale": scale, "rot": rot}
    if window:
        m["mask"] = {"size": window}
    W = {"x.q": bf(torch.randn(Hh * (D + Dr), E, dtype=F64) * 0.15), "x.dkv": bf(torch.randn(R + Dr, E, dtype=F64) * 0.3),
         "x.dkv.norm": bf(1.0 + 0.2 * torch.randn(R, dtype=F64)), "x.uk": bf(torch.randn(Hh * D, R, dtype=F64) * 0.3),
         "x.uv": bf(torch.randn(Hh * Dv, R, dtype=F64) * 0.3), "x.g": bf(torch.randn(Hh * Dv, E, dtype=F64) * 0.3), "x.o": torch.eye(Hh * Dv, dtype=F64)}
    h = torch.randn(T, E, dtype=F64)
    loud = [0, 3, 50, 63, 64, 100, 127, 128, 150]
    h[loud] *= 5.0 if dtype == torch.float32 else 2.0
    h = bf(h)
    want = torch.from_numpy(P.latent_attention(h.numpy(), {n: t.numpy() for n, t in W.items()}, "x", m, eps))
    tol = 3e-5 if dtype == torch.float32 else 2e-2 * (1.0 + float(want.abs().max()))
    if window and window > 1:
        for size in (window + 1, window - 1):
            other = torch.from_numpy(P.latent_attention(h.numpy(), {n: t.numpy() for n, t in W.items()}, "x", dict(m, mask={"size": size}), eps))
            assert float((other - want).abs().max()) > 1.5 * tol, "a window of %d keys instead of %d would not show" % (size, window)
    freq, mag = scaled_frequencies(rot["base"], dims, rot.get("scaling"))
    exact = torch.tensor(freq, dtype=F64)
    inv_freq = torch.stack([exact.float(), (exact - exact.float().double()).float()]).contiguous().to(DEV)

    def chain(portions):
        cells, table = latent_pages(T, R + Dr, dtype, seed=2)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        outs = []
        for a, b in portions:
            n = b - a
            positions = torch.arange(a, b, dtype=torch.int32, device=DEV)
            seq = torch.zeros(n, dtype=torch.int32, device=DEV)
            hp = h[a:b].float().to(DEV)
            qp = (hp @ W["x.q"].float().to(DEV).T).contiguous()
            dk = (hp @ W["x.dkv"].float().to(DEV).T).contiguous()
            gate = (hp @ W["x.g"].float().to(DEV).T).contiguous()
            q_plain, q_full = ops.latent_prepare(qp, dk, W["x.dkv.norm"].float().to(DEV), eps, inv_freq, dims, positions, seq, table, cells, Hh, D,
                                                 Dr, R, status, rot_mag=mag)
            ops.head_linear(q_plain, W["x.uk"].view(Hh, D, R).transpose(1, 2).contiguous().to(dtype).to(DEV), q_full, D, R + Dr)
            mix = torch.empty(n, Hh * R, dtype=dtype, device=DEV)
            if form == "split":
                ops.sink_decode(q_full, positions, seq, table, cells, cells[..., :R], mix, Hh, scale, window or 0, status, 3)
            elif form == "mma":
                tiles = torch.tensor([[0, r0, min(64, n - r0), 0] for r0 in range(0, n, 64)], dtype=torch.int32, device=DEV)
                ops.sink_attention_mma(q_full, positions, tiles, table, cells, cells[..., :R], mix, Hh, scale, window or 0, status)
            else:
                ops.sink_attention(q_full, positions, seq, table, cells, cells[..., :R], mix, Hh, scale, window or 0, status)
            o = torch.empty(n, Hh * Dv, dtype=dtype, device=DEV)
            ops.head_linear(mix, W["x.uv"].view(Hh, Dv, R).contiguous().to(dtype).to(DEV), o, R, Dv, gate=gate)
            outs.append(o.double().cpu())
        assert int(status.item()) == 0
        return torch.cat(outs)

    for portions in ([(0, T)], [(0, 3), (3, 5), (5, 64), (64, 130), (130, 131), (131, T)]):
        err = (chain(portions) - want).abs().max(dim=1).values
        bad = torch.nonzero(err > tol)
        assert bad.numel() == 0, f"portions {portions}: first wrong position {int(bad[0])} (|diff| {float(err[int(bad[0])]):.3g})"


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------

def make_runner(folder, dtype, n_pages, slots=4, **kw):
    from lgml_b200.engine.engine import parse_dtype
    from lgml_b200.engine.runner import ModelRunner

    return ModelRunner.from_folder(folder, parse_dtype(dtype), DEV, n_pages=n_pages, max_slots=slots, max_step_tokens=n_pages * 64, **kw)


def sequences(cfg, lens, seed=50, weights=None):
    """Random requests; with ``weights`` (the bfloat16 runs) such that no router decides by a close call."""
    if weights is not None:
        return {f"r{i}": L.clear_ids(cfg, weights, n, seed + i) for i, n in enumerate(lens)}
    return {f"r{i}": H.random_ids(n, cfg["vocab"], seed + i) for i, n in enumerate(lens)}


# one mechanism at a time: a model of one layer that has nothing else
ALONE = {
    "recurrence": L.config(53, 40, [L.mingru(56)], eps=1e-5),
    "recurrence_scaled": L.config(53, 40, [L.mingru(24)], eps=1e-5, mult=0.25),
    "latent_window": L.config(53, 40, [L.latent(3, 8, 4, 12, 20, scale=0.4, base=100.0, window=7)], eps=1e-5),
    "latent_far": L.config(53, 40, [L.latent(2, 16, 8, 8, 24, scale=0.4, base=9000.0, dims=6, scaling=(16.0, 48, 6.0, 0.5))], eps=1e-5),
    "dense": L.config(53, 40, [L.mingru(8, mlp=L.dense(72))], eps=1e-5, mult=2.0),
    "experts": L.config(53, 40, [L.mingru(8, mlp=L.moe(20, 7, 3, scale=3.0))], eps=1e-5),
    "experts_shared": L.config(53, 40, [L.mingru(8, mlp=L.moe(12, 2, 1, shared=28))], eps=1e-5, mult=0.6),
    "token_input": L.config(53, 40, [L.mingru(8), L.mingru(8)], eps=1e-5, mult=0.8, side=9),
    "loop_of_one": L.config(53, 40, [L.mingru(16, mlp=L.dense(24)), L.latent(2, 8, 4, 8, 12, scale=0.3, window=33)], eps=1e-5, mult=0.5, side=4,
                            loop=(1, 2, 4)),
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_mechanism_at_a_time(name, tmp_path):
    """Models of one layer, in float32: whole, in portions down to two tokens, token by token."""
    cfg = ALONE[name]
    weights = L.random_weights(cfg, seed=21, sharpen=2.0)
    folder = L.write_folder(tmp_path / name, cfg, weights)
    seqs = sequences(cfg, [1, 2, 70, 150], seed=30)
    for trace in (H.trace_whole(seqs), H.trace_portions(seqs), H.trace_tail(seqs, tail=40)):
        runner = make_runner(folder, "float32", n_pages=4)
        L.compare(H.run_trace(runner, trace), cfg, weights, seqs, **TOL["float32"])


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
    """Whole; the last 32 tokens one by one; portions down to two tokens; and up to three live requests
    with so few pages and slots that both are used again."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [1, 5, 23, 64, 65, 97, 150, 201], weights=weights if dtype == "bfloat16" else None)
    results = {}
    for kind, trace in (("whole", H.trace_whole(seqs)), ("tail", H.trace_tail(seqs)), ("portions", H.trace_portions(seqs))):
        runner = make_runner(folder, dtype, n_pages=4)
        results[kind] = H.run_trace(runner, trace)
        assert all(g.pool.n_held == 0 for g in runner.cache.groups)
    trace = H.trace_mixed(seqs, max_tokens=64 * 7, seed=5, max_live=3)
    assert max(len(st["entries"]) for st in trace) >= 3
    runner = make_runner(folder, dtype, n_pages=7, slots=3)
    results["mixed"] = H.run_trace(runner, trace)
    assert all(g.pool.taken_total > g.pool.n_pages for g in runner.cache.groups if g.spec.window is None), "no page was used twice"
    from lgml_b200.parts.mingru import MINGRU_PIECES_FROM

    for kind, got in results.items():
        worst = L.compare(got, cfg, weights, seqs, **TOL[dtype])
        print(f"{name} {dtype} {kind}: max |diff| {worst:.3g}")
    if dtype == "float32":
        # short portions run the recurrence as one scan, in whichever step they come: bit-equal.  A longer
        # portion runs it in pieces (a piece's start is a product of the pieces before it), which rounds differently.
        for key, row in results["tail"].items():
            if len(seqs[key[0]]) - 32 <= MINGRU_PIECES_FROM:
                assert torch.equal(row, results["portions"][key]), f"float32 portions differ from tail at {key}"
        for kind in ("tail", "portions", "mixed"):
            for key, row in results["whole"].items():
                assert float((row - results[kind][key]).abs().max()) < 2e-5 * (1.0 + float(row.abs().max())), f"float32 {kind} differs from whole at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_then_long_decoding_over_every_window(model, dtype):
    """Three tokens of prompt, then 230 tokens one by one (through captured steps): every window of the
    models (1 to 100) passes over decoded tokens, and the recurrent states are carried 230 times."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [233], seed=70, weights=weights if dtype == "bfloat16" else None)
    runner = make_runner(folder, dtype, n_pages=4)
    got = H.run_trace(runner, H.trace_tail(seqs, tail=230))
    assert runner.graph_replays > 100
    L.compare(got, cfg, weights, seqs, **TOL[dtype])


def test_a_slot_that_is_used_again_starts_from_nothing(model):
    """A request that ends leaves its recurrent states, its last rows and its pages behind; the next request that
    gets the same slot and pages computes what it computes on an engine that never saw another."""
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


def test_a_window_gives_its_pages_back(model):
    name, cfg, made = model
    weights, folder = made["float32"]
    runner = make_runner(folder, "float32", n_pages=12)
    seqs = sequences(cfg, [700], seed=75)
    req = runner.open("a")
    ids = seqs["r0"]
    for a in range(0, 700, 50):
        runner.step([(req, ids[a:a + 50], [])])
    for g, table in zip(runner.cache.groups, req.tables):
        if g.spec.window is None:
            assert all(p >= 0 for p in table)
            continue
        first = max(0, 700 - g.spec.window + 1) // 64
        assert all(p < 0 for p in table[:first]) and all(p >= 0 for p in table[first:])
    row = runner.step([(req, [ids[0]], [0])])
    want = L.oracle_logits(cfg, weights, ids + [ids[0]])[-1]
    assert float((row[0].double().cpu() - want).abs().max()) < 3e-5 + 2e-4 * float(want.abs().max())
    runner.close(req)
    runner.cache.check()


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
    """A portion of 290 tokens beside a decoded token: the recurrence runs in pieces side by side, the token input as
    products, the experts in the grouped form and attention on tensor cores where the sizes allow (bfloat16); then the
    same request goes on token by token from the states and pages that step left."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [320, 80], seed=140, weights=weights if dtype == "bfloat16" else None)
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
    """Engine.generate (scheduler, portions of 16 prompt tokens, sampling on the device, steps run ahead)
    and Engine.greedy against greedy decoding with the plain model."""
    import lgml_b200

    name, cfg, made = model
    weights, folder = made[dtype]
    prompts = [L.clear_ids(cfg, weights, n, 200 + n) if dtype == "bfloat16" else H.random_ids(n, cfg["vocab"], 200 + n) for n in (37, 5, 70)]
    eng = lgml_b200.Engine(str(folder), dtype=dtype, n_ctx=256, slots=2, ubatch=16)
    outs = eng.generate(prompts, max_tokens=10, temperature=0.0, stop=[])
    solo, _ = eng.greedy(prompts[0], 10)
    for prompt, got in zip(prompts, outs):
        assert len(got) == 10
        checked = 0
        for i, tok in enumerate(got):
            if dtype == "bfloat16":
                # a generated token may bring a close call between two experts, which bfloat16 may decide the other way: stop there
                gaps = []
                P.forward(cfg, L.numpy_of(weights), prompt + got[:i], router_gaps=gaps)
                if gaps and float(np.min(np.stack(gaps))) < 0.02:
                    break
            row = L.oracle_logits(cfg, weights, prompt + got[:i])[-1]
            gap = float(row.max() - row[tok])
            bound = 0.0 if dtype == "float32" and gap > 1e-4 else (1e-4 if dtype == "float32" else 5e-2 * float(row.abs().max()))
            assert gap <= bound, f"{dtype}: token {i} is {tok}, the plain model prefers {int(row.argmax())} by {gap:.3g}"
            checked += 1
        assert checked >= 1
    if dtype == "float32":
        assert solo == outs[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_process(model, tmp_path, dtype):
    """bin/trace_run as a process on a mixed trace with two live requests and four pages."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [70, 20, 131], seed=300, weights=weights if dtype == "bfloat16" else None)
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
        rows = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        r = 0
        for e in st["entries"]:
            for i in e["want"]:
                got[(e["id"], fed[e["id"]] + i)] = torch.from_numpy(rows[r].copy())
                r += 1
            fed[e["id"]] += len(e["tokens"])
        assert r == rows.shape[0]
    L.compare(got, cfg, weights, seqs, **TOL[dtype])


def test_command_line_generates_with_the_folders_architecture(model):
    name, cfg, made = model
    weights, folder = made["float32"]
    prompt = H.random_ids(19, cfg["vocab"], 400)
    proc = subprocess.run([sys.executable, "-m", "lgml_b200", "-m", str(folder), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                           "-n", "5", "--temperature", "0", "--repeat-stop", "0"], capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(t) for t in proc.stdout.strip().splitlines()[-1].split(",")]
    assert len(got) == 5
    for i, tok in enumerate(got):
        row = L.oracle_logits(cfg, weights, prompt + got[:i])[-1]
        assert float(row.max() - row[tok]) <= 1e-4
