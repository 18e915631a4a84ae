"""Test material for the Konovik design: small configurations that differ from each other in every
size and option, random weights made so that the mechanisms show, and the oracle."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np
import torch

from tests.plain import konovik_plain as P


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, scale=None, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if scale is not None:
        f["router"]["scale"] = scale
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def mingru(width, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, dims=None, window=None, scaling=None, mlp=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def config(vocab, width, layers, eps=1e-5, mult=None, side=None, loop=None):
    cfg = {"architecture": "Konovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if mult is not None:
        cfg["residual_mult"] = mult
    if side is not None:
        cfg["token_side"] = {"dim": side}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# A loop in the middle that runs three times over a recurrent and an attention layer; recurrences
# narrower and wider than the model; windows below a page and across pages; stretched frequencies whose
# ramp lies inside the rotated pairs; a layer without a feed-forward; experts with and without a shared one.
LOOPED = config(97, 64, [
    mingru(48, mlp=dense(80)),
    latent(3, 16, 8, 12, 24, scale=0.2, base=5000.0, window=20, scaling=(4.0, 64, 8.0, 1.0), mlp=moe(24, 5, 2, scale=1.5, shared=40)),
    mingru(64, mlp=moe(16, 3, 1, shared=24)),
    latent(2, 24, 12, 20, 40, scale=0.15, base=300.0, window=70),
    mingru(80, mlp=dense(48)),
], eps=1e-5, mult=0.5, side=12, loop=(1, 3, 3))

# One head, sizes that are no multiple of 8 or of 4, a window of 1, one expert, no loop, no residual
# multiplier, two attention layers in a row, fewer rotated pairs than the rotated part holds.
ODD = config(61, 36, [
    latent(1, 12, 2, 20, 10, scale=0.3, base=77.0, window=1, mlp=moe(20, 1, 1, scale=0.7)),
    latent(5, 12, 6, 4, 14, scale=0.35, base=50.0, dims=4, window=65, scaling=(2.0, 32, 4.0, 2.0), mlp=dense(20)),
    mingru(21, mlp=moe(10, 4, 4, shared=6)),
    mingru(36),
], eps=3e-6, side=5)

# No token input, a latent layer without a window beside one with a window of exactly a page, a loop over
# all layers, all experts chosen.
NO_SIDE = config(83, 48, [
    latent(4, 8, 8, 8, 16, scale=0.25, base=1000.0, mlp=moe(16, 6, 6, scale=2.5)),
    mingru(40, mlp=dense(64)),
    latent(2, 16, 4, 24, 20, scale=0.2, base=20000.0, window=64, scaling=(8.0, 128, 16.0, 1.0), mlp=moe(16, 6, 3, shared=16)),
], eps=1e-5, mult=0.3, loop=(0, 3, 2))

# Cells of 64 and 128 numbers (latent + rotated part), which the tensor-core attention kernels take, under
# windows; a wide recurrence; a loop at the end.
WIDE_HEADS = config(101, 96, [
    latent(4, 32, 32, 32, 96, scale=0.1, base=30000.0, window=100, scaling=(4.0, 256, 32.0, 1.0), mlp=moe(40, 8, 2, scale=2.0, shared=48)),
    mingru(128, mlp=dense(72)),
    latent(2, 64, 16, 64, 48, scale=0.1, base=500.0, window=40, mlp=dense(64)),
    mingru(96, mlp=moe(40, 8, 2)),
], eps=1e-5, mult=0.7, side=16, loop=(2, 4, 2))

# Cells wider than any tensor-core attention kernel takes (160 and 288 numbers), a loop from the
# first layer, a recurrence far wider than the model.
BIG_CELLS = config(211, 72, [
    latent(2, 16, 32, 16, 128, scale=0.2, base=10000.0, window=48, scaling=(8.0, 64, 32.0, 1.0), mlp=moe(12, 6, 2, scale=2.0, shared=20)),
    mingru(200, mlp=dense(56)),
    latent(3, 24, 16, 8, 272, scale=0.15, base=2000.0, window=130, mlp=dense(40)),
], eps=1e-6, mult=0.3, side=24, loop=(0, 2, 2))

# how far apart a router's choice must lie in the plain model for a bfloat16 run to be compared on a token: the wide
# cells' scores are sums over hundreds of rounded numbers, and what comes after them wobbles more
CLEAR_GAP = {id(BIG_CELLS): 0.05}

CONFIGS = {"looped": LOOPED, "odd": ODD, "no_side": NO_SIDE, "wide_heads": WIDE_HEADS, "big_cells": BIG_CELLS}


def random_weights(cfg: dict, seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    """Weights as bfloat16-representable float32 tensors, scaled so that no mechanism is lost in the
    noise: attention far from uniform, shifts between 0 and 1, gates of the recurrence on both sides,
    candidates on both sides of 0, router scores apart, a correction that changes choices."""
    g = torch.Generator().manual_seed(seed)
    E = cfg["width"]
    n_layers = len(cfg["layers"])

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def vec(n, sd, mean=0.0):
        return torch.randn(n, generator=g) * sd + mean

    one = lambda: torch.tensor(1.0) + 0.2 * (torch.rand((), generator=g) - 0.5)
    w = {"embed": torch.randn(cfg["vocab"], E, generator=g) * 0.5, "head": mat(cfg["vocab"], E), "embed.norm": one(), "final.norm": one()}
    side = cfg.get("token_side")
    if side:
        w["side.embed"] = torch.randn(cfg["vocab"], n_layers * side["dim"], generator=g)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        w[p + "norm1"] = one()
        w[p + "shift"] = torch.rand(E, generator=g)
        if layer["type"] == "mingru":
            W = m["width"]
            w[p + "mix.z"], w[p + "mix.z.b"] = mat(W, E, 2.0), vec(W, 0.5)
            w[p + "mix.x"], w[p + "mix.x.b"] = mat(W, E, 2.0), vec(W, 0.5)
            w[p + "mix.g"], w[p + "mix.o"] = mat(W, E, 1.5), mat(E, W)
        else:
            H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[p + "mix.q"] = mat(H * (D + Dr), E, 1.5 * sharpen)
            w[p + "mix.dkv"] = mat(R + Dr, E, 1.5 * sharpen)
            w[p + "mix.dkv.norm"] = vec(R, 0.2, 1.0)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * D, R, 1.5), mat(H * Dv, R, 1.5)
            w[p + "mix.g"], w[p + "mix.o"] = mat(H * Dv, E, 2.0), mat(E, H * Dv)
        f = layer.get("mlp")
        if f:
            w[p + "norm2"] = one()
            if f["kind"] == "dense":
                F = f["ff"]
                w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(F, E, 2.0), mat(F, E, 2.0), mat(E, F)
            else:
                F, X = f["expert"]["ff"], f["router"]["experts"]
                w[p + "mlp.router"], w[p + "mlp.correction"] = mat(X, E, 4.0), vec(X, 0.3)
                for e in range(X):
                    w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(F, E, 2.0), mat(E, F, 1.0 + 0.3 * e)
                if f.get("shared"):
                    Fs = f["shared"]["ff"]
                    w[p + "mlp.shared.up"], w[p + "mlp.shared.down"], w[p + "mlp.shared.sg"] = mat(Fs, E, 2.0), mat(E, Fs), mat(1, E, 2.0)
        if side:
            n = side["dim"]
            w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"] = mat(n, E, 0.5), mat(E, n), vec(E, 0.2, 1.0)
    return {n: t.to(torch.bfloat16).float() for n, t in w.items()}


def write_folder(folder: Path, cfg: dict, weights: Dict[str, torch.Tensor]) -> Path:
    """config.json and model.safetensors (bfloat16) of a model."""
    from lgml_b200.weights import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {n: t.to(torch.bfloat16) for n, t in weights.items()})
    return folder


def as_numpy(weights: Dict[str, torch.Tensor]) -> Dict[str, np.ndarray]:
    return {n: t.double().numpy() for n, t in weights.items()}


_oracle: Dict[Tuple[int, Tuple[int, ...]], torch.Tensor] = {}
_numpy: Dict[int, Dict[str, np.ndarray]] = {}


def numpy_of(weights):
    if id(weights) not in _numpy:
        _numpy[id(weights)] = as_numpy(weights)
    return _numpy[id(weights)]


def oracle_logits(cfg: dict, weights: Dict[str, torch.Tensor], ids: List[int]) -> torch.Tensor:
    key = (id(weights), tuple(ids))
    if key not in _oracle:
        _oracle[key] = torch.from_numpy(P.forward(cfg, numpy_of(weights), list(ids)))
    return _oracle[key]


def clear_ids(cfg: dict, weights: Dict[str, torch.Tensor], n: int, seed: int, gap: float = None, small: float = 0.2) -> List[int]:
    """n random token ids on which a bfloat16 run may be compared: no router of the plain model decides by less
    than ``gap`` (the choice scores are sigmoids plus a correction, so they lie close together), and no token
    input is smaller than ``small`` times that layer's median before it is divided by its root mean square (a
    few numbers per layer can all but cancel, and the unit vector made of the rest magnifies every rounding
    ahead of it).  The model is causal, so the first such position is redrawn and the sequence checked again."""
    import random

    if gap is None:
        gap = CLEAR_GAP.get(id(cfg), 0.02)
    rng = random.Random(seed)
    ids = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    for _ in range(40 * n):
        gaps: list = []
        sizes: list = []
        P.forward(cfg, numpy_of(weights), ids, router_gaps=gaps, side_sizes=sizes)
        bad = np.zeros(n, dtype=bool)
        if gaps:
            bad |= np.min(np.stack(gaps), axis=0) < gap
        for r in sizes:
            bad |= r < small * max(float(np.median(r)), 1e-3)
        close = np.nonzero(bad)[0]
        if close.size == 0:
            return ids
        ids[int(close[0])] = rng.randrange(cfg["vocab"])
    raise AssertionError("no sequence without a close call was found")


def compare(got: Dict[Tuple[str, int], torch.Tensor], cfg, weights, seqs: Dict[str, List[int]], atol: float, rtol: float) -> float:
    """Largest error over all rows that ``got`` holds; raises naming the first wrong (request, position)."""
    worst = 0.0
    for rid, ids in seqs.items():
        ref = oracle_logits(cfg, weights, ids)
        for p in range(len(ids)):
            if (rid, p) not in got:
                continue
            row = got[(rid, p)].double()
            err = (row - ref[p]).abs()
            bound = atol + rtol * ref[p].abs().max()
            if bool((err > bound).any()):
                j = int(err.argmax())
                raise AssertionError(f"request {rid} position {p} (page {p // 64}, cell {p % 64}): logit {j} is {row[j]:.6g}, "
                                     f"oracle {ref[p, j]:.6g}, |diff| {err[j]:.3g} > {bound:.3g}")
            worst = max(worst, float(err.max()))
    return worst
