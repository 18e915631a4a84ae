"""Test material for the Dizepel design: small configurations that differ from each other in every size and
option, random weights made so that the mechanisms show, and the oracle."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np
import torch

from tests.plain import dizepel_plain as P


def left(heads, kv_heads, dim, vdim, conv, scale, base=10000.0, dims=None, scaling=None, softcap=None):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale, "rot": rot}
    if softcap is not None:
        m["softcap"] = softcap
    return m


def right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def parallel(l, r, ff=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(vocab, width, layers, eps=1e-5, scale=None, taps=None, loop=None):
    cfg = {"architecture": "Dizepel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if scale is not None:
        cfg["embedding"] = {"scale": scale}
    if taps is not None:
        cfg["canon"] = {"taps": taps}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# A loop in the middle that runs three times; layers that differ in every size; heads of 16 and 24 entries of
# which 8 and 24 turn; values shorter than keys; stretched frequencies whose ramp lies inside the pairs;
# convolutions of 2 to 4 taps; a layer without a feed-forward.
LOOPED = config(97, 64, [
    parallel(left(4, 2, 16, 16, 4, 0.3, base=5000.0, dims=8, scaling=(4.0, 64, 8.0, 1.0), softcap=8.0), right(4, 8, 12, 2, 3, 2), ff=80),
    parallel(left(3, 3, 24, 20, 2, 0.2, base=300.0, softcap=30.0), right(6, 12, 20, 3, 4, 1), ff=None),
    parallel(left(2, 1, 32, 32, 3, 0.18, base=20000.0, dims=16), right(2, 40, 33, 1, 2, 4), ff=48),
    parallel(left(6, 2, 8, 4, 4, 0.4, base=50.0, dims=2, softcap=3.0), right(8, 4, 8, 8, 3, 8), ff=100),
], eps=1e-5, scale=2.5, taps=3, loop=(1, 3, 3))

# Sizes that are no multiple of 8 or of 4, one head, convolutions of one tap, no cap, no loop, no embedding scale,
# four taps on what the sublayers read.
ODD = config(61, 36, [
    parallel(left(1, 1, 12, 12, 1, 0.35, base=77.0, dims=4), right(1, 20, 5, 1, 1, 1), ff=20),
    parallel(left(5, 5, 10, 6, 3, 0.3, base=900.0, dims=10, scaling=(2.0, 32, 4.0, 2.0), softcap=5.0), right(3, 7, 48, 3, 5, 3), ff=52),
], eps=3e-6, taps=4)

# Heads of 64 and 128 entries (the tcgen05 prompt attention in bfloat16), a state of 128 numbers, a loop over all
# layers that runs twice, no convolution on what the sublayers read.
WIDE_HEADS = config(101, 96, [
    parallel(left(4, 2, 64, 64, 4, 0.11, base=150000.0, dims=48, scaling=(6.0, 128, 24.0, 1.0), softcap=25.0), right(3, 32, 128, 1, 4, 3), ff=72),
    parallel(left(2, 1, 128, 128, 2, 0.09, base=10000.0, dims=64, softcap=15.0), right(6, 16, 64, 2, 3, 2), ff=64),
], eps=1e-5, scale=4.0, loop=(0, 2, 2))

# A loop at the end that runs once more than the layers before it, heads of 48 and 80 (the mma.sync prompt attention),
# values of 16 from keys of 48, two taps on the sublayers' input.
TAIL_LOOP = config(83, 48, [
    parallel(left(2, 2, 48, 16, 3, 0.15, base=1000.0, dims=24, softcap=10.0), right(4, 12, 24, 4, 2, 2), ff=64),
    parallel(left(3, 1, 80, 80, 4, 0.11, base=40000.0, dims=40, scaling=(16.0, 48, 6.0, 0.5)), right(2, 24, 16, 2, 4, 1), ff=40),
    parallel(left(4, 4, 16, 16, 2, 0.25, base=100.0, dims=6, softcap=50.0), right(12, 4, 10, 6, 3, 6), ff=None),
], eps=1e-6, scale=0.7, taps=2, loop=(1, 3, 2))

CONFIGS = {"looped": LOOPED, "odd": ODD, "wide_heads": WIDE_HEADS, "tail_loop": TAIL_LOOP}


def random_weights(cfg: dict, seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    """Weights as bfloat16-representable float32 tensors, scaled so that no mechanism is lost in the noise:
    attention far from uniform with scores that reach the cap, sinks that weigh as much as a key, decays so
    slow that a state from hundreds of tokens back still counts, both sides of the mixer of equal weight."""
    g = torch.Generator().manual_seed(seed)
    E = cfg["width"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def vec(n, sd, mean=0.0):
        return torch.randn(n, generator=g) * sd + mean

    w = {"embed": torch.randn(cfg["vocab"], E, generator=g) * 0.5, "head": mat(cfg["vocab"], E), "final.norm": vec(E, 0.2, 1.0)}
    if cfg.get("loop"):
        w["loop.step"] = torch.randn(cfg["loop"]["times"], E, generator=g) * 0.5
    taps = cfg.get("canon", {}).get("taps")
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        l, r = layer["mixer"]["left"], layer["mixer"]["right"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if layer.get("mlp") else ()):
            w[p + n] = vec(E, 0.2, 1.0)
        if taps:
            w[p + "canon1"] = torch.randn(E, taps, generator=g) * 0.4
            if layer.get("mlp"):
                w[p + "canon2"] = torch.randn(E, taps, generator=g) * 0.4
        H, G, D, Dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
        q = p + "mix.left."
        w[q + "q"], w[q + "q.b"] = mat(H * D, E, 1.2 * sharpen), vec(H * D, 0.3)
        w[q + "k"], w[q + "k.b"] = mat(G * D, E, 1.2 * sharpen), vec(G * D, 0.3)
        w[q + "q.conv"] = torch.randn(H * D, l["conv"], generator=g) * 0.5 + torch.eye(l["conv"])[-1] * 0.7
        w[q + "k.conv"] = torch.randn(G * D, l["conv"], generator=g) * 0.5 + torch.eye(l["conv"])[-1] * 0.7
        w[q + "sink"], w[q + "o"], w[q + "out"] = vec(H, 1.5), mat(E, H * Dv), vec(E, 0.2, 1.0)
        Hs, Pd, N, Gs = r["heads"], r["vdim"], r["state"], r["groups"]
        inner, C = Hs * Pd, Hs * Pd + 2 * Gs * N
        q = p + "mix.right."
        w[q + "in"] = mat(inner + C + Hs, E, 1.5)
        w[q + "conv"], w[q + "conv.b"] = torch.randn(C, r["conv"], generator=g) * 0.5 + torch.eye(r["conv"])[-1] * 0.7, vec(C, 0.2)
        w[q + "dt_bias"] = vec(Hs, 1.0, -2.0)
        w[q + "A_log"] = vec(Hs, 1.0, -2.5)
        w[q + "D"], w[q + "norm"] = vec(Hs, 0.5, 1.0), vec(inner, 0.2, 1.0)
        w[q + "o"], w[q + "out"] = mat(E, inner), vec(E, 0.2, 1.0)
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(F, E, 1.5), mat(E, F)
            w[p + "mlp.act"] = torch.tensor([1.0, 0.6, -0.4, 0.1]) + 0.2 * torch.randn(4, generator=g)
    return {n: t.to(torch.bfloat16).float() for n, t in w.items()}


def write_folder(folder: Path, cfg: dict, weights: Dict[str, torch.Tensor]) -> Path:
    """config.json and model.safetensors (bfloat16) of a model."""
    from lgml_b200.weights import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {n: t.to(torch.bfloat16) for n, t in weights.items()})
    return folder


_oracle: Dict[Tuple[int, Tuple[int, ...]], torch.Tensor] = {}
_numpy: Dict[int, Dict[str, np.ndarray]] = {}


def numpy_of(weights):
    if id(weights) not in _numpy:
        _numpy[id(weights)] = {n: t.double().numpy() for n, t in weights.items()}
    return _numpy[id(weights)]


def oracle_logits(cfg: dict, weights: Dict[str, torch.Tensor], ids: List[int]) -> torch.Tensor:
    key = (id(weights), tuple(ids))
    if key not in _oracle:
        _oracle[key] = torch.from_numpy(P.forward(cfg, numpy_of(weights), list(ids)))
    return _oracle[key]


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
