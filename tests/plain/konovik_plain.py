"""The Konovik decoder, plain and slow: float64 NumPy over whole sequences, one function per
mechanism, no cache, no batching, nothing shared with the engine.

``cfg`` is the configuration as a dictionary (the keys of config.json), ``W`` maps tensor names
to float64 arrays.  A sequence is a list of token ids; position t is its index.

Notation: T tokens, E the width, H heads, D the unrotated and Dr the rotated query/key size per
head, Dv the value size per head, R the latent's rank, m the residual multiplier.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    """The model's norm: x over its root mean square, times ONE learned number."""
    return rms_unit(x, eps) * float(g)


def token_shift(h, mu):
    """Every row moves towards the row before it: h_t + (h_(t-1) - h_t) mu, with zeros before the
    first token; the rows before them are the unshifted ones."""
    before = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (before - h) * mu


def min_gru(h, W, p):
    """A gated recurrence whose gates read the current token only: z = sigmoid(W_z h + b_z),
    u = W_x h + b_x, c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0); S_t = (1 - z) S_(t-1) + z c from
    S = 0; out = W_o (S_t silu(W_g h))."""
    z = sigmoid(h @ W[p + ".z"].T + W[p + ".z.b"])
    u = h @ W[p + ".x"].T + W[p + ".x.b"]
    c = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(z.shape[1])
    out = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        out[t] = S
    g = h @ W[p + ".g"].T
    return (out * g * sigmoid(g)) @ W[p + ".o"].T


def yarn_frequencies(base, dims, scaling):
    """The rotary frequencies f_i = base^(-2i / dims), i < dims / 2, and the factor on cos and sin.
    With ``scaling`` (factor, original, fast, slow) the slow frequencies are divided by ``factor``,
    the fast ones stay, with a linear ramp between: n(t) = dims ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dims - 1), r_i = clamp((i - lo) / max(hi - lo,
    0.001), 0, 1), f_i <- f_i / factor r_i + f_i (1 - r_i); cos and sin times 0.1 ln(factor) + 1."""
    half = dims // 2
    f = np.array([float(base) ** (-2.0 * i / dims) for i in range(half)])
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    n = lambda t: dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(n(float(scaling["fast"]))), 0)
    hi = min(math.ceil(n(float(scaling["slow"]))), dims - 1)
    r = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * r + f * (1.0 - r), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, rot, positions):
    """Rotary positions on the first ``rot.dims`` entries of the last axis of x [T, ..., n]: the pair
    (2i, 2i + 1) turns by positions * f_i; the rest passes unchanged."""
    dims = rot["dims"]
    f, mag = yarn_frequencies(rot["base"], dims, rot.get("scaling"))
    out = x.copy()
    half = dims // 2
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = (np.cos(a) * mag).reshape(shape), (np.sin(a) * mag).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T, window):
    """Position i sees j <= i, and with a window only the last ``window`` of them (itself included)."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    see = j <= i
    if window is not None:
        see &= (i - j) < window
    return see


def softmax_rows(s, see):
    s = np.where(see, s, -np.inf)
    e = np.where(see, np.exp(s - s.max(axis=-1, keepdims=True)), 0.0)
    return e / e.sum(axis=-1, keepdims=True)


def latent_attention(h, W, p, m, eps):
    """Keys and values of every head come from one latent c [T, R] (RMS-normed, a plain weight) and
    one rotated key part [T, Dr] shared by the heads; a sliding window; the concatenated heads times
    sigmoid(W_g h) before the output projection."""
    T = h.shape[0]
    H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    q = (h @ W[p + ".q"].T).reshape(T, H, D + Dr)
    q_plain, q_rot = q[:, :, :D], rotate_interleaved(q[:, :, D:], m["rot"], pos)
    down = h @ W[p + ".dkv"].T
    c = rms_unit(down[:, :R], eps) * W[p + ".dkv.norm"]
    k_rot = rotate_interleaved(down[:, R:], m["rot"], pos)
    k_plain = (c @ W[p + ".uk"].T).reshape(T, H, D)
    v = (c @ W[p + ".uv"].T).reshape(T, H, Dv)
    see = visible(T, m["mask"]["size"] if m.get("mask") else None)
    out = np.zeros((T, H, Dv))
    for hd in range(H):
        s = (q_plain[:, hd, :] @ k_plain[:, hd, :].T + q_rot[:, hd, :] @ k_rot.T) * m["scale"]
        out[:, hd, :] = softmax_rows(s, see) @ v[:, hd, :]
    return (out.reshape(T, H * Dv) * sigmoid(h @ W[p + ".g"].T)) @ W[p + ".o"].T


def dense_ff(h, W, p):
    a = h @ W[p + ".gate"].T
    return (a * sigmoid(a) * (h @ W[p + ".up"].T)) @ W[p + ".down"].T


def relu2_expert(h, W, p):
    return np.maximum(h @ W[p + ".up"].T, 0.0) ** 2 @ W[p + ".down"].T


def routed_ff(h, W, p, f, gaps=None):
    """Scores s = sigmoid(W_router h); the ``top`` experts with the largest s + correction are chosen;
    their weights are their s over the sum of those (+ 1e-20), times router.scale; a shared expert,
    if there is one, is added times sigmoid(W_sg h).  ``gaps`` (a list) receives, per token, how far
    the last chosen choice score lies above the first one left out."""
    n_exp, top, scale = f["router"]["experts"], f["router"]["top"], f["router"].get("scale", 1.0)
    s = sigmoid(h @ W[p + ".router"].T)
    choice = s + W[p + ".correction"]
    if gaps is not None:
        ranked = -np.sort(-choice, axis=1)
        gaps.append(ranked[:, top - 1] - ranked[:, top] if top < n_exp else np.full(h.shape[0], np.inf))
    out = np.zeros((h.shape[0], W[p + ".e0.down"].shape[0]))
    for t in range(h.shape[0]):
        chosen = np.argsort(-choice[t], kind="stable")[:top]
        w = s[t, chosen] / (s[t, chosen].sum() + 1e-20) * scale
        for e, we in zip(chosen, w):
            out[t] += we * relu2_expert(h[t], W, f"{p}.e{e}")
    if f.get("shared") is not None:
        out += sigmoid(h @ W[p + ".shared.sg"].T) * relu2_expert(h, W, p + ".shared")
    return out


def side_input(x, W, p, e, eps, sizes=None):
    """What a layer adds from its own small token table: y = W_proj (gelu_tanh(W_gate x) e), then y
    over its root mean square times a plain weight.  ``sizes``, a list, receives the root mean square of y
    per token: where it is tiny, the result is a unit vector of whatever the last bits of y hold."""
    y = (gelu_tanh(x @ W[p + ".gate"].T) * e) @ W[p + ".proj"].T
    if sizes is not None:
        sizes.append(np.sqrt(np.mean(y * y, axis=-1)))
    return rms_unit(y, eps) * W[p + ".norm"]


def layer_runs(cfg):
    """The layers in the order in which they run: layers start .. stop - 1 ``times`` times in a row,
    as (layer, first layer of a pass after the first?)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for r in range(times):
        runs += [(i, r > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(cfg, W, tokens, return_layers=False, router_gaps=None, side_sizes=None):
    """Logits [T, vocab] of a whole sequence (and, on request, the residual stream after every layer
    run; ``router_gaps``, a list, receives one array per routed layer run, ``side_sizes`` one per token input)."""
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    ids = np.asarray(tokens)
    x0 = scalar_norm(W["embed"][ids], W["embed.norm"], eps)
    x = x0.copy()
    side = cfg.get("token_side")
    layers = []
    for i, again in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}"
        if again:
            x = x + x0
        h = scalar_norm(x, W[p + ".norm1"], eps)
        if p + ".shift" in W:
            h = token_shift(h, W[p + ".shift"])
        if layer["type"] == "mingru":
            d = min_gru(h, W, p + ".mix")
        elif layer["type"] == "latent_attention":
            d = latent_attention(h, W, p + ".mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * d
        f = layer.get("mlp")
        if f is not None:
            h = scalar_norm(x, W[p + ".norm2"], eps)
            x = x + m * (dense_ff(h, W, p + ".mlp") if f["kind"] == "dense" else routed_ff(h, W, p + ".mlp", f, router_gaps))
        if side:
            n = side["dim"]
            x = x + m * side_input(x, W, p + ".side", W["side.embed"][ids, i * n:(i + 1) * n], eps, side_sizes)
        layers.append(x.copy())
    logits = scalar_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, layers) if return_layers else logits
