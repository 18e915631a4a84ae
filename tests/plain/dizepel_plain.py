"""The Dizepel decoder, plain and slow: float64 NumPy over whole sequences, one function per
mechanism, no cache, no batching, nothing shared with the engine.

``cfg`` is the configuration as a dictionary (the keys of config.json), ``W`` maps tensor names
to float64 arrays.  A sequence is a list of token ids; position t is its index.

Notation: T tokens, E the width, H query heads on G key heads of size D, values of size Dv; for
the state-space side Hs heads of size P on Gs groups with a state of N numbers.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(z))


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w along the last axis; no bias."""
    d = x - np.mean(x, axis=-1, keepdims=True)
    return d / np.sqrt(np.mean(d * d, axis=-1, keepdims=True) + eps) * w


def causal_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j); rows before the start are zero.
    The last column of w weighs the current row."""
    T, taps = u.shape[0], w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u], axis=0)
    y = np.zeros_like(u)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y if bias is None else y + bias


def stretched_frequencies(base, dims, scaling):
    """f_i = base^(-2i / dims) for i < dims / 2 and the factor on cos and sin.  With ``scaling``
    (factor, original, fast, slow): n(t) = dims ln(original / (2 pi t)) / (2 ln base), lo =
    max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dims - 1), r_i = clamp((i - lo) / max(hi - lo,
    0.001), 0, 1), f_i <- f_i / factor r_i + f_i (1 - r_i), and cos and sin times 0.1 ln(factor) + 1."""
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


def rotate_halves(x, rot, positions):
    """Rotary positions on the first ``rot.dims`` entries of the last axis of x [T, heads, n]: entry i
    pairs with entry i + dims / 2; the pair (u, v) at position p becomes (u cos a - v sin a,
    v cos a + u sin a), a = p f_i.  The rest passes unchanged."""
    dims = rot["dims"]
    half = dims // 2
    f, mag = stretched_frequencies(rot["base"], dims, rot.get("scaling"))
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(a) * mag)[:, None, :], (np.sin(a) * mag)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def capped_sink_attention(q, k, v, scale, softcap, sink):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; head h reads key head h // (H / G).  Scores q . k times
    ``scale``, then cap tanh(score / cap) when a cap is given; causal; the softmax's denominator holds
    exp(sink_h) as well, which has no value.  Returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        for t in range(T):
            row = s[t, :t + 1]
            m = max(row.max(), sink[h])
            e = np.exp(row - m)
            out[t, h] = (e @ v[:t + 1, g]) / (e.sum() + math.exp(sink[h] - m))
    return out


def attention_side(h, W, p, m):
    """The left mixer: q and k projections with biases, a short causal convolution on each of their
    channels, the values are the convolved keys before rotation, rotary positions on q and k, capped
    scores, a sink, then W_o."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(h @ W[p + ".q"].T + W[p + ".q.b"], W[p + ".q.conv"]).reshape(T, H, D)
    k = causal_conv(h @ W[p + ".k"].T + W[p + ".k.b"], W[p + ".k.conv"]).reshape(T, G, D)
    v = k[..., :Dv].copy()
    pos = np.arange(T)
    q, k = rotate_halves(q, m["rot"], pos), rotate_halves(k, m["rot"], pos)
    o = capped_sink_attention(q, k, v, m["scale"], m.get("softcap"), W[p + ".sink"])
    return o.reshape(T, H * Dv) @ W[p + ".o"].T


def state_space_scan(x, dt, a, B, C, Dskip):
    """x [T, Hs, P], dt [T, Hs] (already positive), a [Hs] (= exp(A_log)), B, C [T, Gs, N], Dskip [Hs]:
    S_t = exp(-a dt_t) S_(t-1) + dt_t B_t x_t^T (S is [N, P] per head, zero at the start),
    y_t = S_t^T C_t + Dskip x_t.  Head h reads group h // (Hs / Gs)."""
    T, Hs, P = x.shape
    Gs, N = B.shape[1], B.shape[2]
    y = np.zeros_like(x)
    for h in range(Hs):
        g = h // (Hs // Gs)
        S = np.zeros((N, P))
        for t in range(T):
            S = math.exp(-a[h] * dt[t, h]) * S + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + Dskip[h] * x[t, h]
    return y


def grouped_rms(y, n_groups, eps):
    """Each of ``n_groups`` equal parts of the last axis over its own root mean square."""
    T, n = y.shape
    return rms_unit(y.reshape(T, n_groups, n // n_groups), eps).reshape(T, n)


def state_space_side(h, W, p, m, eps):
    """The right mixer: one projection into z | x | B | C | dt; x, B, C through a causal convolution with
    a bias and silu; dt = softplus(dt + dt_bias); the scan; the gate silu(z) before the grouped norm; W_o."""
    T = h.shape[0]
    Hs, P, N, Gs = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hs * P
    proj = h @ W[p + ".in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * Gs * N], proj[:, 2 * inner + 2 * Gs * N:]
    xbc = silu(causal_conv(xbc, W[p + ".conv"], W[p + ".conv.b"]))
    x = xbc[:, :inner].reshape(T, Hs, P)
    B = xbc[:, inner:inner + Gs * N].reshape(T, Gs, N)
    C = xbc[:, inner + Gs * N:].reshape(T, Gs, N)
    dt = softplus(dt + W[p + ".dt_bias"])
    y = state_space_scan(x, dt, np.exp(W[p + ".A_log"]), B, C, W[p + ".D"]).reshape(T, inner)
    y = grouped_rms(y * silu(z), m["norm_groups"], eps) * W[p + ".norm"]
    return y @ W[p + ".o"].T


def parallel_mixer(h, W, p, m, eps):
    """Both sides read h; each result over its root mean square times its weight; half their sum."""
    left = attention_side(h, W, p + ".left", m["left"])
    right = state_space_side(h, W, p + ".right", m["right"], eps)
    return 0.5 * (rms_unit(left, eps) * W[p + ".left.out"] + rms_unit(right, eps) * W[p + ".right.out"])


def poly_norm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e with powers taken element by element and N a row over its root
    mean square."""
    a, b, c, e = (float(v) for v in coef)
    return a * rms_unit(z, eps) + b * rms_unit(z * z, eps) + c * rms_unit(z ** 3, eps) + e


def feed_forward(h, W, p, eps):
    return poly_norm(h @ W[p + ".up"].T, W[p + ".act"], eps) @ W[p + ".down"].T


def layer_runs(cfg):
    """[(layer, pass or None)]: the order in which layers run; ``pass`` is the number of the pass a looped
    range starts with this run (its step vector is added before it)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def layer(x, W, i, spec, eps, input_conv=True):
    """One layer; ``input_conv``: what each sublayer reads gains a causal convolution of itself."""
    p = f"l{i}"
    h = layer_norm(x, W[p + ".norm1"], eps)
    if input_conv:
        h = h + causal_conv(h, W[p + ".canon1"])
    x = x + layer_norm(parallel_mixer(h, W, p + ".mix", spec["mixer"], eps), W[p + ".norm1b"], eps)
    if spec.get("mlp") is not None:
        h = layer_norm(x, W[p + ".norm2"], eps)
        if input_conv:
            h = h + causal_conv(h, W[p + ".canon2"])
        x = x + layer_norm(feed_forward(h, W, p + ".mlp", eps), W[p + ".norm2b"], eps)
    return x


def forward(cfg, W, tokens, trace=None):
    """Logits [T, vocab] of a whole sequence.  ``trace``: a list that receives x after every layer run."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    for i, t in layer_runs(cfg):
        if t is not None:
            x = x + W["loop.step"][t]
        x = layer(x, W, i, cfg["layers"][i], eps, input_conv=cfg.get("canon") is not None)
        if trace is not None:
            trace.append(x.copy())
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T
