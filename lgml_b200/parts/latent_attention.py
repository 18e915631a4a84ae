"""Latent attention: the keys and values of all heads come from one small latent per token, and
only that latent and one rotated key part are cached.

    q        = W_q h                  per head [D plain | Dr rotated]
    c | r    = W_dkv h                c: the first R entries over their root mean square, times a weight
                                      r: the last Dr entries, rotated by the position
    k_h      = [W_uk,h c | r],  v_h = W_uv,h c
    s_j      = (q_plain . W_uk,h c_j + q_rot . r_j) * scale,   causal softmax,   out = W_o [sum_j w_j v_h,j]

The up-projections are taken to the other side of the two products: q_plain . (W_uk,h c_j) =
(W_uk,h^T q_plain) . c_j and sum_j w_j W_uv,h c_j = W_uv,h (sum_j w_j c_j).  Attention then runs with
H query heads of size R + Dr on ONE cached key head [c | r] whose first R entries are also the value:
the cache holds R + Dr numbers per token whatever the number of heads, and prompts, portions and
decoding are one path.  Rotation: the first ``rope_dims`` of the Dr entries, pairs (2i, 2i + 1), angle
pos * f_i, f_i = base^(-2i / rope_dims).

Options: ``window`` (a token sees itself and the window - 1 before it; the cache then keeps no more),
``out_gate`` (the concatenated heads times sigmoid(W_g h) before W_o, tensor ``.g``), and
``rope_scaling`` (factor, original, fast, slow), which stretches the slow frequencies for contexts
longer than ``original``: with n(t) = rope_dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(n(fast)), 0),
hi = min(ceil(n(slow)), rope_dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency
is f_i / factor * r_i + f_i (1 - r_i), and cosines and sines are multiplied by 0.1 ln(factor) + 1.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, Optional

import torch

from .. import ops
from ..cache import PagedKV
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part


def scaled_frequencies(base: float, dims: int, scaling: Optional[Dict[str, float]]):
    """The rotary frequencies of ``dims`` rotated entries as Python floats (double precision), and the
    factor on cosines and sines; ``scaling`` as in this module's description, or None."""
    half = dims // 2
    freq = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    turns = lambda t: dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turns(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freq):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * r + f * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


class LatentAttention(Part):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, rank: int, scale: float, eps: float,
                 rope_base: float, rope_dims: Optional[int] = None, window: Optional[int] = None, out_gate: bool = False,
                 rope_scaling: Optional[Dict[str, float]] = None):
        self.width, self.n_heads, self.head_dim, self.rot_dim = width, n_heads, head_dim, rot_dim
        self.v_head_dim, self.rank = v_head_dim, rank
        self.scale, self.eps = float(scale), float(eps)
        self.rope_base = float(rope_base)
        self.rope_dims = rot_dim if rope_dims is None else int(rope_dims)
        if self.rope_dims % 2 or self.rope_dims > rot_dim:
            raise ValueError(f"{self.rope_dims} rotated dimensions must be even and at most rot_dim {rot_dim}")
        self.window = int(window) if window else None
        self.out_gate = bool(out_gate)
        self.rope_scaling = dict(rope_scaling) if rope_scaling else None
        self.rot_mag = 1.0
        self.w_in = self.w_uk_t = self.w_uv = self.wo = self.norm_w = self.inv_freq = None

    def cache_spec(self):
        return PagedKV(1, self.rank + self.rot_dim, self.window, self.rank, v_in_k=True)

    def tensor_specs(self, prefix):
        H, D, Dr, Dv, R, E = self.n_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.rank, self.width
        gate = [TensorSpec(prefix + ".g", (H * Dv, E))] if self.out_gate else []
        return [TensorSpec(prefix + ".q", (H * (D + Dr), E)), TensorSpec(prefix + ".dkv", (R + Dr, E)),
                TensorSpec(prefix + ".dkv.norm", (R,), VECTOR, init=(1.0, 1.0)), TensorSpec(prefix + ".uk", (H * D, R)),
                TensorSpec(prefix + ".uv", (H * Dv, R)), TensorSpec(prefix + ".o", (E, H * Dv))] + gate

    def bind(self, prefix, tensors, rt):
        H, D, Dv, R = self.n_heads, self.head_dim, self.v_head_dim, self.rank
        # one product for everything that reads the mixer's input: queries, the down-projection, the output gate's logits
        self.w_in = torch.cat([tensors[prefix + ".q"], tensors[prefix + ".dkv"]] + ([tensors[prefix + ".g"]] if self.out_gate else []),
                              dim=0).contiguous()
        self.norm_w = tensors[prefix + ".dkv.norm"]
        self.w_uk_t = tensors[prefix + ".uk"].view(H, D, R).transpose(1, 2).contiguous()       # [H, R, D]: q_plain -> the latent's side
        self.w_uv = tensors[prefix + ".uv"].view(H, Dv, R).contiguous()
        self.wo = tensors[prefix + ".o"]
        freq, self.rot_mag = scaled_frequencies(self.rope_base, self.rope_dims, self.rope_scaling)
        exact = torch.tensor(freq or [0.0], dtype=torch.float64)
        hi = exact.to(torch.float32)
        self.inv_freq = torch.stack([hi, (exact - hi.double()).to(torch.float32)]).contiguous().to(rt.device)

    def first_weights(self):
        return [self.w_in]

    def forward(self, rt, h, batch, cache):
        H, D, Dr, Dv, R = self.n_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.rank
        n = h.shape[0]
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)
        nq = H * (D + Dr)
        q_plain, q_full = ops.latent_prepare(proj[:, :nq], proj[:, nq:nq + R + Dr], self.norm_w, self.eps, self.inv_freq, self.rope_dims, batch.positions,
                                             batch.seq_of_token, cache.block_table, cache.k, H, D, Dr, R, rt.status, write_kv=cache.writable,
                                             rot_mag=self.rot_mag)
        gate = proj[:, nq + R + Dr:] if self.out_gate else None
        window = self.window or 0
        ops.head_linear(q_plain, self.w_uk_t, q_full, D, R + Dr)
        o = torch.empty((n, H * Dv), dtype=h.dtype, device=h.device)
        if rt.dtype == torch.bfloat16 and (R + Dr) in (64, 128):
            # A cell of 64 or 128 numbers is a head size the plain causal attention kernels are built for (tcgen05 for
            # prompts, the split form for decoding): the whole cell serves as the value, and the product behind
            # attention reads only the first R entries of every head's result.
            whole = dataclasses.replace(cache, v=cache.k, writable=False)
            mix = torch.empty((n, H * (R + Dr)), dtype=h.dtype, device=h.device)
            rt.attention(q_full, batch, whole, mix, H, self.scale, window)
            ops.head_linear(mix, self.w_uv, o, R + Dr, Dv, gate=gate)
        else:
            mix = torch.empty((n, H * R), dtype=h.dtype, device=h.device)          # sum_j w_j c_j per head
            rt.sink_attention(q_full, batch, cache, mix, H, self.scale, window, None, None, None)
            ops.head_linear(mix, self.w_uv, o, R, Dv, gate=gate)
        return rt.linear(o, self.wo, partials_ok=True)


register_part("mixer", "latent_attention", LatentAttention)
