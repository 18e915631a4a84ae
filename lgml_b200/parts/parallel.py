"""Two mixers side by side on the same input, and the two kinds this package has for it.

``ParallelMixer``: both sides read the same h; each result is divided by its root mean square over the
model width and multiplied by its own weight, and the mixer's result is half their sum:

    out = 1/2 (left(h) / rms(left(h)) * w_left + right(h) / rms(right(h)) * w_right)

The two in-projections are one product (the sides' matrices are stacked when bound); each side then gets
its columns of the float32 result.  The combination itself is not computed here: the part hands both
results and the two weights on as a ``UnitMix`` and the norm kernel that reads it does the arithmetic.
A side is any mixer with the two-step interface ``in_rows()`` -> (matrix, bias or None) and
``forward_projected(rt, proj, batch, cache)`` -> float32 [tokens, width].

``ConvAttention``: attention whose values are its keys.  q = W_q h + b_q and k = W_k h + b_k pass a short
causal convolution over time per channel; v is the convolved k's first Dv entries; q and k then turn by
their positions (the first ``rope_dims`` entries of each head, pairs (i, i + dims / 2), optionally with
stretched frequencies); score = cap tanh((q . k) scale / cap); causal softmax whose denominator also holds
exp(sink_h); W_o on the heads.  Its state: pages of k and v, and the last taps - 1 projected rows.

``StateSpaceDual``: the selective state-space recurrence with one decay per head.  W_in h = z | x | B | C | dt;
x, B, C pass a short causal convolution with a bias and silu; dt = softplus(dt + dt_bias);
S <- exp(-exp(A_log) dt) S + dt B x^T per head, y = S^T C + D x; (y silu(z)) over the root mean square of
each of ``norm_groups`` parts, times a weight; W_o.  Its state: S (float32) and the convolution's last inputs.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional

import torch

from .. import ops
from ..cache import FixedState, PagedKV
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part
from .latent_attention import scaled_frequencies
from .norm import UnitMix


# portions of a request longer than this run the state-space recurrence in pieces side by side
SSD_PIECES_FROM = 128


def _split_specs(spec):
    """(paged spec or None, fixed-state floats) of a mixer's cache spec."""
    specs = spec if isinstance(spec, (tuple, list)) else (spec,)
    paged = next((s for s in specs if isinstance(s, PagedKV)), None)
    fixed = next((s for s in specs if isinstance(s, FixedState)), None)
    if fixed is not None and (len(fixed.shape) != 1 or fixed.dtype != torch.float32):
        raise TypeError(f"sides share a state slot only as one row of float32 each, not {fixed}")
    return paged, (fixed.shape[0] if fixed is not None else 0)


class ConvAttention(Part):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, taps: int, scale: float,
                 rope_base: float, rope_dims: int, rope_scaling: Optional[Dict[str, float]] = None, softcap: Optional[float] = None,
                 sink: bool = True):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are no multiple of {n_kv_heads} key heads")
        if v_head_dim > head_dim:
            raise ValueError(f"values of {v_head_dim} entries cannot be taken from keys of {head_dim}")
        if rope_dims % 2 or rope_dims > head_dim:
            raise ValueError(f"{rope_dims} rotated entries must be even and at most the head size {head_dim}")
        if not 1 <= taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"a convolution of {taps} taps (1 to {ops.CONV_MAX_TAPS})")
        self.width, self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim = width, n_heads, n_kv_heads, head_dim, v_head_dim
        self.taps, self.scale, self.softcap, self.has_sink = int(taps), float(scale), float(softcap or 0.0), bool(sink)
        self.rope_base, self.rope_dims = float(rope_base), int(rope_dims)
        self.rope_scaling = dict(rope_scaling) if rope_scaling else None
        self.channels = (n_heads + n_kv_heads) * head_dim
        self.rot_mag = 1.0
        self.w_in = self.b_in = self.conv_w = self.wo = self.sinks = self.inv_freq = None

    def cache_spec(self):
        pages = PagedKV(self.n_kv_heads, self.head_dim, None, self.v_head_dim)
        return (pages, FixedState(((self.taps - 1) * self.channels,), torch.float32)) if self.taps > 1 else pages

    def tensor_specs(self, prefix):
        H, G, D, Dv, E = self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim, self.width
        specs = [TensorSpec(prefix + ".q", (H * D, E)), TensorSpec(prefix + ".q.b", (H * D,), VECTOR),
                 TensorSpec(prefix + ".k", (G * D, E)), TensorSpec(prefix + ".k.b", (G * D,), VECTOR),
                 TensorSpec(prefix + ".q.conv", (H * D, self.taps), VECTOR, init=(0.0, 10.0)),
                 TensorSpec(prefix + ".k.conv", (G * D, self.taps), VECTOR, init=(0.0, 10.0)),
                 TensorSpec(prefix + ".o", (E, H * Dv))]
        if self.has_sink:
            specs.append(TensorSpec(prefix + ".sink", (H,), VECTOR))
        return specs

    def bind(self, prefix, tensors, rt):
        t = lambda n: tensors[prefix + n]
        self.w_in = torch.cat([t(".q"), t(".k")], dim=0).contiguous()
        self.b_in = torch.cat([t(".q.b").float(), t(".k.b").float()]).contiguous()
        # [taps, channels]: the kernels read a tap's weights of neighbouring channels together
        self.conv_w = torch.cat([t(".q.conv"), t(".k.conv")], dim=0).float().t().contiguous()
        self.wo = t(".o")
        self.sinks = t(".sink").float().contiguous() if self.has_sink else None
        freq, self.rot_mag = scaled_frequencies(self.rope_base, self.rope_dims, self.rope_scaling)
        exact = torch.tensor(freq or [0.0], dtype=torch.float64)
        hi = exact.to(torch.float32)
        self.inv_freq = torch.stack([hi, (exact - hi.double()).to(torch.float32)]).contiguous().to(rt.device)

    def in_rows(self):
        return self.w_in, self.b_in

    def first_weights(self):
        return [self.w_in]

    def forward_projected(self, rt, proj, batch, cache):
        H, Dv = self.n_heads, self.v_head_dim
        q = ops.conv_rope_store(proj, self.conv_w, cache.state, batch.positions, batch.seq_of_token, batch.seq_start, batch.slots,
                                cache.block_table, self.inv_freq, self.rot_mag, self.rope_dims, cache.k, cache.v, H, rt.status,
                                write_kv=cache.writable)
        o = torch.empty((q.shape[0], H * Dv), dtype=q.dtype, device=q.device)
        rt.sink_attention(q, batch, cache, o, H, self.scale, 0, None, self.sinks, None, softcap=self.softcap)
        return rt.linear(o, self.wo, out_dtype=torch.float32)

    def forward(self, rt, h, batch, cache):
        return self.forward_projected(rt, rt.linear(h, self.w_in, bias=self.b_in, out_dtype=torch.float32), batch, cache)


class StateSpaceDual(Part):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, head_dim: int, n_state: int, n_groups: int, taps: int, norm_groups: int, eps: float):
        if n_heads % n_groups:
            raise ValueError(f"{n_heads} heads are no multiple of {n_groups} groups")
        if (n_heads * head_dim) % norm_groups:
            raise ValueError(f"{n_heads * head_dim} channels do not split into {norm_groups} equal parts")
        if not 1 <= taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"a convolution of {taps} taps (1 to {ops.CONV_MAX_TAPS})")
        self.width, self.n_heads, self.head_dim, self.n_state, self.n_groups = width, n_heads, head_dim, n_state, n_groups
        self.taps, self.norm_groups, self.eps = int(taps), int(norm_groups), float(eps)
        self.inner = n_heads * head_dim
        self.conv_channels = self.inner + 2 * n_groups * n_state
        self.state_floats = self.inner * n_state
        self.w_in = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm_w = self.wo = None

    def cache_spec(self):
        return FixedState((self.state_floats + (self.taps - 1) * self.conv_channels,), torch.float32)

    def tensor_specs(self, prefix):
        Hs, E, C = self.n_heads, self.width, self.conv_channels
        return [TensorSpec(prefix + ".in", (self.inner + C + Hs, E)),
                TensorSpec(prefix + ".conv", (C, self.taps), VECTOR, init=(0.0, 10.0)), TensorSpec(prefix + ".conv.b", (C,), VECTOR),
                TensorSpec(prefix + ".dt_bias", (Hs,), VECTOR), TensorSpec(prefix + ".A_log", (Hs,), VECTOR),
                TensorSpec(prefix + ".D", (Hs,), VECTOR, init=(1.0, 1.0)), TensorSpec(prefix + ".norm", (self.inner,), VECTOR, init=(1.0, 1.0)),
                TensorSpec(prefix + ".o", (E, self.inner))]

    def bind(self, prefix, tensors, rt):
        t = lambda n: tensors[prefix + n]
        self.w_in, self.wo = t(".in"), t(".o")
        self.conv_w = t(".conv").float().t().contiguous()
        self.conv_b = t(".conv.b").float().contiguous()
        self.dt_bias, self.a_log, self.d_skip = (t(n).float().contiguous() for n in (".dt_bias", ".A_log", ".D"))
        self.norm_w = t(".norm").float().contiguous()

    def in_rows(self):
        return self.w_in, None

    def first_weights(self):
        return [self.w_in]

    def forward_projected(self, rt, proj, batch, cache):
        inner, C, Hs = self.inner, self.conv_channels, self.n_heads
        n = proj.shape[0]
        xbc = torch.empty((n, C), dtype=torch.float32, device=proj.device)
        ops.short_conv(proj[:, inner:inner + C], self.conv_w, self.conv_b, cache.state[:, self.state_floats:] if self.taps > 1 else None,
                       batch.seq_of_token, batch.seq_start, batch.slots, xbc, act="silu")
        # a long portion's recurrence runs in pieces side by side
        pieces = batch.scan_pieces(ops.SSD_PIECE_TOKENS) if batch.max_q_len > SSD_PIECES_FROM else None
        y = ops.ssd_scan(xbc, proj[:, inner + C:inner + C + Hs], self.dt_bias, self.a_log, self.d_skip, cache.state, batch.seq_start, batch.slots,
                         Hs, self.n_groups, self.head_dim, self.n_state, pieces=pieces)
        g = ops.ssd_gate_norm(y, proj[:, :inner], self.norm_w, self.norm_groups, self.eps, rt.dtype)
        return rt.linear(g, self.wo, out_dtype=torch.float32)

    def forward(self, rt, h, batch, cache):
        return self.forward_projected(rt, rt.linear(h, self.w_in, out_dtype=torch.float32), batch, cache)


class ParallelMixer(Part):
    def __init__(self, width: int, left, right, eps: float, names=(".left", ".right"), out_suffix: str = ".out"):
        self.width, self.left, self.right, self.eps = width, left, right, float(eps)
        self.names, self.out_suffix = tuple(names), out_suffix
        self.w_in = self.b_in = self.u_left = self.u_right = None
        self.n_left = 0
        lp, lf = _split_specs(left.cache_spec())
        rp, rf = _split_specs(right.cache_spec())
        if lp is not None and rp is not None:
            raise TypeError("at most one side of a parallel mixer keeps pages")
        self._paged, self._floats = lp or rp, (lf, rf)

    @property
    def graph_safe(self):
        return bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    def cache_spec(self):
        fixed = FixedState((sum(self._floats),), torch.float32) if sum(self._floats) else None
        both = tuple(s for s in (self._paged, fixed) if s is not None)
        return both if len(both) > 1 else (both[0] if both else None)

    def tensor_specs(self, prefix):
        return (self.left.tensor_specs(prefix + self.names[0]) + self.right.tensor_specs(prefix + self.names[1])
                + [TensorSpec(prefix + self.names[0] + self.out_suffix, (self.width,), VECTOR, init=(1.0, 1.0)),
                   TensorSpec(prefix + self.names[1] + self.out_suffix, (self.width,), VECTOR, init=(1.0, 1.0))])

    def bind(self, prefix, tensors, rt):
        self.left.bind(prefix + self.names[0], tensors, rt)
        self.right.bind(prefix + self.names[1], tensors, rt)
        (wl, bl), (wr, br) = self.left.in_rows(), self.right.in_rows()
        self.n_left = wl.shape[0]
        self.w_in = torch.cat([wl, wr], dim=0).contiguous()
        self.b_in = None
        if bl is not None or br is not None:
            zeros = lambda w: torch.zeros(w.shape[0], dtype=torch.float32, device=w.device)
            self.b_in = torch.cat([bl if bl is not None else zeros(wl), br if br is not None else zeros(wr)]).contiguous()
        self.u_left = tensors[prefix + self.names[0] + self.out_suffix].float().contiguous()
        self.u_right = tensors[prefix + self.names[1] + self.out_suffix].float().contiguous()

    def first_weights(self):
        return [self.w_in]

    def _side_cache(self, cache, first: int, floats: int, paged: bool):
        state = cache.state[:, first:first + floats] if floats else None
        if paged:
            return dataclasses.replace(cache, state=state)
        return dataclasses.replace(cache, k=None, v=None, block_table=None, state=state)

    def forward(self, rt, h, batch, cache):
        proj = rt.linear(h, self.w_in, bias=self.b_in, out_dtype=torch.float32)
        lf, rf = self._floats
        left_paged = self._paged is not None and _split_specs(self.left.cache_spec())[0] is not None
        a = self.left.forward_projected(rt, proj[:, :self.n_left], batch, self._side_cache(cache, 0, lf, left_paged))
        b = self.right.forward_projected(rt, proj[:, self.n_left:], batch, self._side_cache(cache, lf, rf, self._paged is not None and not left_paged))
        return UnitMix(a, b, self.u_left, self.u_right, self.eps)


register_part("mixer", "conv_attention", ConvAttention)
register_part("mixer", "state_space_dual", StateSpaceDual)
register_part("mixer", "parallel", ParallelMixer)
