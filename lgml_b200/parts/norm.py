"""Norm parts.  RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, in float32
(``src/lgml.c:1626-1633``; the weight is the separate multiply of
``lua/lgml/transformer.lua:1760``, ``:2044``, ``:2095``).  DynamicTanh: y = tanh(alpha x) * w + b."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part


@dataclass
class UnitMix:
    """Half the sum of two results, each over its own root mean square and times its own weight:
    1/2 (a / rms(a) u_a + b / rms(b) u_b), not yet computed: the norm kernel that reads it does the arithmetic."""

    a: torch.Tensor
    b: torch.Tensor
    u_a: torch.Tensor
    u_b: torch.Tensor
    eps: float

    def tensor(self) -> torch.Tensor:
        """The combination itself, float32 (for a reader that takes plain tensors only)."""
        out = torch.zeros_like(self.a)
        ops.sandwich_norm(out, None, self.eps, None, delta=(self.a, self.b), units=(self.u_a, self.u_b))
        return out


@dataclass
class PendingDelta:
    """What a layer has computed but not yet added to the residual stream: ``delta`` (a float32 tensor or a
    ``UnitMix``; None: nothing) goes through a norm with the weight ``w_post`` first (None: as it is); ``row_add``
    is one row that every token's x gains as well."""

    delta: object = None
    w_post: Optional[torch.Tensor] = None
    row_add: Optional[torch.Tensor] = None
    eps: float = 0.0            # of the norm with ``w_post``


class RMSNorm(Part):
    """``single``: the learned weight is ONE number for all coordinates (a tensor without dimensions);
    the kernel reads it as a row of equal entries."""

    graph_safe = True
    def __init__(self, width: int, eps: float, suffix: str = ".weight", single: bool = False):
        self.width = width
        self.eps = float(eps)
        self.suffix = suffix        # what the weight's name adds to the part's prefix ("" when the prefix is the name)
        self.single = bool(single)
        self.weight = None

    def tensor_specs(self, prefix):
        return [TensorSpec(prefix + self.suffix, () if self.single else (self.width,), VECTOR, init=(1.0, 1.0))]

    def bind(self, prefix, tensors, rt):
        self.weight = tensors[prefix + self.suffix]
        if self.single:
            self.weight = self.weight.reshape(1).expand(self.width).contiguous()

    def forward(self, rt, x, out_dtype, delta=None, rows=None, delta_scale: float = 1.0):
        """Norm of x (+ delta_scale * delta).  x is the float32 residual stream; with ``delta`` the sum
        is written back to x.  ``rows`` (int32 on the device) picks the rows to norm."""
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        return ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows, delta_scale=delta_scale)


class DynamicTanh(Part):
    """Dynamic tanh: y = tanh(alpha x) * w + b, element by element, with a learned scalar alpha: a
    norm that computes no mean and no variance.  Tensors: the weight under the part's prefix itself,
    ``.b`` and ``.alpha`` beside it.  ``pre_scale`` multiplies x first (a norm that follows a scaled
    embedding takes the scale with it and the scaled rows are never written)."""

    graph_safe = True

    def __init__(self, width: int, pre_scale: float = 1.0):
        self.width = width
        self.pre_scale = float(pre_scale)
        self.weight = self.shift = self.alpha = None

    def tensor_specs(self, prefix):
        return [TensorSpec(prefix, (self.width,), VECTOR, init=(1.0, 1.0)), TensorSpec(prefix + ".b", (self.width,), VECTOR),
                TensorSpec(prefix + ".alpha", (), VECTOR, init=(0.5, 1.0))]

    def bind(self, prefix, tensors, rt):
        self.weight, self.shift = tensors[prefix], tensors[prefix + ".b"]
        self.alpha = tensors[prefix + ".alpha"].reshape(1).contiguous()

    def forward(self, rt, x, out_dtype, delta=None, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        return ops.dyt_norm(x, self.weight, self.shift, self.alpha, out, delta=delta, rows=rows, pre_scale=self.pre_scale)


class LayerNorm(Part):
    """y = (x - mean) / sqrt(var + eps) * w with var the mean of the squared deviations; no bias.  The same kernel
    first adds what is pending for the residual stream: ``delta`` may be a float32 tensor (added as it is) or a
    ``PendingDelta`` (normed with its own weight before the sum, and possibly one more row for every token)."""

    graph_safe = True
    takes_pending = True

    def __init__(self, width: int, eps: float, suffix: str = ""):
        self.width, self.eps, self.suffix = width, float(eps), suffix
        self.weight = None

    def tensor_specs(self, prefix):
        return [TensorSpec(prefix + self.suffix, (self.width,), VECTOR, init=(1.0, 1.0))]

    def bind(self, prefix, tensors, rt):
        self.weight = tensors[prefix + self.suffix].float().contiguous()

    def forward(self, rt, x, out_dtype, delta=None, rows=None, conv=None):
        """``conv``: (weights [taps, width], state slots, the rows' slots) of a convolution over time of the normed rows that the same
        kernel adds to them, for a step of one token a request (``ops.sandwich_norm``)."""
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        pend = delta if isinstance(delta, PendingDelta) else PendingDelta(delta)
        d, units = pend.delta, None
        if isinstance(d, ops.Partials):
            d = d.sum()
        if isinstance(d, UnitMix):
            d, units = (d.a, d.b), (d.u_a, d.u_b)
        return ops.sandwich_norm(x, self.weight, self.eps, out, delta=d, w_post=pend.w_post, units=units, row_add=pend.row_add, rows=rows, conv=conv)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
