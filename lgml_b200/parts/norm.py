"""Norm parts.  RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, in float32
(``src/lgml.c:1626-1633``; the weight is the separate multiply of
``lua/lgml/transformer.lua:1760``, ``:2044``, ``:2095``).  DynamicTanh: y = tanh(alpha x) * w + b."""
from __future__ import annotations

import torch

from .. import ops
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part


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


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
