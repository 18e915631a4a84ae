"""Feed-forward parts.  The gated one: down(act(gate(h)) * up(h)) with act = SiLU
(``lua/lgml/transformer.lua:2047-2049``; silu(a) = a * sigmoid(a),
``src/lgml.c:1476-1482``).  Gate and up are one fused product: the two matrices
are concatenated row-wise when they are bound, gate first."""
from __future__ import annotations

import torch

from .. import ops
from ..weights import MATRIX, VECTOR, TensorSpec
from .base import Part, register_part


class GatedMLP(Part):
    graph_safe = True
    def __init__(self, width: int, inner: int, activation: str = "silu", bias: bool = False,
                 names=(".gate_proj.weight", ".up_proj.weight", ".down_proj.weight")):
        if activation != "silu":
            raise ValueError(f"activation '{activation}' is not supported (only 'silu')")
        self.width, self.inner, self.bias = width, inner, bool(bias)
        self.names = tuple(names)       # what the three matrices' names add to the part's prefix: gate, up, down
        if self.bias and self.names != (".gate_proj.weight", ".up_proj.weight", ".down_proj.weight"):
            raise ValueError("biases come with the default tensor names only")
        self.wgu = self.bgu = self.wd = self.bd = None

    def tensor_specs(self, prefix):
        E, F = self.width, self.inner
        specs = [TensorSpec(prefix + self.names[0], (F, E)), TensorSpec(prefix + self.names[1], (F, E)),
                 TensorSpec(prefix + self.names[2], (E, F))]
        if self.bias:
            specs += [TensorSpec(prefix + ".gate_proj.bias", (F,), VECTOR), TensorSpec(prefix + ".up_proj.bias", (F,), VECTOR),
                      TensorSpec(prefix + ".down_proj.bias", (E,), VECTOR)]
        return specs

    def bind(self, prefix, tensors, rt):
        wg, wu = tensors[prefix + self.names[0]], tensors[prefix + self.names[1]]
        self.wd = tensors[prefix + self.names[2]]
        bg = bu = None
        if self.bias:
            bg, bu = tensors[prefix + ".gate_proj.bias"], tensors[prefix + ".up_proj.bias"]
            self.bd = tensors[prefix + ".down_proj.bias"]
        # bfloat16: the gate and up rows of a feature lie next to each other, so the product's
        # epilogue has both and applies the activation itself; float32: gate rows, then up rows.
        self.paired = rt.dtype == torch.bfloat16
        if self.paired:
            self.wgu = torch.stack([wg, wu], dim=1).reshape(2 * self.inner, self.width).contiguous()
            self.bgu = torch.stack([bg, bu], dim=1).reshape(2 * self.inner).contiguous() if self.bias else None
        else:
            self.wgu = torch.cat([wg, wu], dim=0).contiguous()
            self.bgu = torch.cat([bg, bu], dim=0).contiguous() if self.bias else None

    def first_weights(self):
        return [self.wgu]

    def forward(self, rt, h):
        if self.paired and rt.fused_swiglu(h, self.wgu):
            act = ops.gemm_bf16_swiglu(h, self.wgu, self.bgu, rt.status)
        else:
            gu = rt.linear(h, self.wgu, bias=self.bgu)
            act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
            ops.silu_mul(gu, act, paired=self.paired)
        return rt.linear(act, self.wd, bias=self.bd, partials_ok=True)


class DenseMLP(Part):
    """The dense feed-forward down(act(up(h) + b_up)) + b_down with act = relu squared."""

    graph_safe = True

    def __init__(self, width: int, inner: int, activation: str = "relu2", bias: bool = True):
        if activation != "relu2":
            raise ValueError(f"activation '{activation}' is not supported (only 'relu2')")
        self.width, self.inner, self.bias = width, inner, bool(bias)
        self.wu = self.bu = self.wd = self.bd = None

    def tensor_specs(self, prefix):
        E, F = self.width, self.inner
        specs = [TensorSpec(prefix + ".up", (F, E)), TensorSpec(prefix + ".down", (E, F))]
        if self.bias:
            specs += [TensorSpec(prefix + ".up.b", (F,), VECTOR), TensorSpec(prefix + ".down.b", (E,), VECTOR)]
        return specs

    def bind(self, prefix, tensors, rt):
        self.wu, self.wd = tensors[prefix + ".up"], tensors[prefix + ".down"]
        if self.bias:
            self.bu, self.bd = tensors[prefix + ".up.b"], tensors[prefix + ".down.b"]

    def first_weights(self):
        return [self.wu]

    def forward(self, rt, h):
        if rt.fused_swiglu(h, self.wu):       # the product's epilogue applies the activation
            act = ops.gemm_bf16_relu_sq(h, self.wu, self.bu, rt.status)
        else:
            act = ops.relu_sq(rt.linear(h, self.wu, bias=self.bu))
        return rt.linear(act, self.wd, bias=self.bd, partials_ok=True)


class ClampedGLU(Part):
    """The gated feed-forward with clamped branches: g = min(W_gate h, limit), u = clamp(W_up h,
    -limit, limit), y = W_down (g * sigmoid(alpha g) * (u + 1)).  Gate and up are one product."""

    graph_safe = True

    def __init__(self, width: int, inner: int, limit: float, alpha: float = 1.702):
        self.width, self.inner, self.limit, self.alpha = width, inner, float(limit), float(alpha)
        self.wgu = self.wd = None
        self.paired = False

    def tensor_specs(self, prefix):
        E, F = self.width, self.inner
        return [TensorSpec(prefix + ".gate", (F, E)), TensorSpec(prefix + ".up", (F, E)), TensorSpec(prefix + ".down", (E, F))]

    def bind(self, prefix, tensors, rt):
        wg, wu = tensors[prefix + ".gate"], tensors[prefix + ".up"]
        self.wd = tensors[prefix + ".down"]
        # bfloat16: the gate and up rows of a feature lie next to each other, so that the product's
        # epilogue has both and applies the activation itself; float32: gate rows, then up rows
        self.paired = rt.dtype == torch.bfloat16
        if self.paired:
            self.wgu = torch.stack([wg, wu], dim=1).reshape(2 * self.inner, self.width).contiguous()
        else:
            self.wgu = torch.cat([wg, wu], dim=0).contiguous()

    def first_weights(self):
        return [self.wgu]

    def forward(self, rt, h):
        if self.paired and rt.fused_swiglu(h, self.wgu) and ops.GLU_CLAMPED_FUSED:
            act = ops.gemm_bf16_glu_clamped(h, self.wgu, self.alpha, self.limit, rt.status)
        else:
            gu = rt.linear(h, self.wgu)
            act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
            ops.glu_clamped(gu, act, self.alpha, self.limit, paired=self.paired)
        return rt.linear(act, self.wd, partials_ok=True)


class PolyNormMLP(Part):
    """down(act(up(h))) with act(z) = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e: powers element by
    element, every power over its own root mean square along the row (eps inside the root); the four numbers
    are the tensor ``.act``.  The first product's result and the activation are float32."""

    graph_safe = True

    def __init__(self, width: int, inner: int, eps: float, names=(".up", ".down", ".act")):
        self.width, self.inner, self.eps, self.names = width, inner, float(eps), tuple(names)
        self.wu = self.wd = self.coef = None

    def tensor_specs(self, prefix):
        return [TensorSpec(prefix + self.names[0], (self.inner, self.width)), TensorSpec(prefix + self.names[1], (self.width, self.inner)),
                TensorSpec(prefix + self.names[2], (4,), VECTOR, init=(0.5, 5.0))]

    def bind(self, prefix, tensors, rt):
        self.wu, self.wd = tensors[prefix + self.names[0]], tensors[prefix + self.names[1]]
        self.coef = tensors[prefix + self.names[2]].float().contiguous()

    def first_weights(self):
        return [self.wu]

    def forward(self, rt, h):
        z = rt.linear(h, self.wu, out_dtype=torch.float32)
        act = torch.empty(z.shape, dtype=rt.dtype, device=z.device)
        ops.poly_norm(z, self.coef, self.eps, act)
        return rt.linear(act, self.wd, out_dtype=torch.float32)


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "clamped_glu", ClampedGLU)
register_part("feed_forward", "dense_mlp", DenseMLP)
register_part("feed_forward", "polynorm_mlp", PolyNormMLP)
