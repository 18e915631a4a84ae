"""A mixture of experts as a feed-forward part.

    z      = W_router h + b_router               float32 logits, one per expert
    chosen = the ``top`` experts with the largest z;  w = softmax over the chosen z alone
    y      = sum_e w_e W_down,e (act(W_gate,e h) * (W_up,e h)),   act = silu

Tensors: ``.router`` [X, E], ``.router.b`` [X], ``.e<i>.gate`` / ``.up`` [F, E], ``.e<i>.down`` [E, F]
(no biases in the experts).  The experts' matrices are stacked when they are bound (gate and up of a
feature as neighbouring rows), so that a kernel finds expert e at a fixed stride.

Other forms of the same part, by constructor arguments:

* ``router="sigmoid"``: the scores are s = sigmoid(z); the experts with the largest s + bias are chosen (the
  bias corrects the choice only), and w = s of the chosen over their sum (+ 1e-20), times ``route_scale``;
* ``gated=False``: experts without a gate, W_down,e act(W_up,e h) with act = relu squared;
* ``shared_inner``: one more expert of that inner width and the same form that every token uses
  (``.shared.up``, ``.shared.down``), added times sigmoid(W_sg h), one number per token (``.shared.sg`` [1, E]);
* ``bias_name``: what the bias's name adds to the part's prefix.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part


class RoutedExperts(Part):
    graph_safe = True

    def __init__(self, width: int, inner: int, n_experts: int, top: int, router_bias: bool = True, router: str = "softmax",
                 route_scale: float = 1.0, gated: bool = True, shared_inner: int = 0, bias_name: str = ".router.b"):
        if not 0 < top <= n_experts:
            raise ValueError(f"{top} of {n_experts} experts cannot be chosen")
        if router not in ops.ROUTER_MODES:
            raise ValueError(f"unknown router '{router}' (known: {', '.join(ops.ROUTER_MODES)})")
        if shared_inner and gated:
            raise ValueError("a shared expert comes only with experts without a gate")
        self.width, self.inner, self.n_experts, self.top = width, inner, n_experts, top
        self.router_bias = bool(router_bias)
        self.router, self.route_scale, self.gated = router, float(route_scale), bool(gated)
        self.shared_inner, self.bias_name = int(shared_inner), bias_name
        self.w_router = self.b_router = self.w_gu = self.wd = self.ws_up = self.ws_down = None

    def tensor_specs(self, prefix):
        E, F = self.width, self.inner
        # the router stays float32 (its logits decide which experts run)
        specs = [TensorSpec(prefix + ".router", (self.n_experts, E), VECTOR)]
        if self.router_bias:
            specs.append(TensorSpec(prefix + self.bias_name, (self.n_experts,), VECTOR))
        for e in range(self.n_experts):
            if self.gated:
                specs.append(TensorSpec(f"{prefix}.e{e}.gate", (F, E)))
            specs += [TensorSpec(f"{prefix}.e{e}.up", (F, E)), TensorSpec(f"{prefix}.e{e}.down", (E, F))]
        if self.shared_inner:
            specs += [TensorSpec(prefix + ".shared.up", (self.shared_inner, E)), TensorSpec(prefix + ".shared.down", (E, self.shared_inner)),
                      TensorSpec(prefix + ".shared.sg", (1, E), VECTOR)]
        return specs

    def bind(self, prefix, tensors, rt):
        self.w_router = tensors[prefix + ".router"].contiguous()
        self.b_router = tensors[prefix + self.bias_name] if self.router_bias else None
        if self.shared_inner:
            # the shared expert's gate is one more row of the router's product
            self.w_router = torch.cat([self.w_router, tensors[prefix + ".shared.sg"].reshape(1, self.width).float()], dim=0).contiguous()
            self.ws_up, self.ws_down = tensors[prefix + ".shared.up"], tensors[prefix + ".shared.down"]
        if self.gated:
            # gate and up of an expert as one matrix [2 F, E], the gate row of a feature followed by its up row: a product's
            # epilogue, and a warp of the row form, then has both of a feature
            first = lambda e: torch.stack([tensors[f"{prefix}.e{e}.gate"], tensors[f"{prefix}.e{e}.up"]], dim=1).reshape(2 * self.inner, self.width)
        else:
            first = lambda e: tensors[f"{prefix}.e{e}.up"]
        self.w_gu = torch.stack([first(e) for e in range(self.n_experts)], dim=0).contiguous()
        self.wd = torch.stack([tensors[f"{prefix}.e{e}.down"] for e in range(self.n_experts)], dim=0).contiguous()
        for e in range(self.n_experts):      # the stacked copies are what runs
            for name in ("gate", "up", "down"):
                tensors.pop(f"{prefix}.e{e}.{name}", None)

    def first_weights(self):
        return [self.w_router]

    def forward(self, rt, h):
        also = also_w = None
        if self.shared_inner:
            ids, wts, also_w = ops.moe_router(h, self.w_router, self.b_router, self.top, self.router, self.route_scale, n_extra=1)
            if rt.fused_swiglu(h, self.ws_up):        # the product's epilogue applies the activation
                act = ops.gemm_bf16_relu_sq(h, self.ws_up, None, rt.status)
            else:
                act = ops.relu_sq(rt.linear(h, self.ws_up))
            also = rt.linear(act, self.ws_down, out_dtype=torch.float32)
        else:
            ids, wts = ops.moe_router(h, self.w_router, self.b_router, self.top, self.router, self.route_scale)
        return rt.moe_experts(h, ids, wts, self.w_gu, self.wd, gated=self.gated, also=also, also_w=also_w)


register_part("feed_forward", "routed_experts", RoutedExperts)
