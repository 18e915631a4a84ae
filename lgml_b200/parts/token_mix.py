"""Two small parts that sit around a layer's mixer and feed-forward.

``TokenShift``: what the mixer reads moves towards the previous token's, per channel:

    y_t = h_t + (h_(t-1) - h_t) * mu          h_(-1) = 0; h_(t-1) is the unshifted row

The last h of a step waits, float32, in the request's state slot for the next step.  The part takes
float32 rows (the norm before it writes them so) and gives rows in the compute type.

``TokenSide``: what a layer adds from its own slice of a table indexed by the token's id:

    e = table[token, col0 : col0 + dim];   y = W_proj (gelu_tanh(W_gate x) * e);   x += m y / rms(y) * w

x is the residual stream itself (not a norm of it).  For a few tokens one kernel does all of it
(and the residual sum before it); for many, in bfloat16, the two products run as matrix products.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import FixedState
from ..weights import MATRIX, VECTOR, TensorSpec
from .base import Part, register_part

# tokens of a step from which the token input's two products run as matrix products
SIDE_PRODUCTS_FROM = 64


class TokenShift(Part):
    graph_safe = True
    input_dtype = torch.float32

    def __init__(self, width: int):
        self.width = width
        self.mu = None

    def cache_spec(self):
        return FixedState((self.width,), torch.float32)

    def tensor_specs(self, prefix):
        return [TensorSpec(prefix, (self.width,), VECTOR, init=(0.5, 5.0))]

    def bind(self, prefix, tensors, rt):
        self.mu = tensors[prefix]

    def forward(self, rt, h, batch, state):
        out = torch.empty(h.shape, dtype=rt.dtype, device=h.device)
        return ops.token_shift(h, self.mu, state, batch.seq_of_token, batch.seq_start, batch.slots, out)


class TokenSide(Part):
    graph_safe = True

    def __init__(self, width: int, dim: int, vocab: int, table_name: str, table_cols: int, col0: int, eps: float):
        if col0 < 0 or col0 + dim > table_cols:
            raise ValueError(f"columns {col0} .. {col0 + dim - 1} are outside a table of {table_cols}")
        self.width, self.dim, self.vocab = width, dim, vocab
        self.table_name, self.table_cols, self.col0, self.eps = table_name, table_cols, col0, float(eps)
        self.table = self.w_gate = self.w_proj = self.norm_w = None

    def tensor_specs(self, prefix):
        return [TensorSpec(self.table_name, (self.vocab, self.table_cols), MATRIX), TensorSpec(prefix + ".gate", (self.dim, self.width)),
                TensorSpec(prefix + ".proj", (self.width, self.dim)), TensorSpec(prefix + ".norm", (self.width,), VECTOR, init=(1.0, 1.0))]

    def bind(self, prefix, tensors, rt):
        self.table = tensors[self.table_name]
        self.w_gate, self.w_proj, self.norm_w = tensors[prefix + ".gate"], tensors[prefix + ".proj"], tensors[prefix + ".norm"]

    def forward(self, rt, x, pending, scale, batch):
        """x += scale * pending, then x += scale * (the token input's normed output); all in place."""
        n = x.shape[0]
        if n < SIDE_PRODUCTS_FROM or rt.dtype == torch.float32:      # float32: one order of summation whatever the step holds
            return ops.token_side(x, pending, scale, batch.token_ids, self.table, self.col0, self.w_gate, self.w_proj, self.norm_w, self.eps, scale)
        xb = ops.residual_fold(x, pending, scale, copy_dtype=rt.dtype if rt.dtype != torch.float32 else None)
        gate = rt.linear(x if xb is None else xb, self.w_gate, out_dtype=torch.float32)
        g = ops.side_gate(gate, batch.token_ids, self.table, self.col0, rt.dtype)
        y = rt.linear(g, self.w_proj, out_dtype=torch.float32)
        return ops.side_add(x, y, self.norm_w, self.eps, scale)


class InputConv(Part):
    """What a sublayer reads gains a causal convolution of itself over time, per channel:

        y_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j)        zeros before a request's start

    The tensor is [width, taps]; its last column weighs the current row.  The last taps - 1 rows of h wait,
    float32, in the request's state slot.  Takes float32 rows (the norm before it writes them so) and gives
    rows in the compute type."""

    graph_safe = True
    input_dtype = torch.float32

    def __init__(self, width: int, taps: int):
        if not 1 <= taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"a convolution of {taps} taps (1 to {ops.CONV_MAX_TAPS})")
        self.width, self.taps = width, int(taps)
        self.w_t = None

    def cache_spec(self):
        return FixedState(((self.taps - 1) * self.width,), torch.float32) if self.taps > 1 else None

    def tensor_specs(self, prefix):
        return [TensorSpec(prefix, (self.width, self.taps), VECTOR, init=(0.0, 10.0))]

    def bind(self, prefix, tensors, rt):
        self.w_t = tensors[prefix].float().t().contiguous()

    def forward(self, rt, h, batch, state):
        out = torch.empty(h.shape, dtype=rt.dtype, device=h.device)
        return ops.short_conv(h, self.w_t, None, state, batch.seq_of_token, batch.seq_start, batch.slots, out, residual=True)


register_part("token_input", "token_shift", TokenShift)
register_part("token_input", "input_conv", InputConv)
register_part("token_input", "token_side", TokenSide)
