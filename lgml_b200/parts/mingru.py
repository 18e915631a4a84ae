"""minGRU as a mixer: a gated recurrence per channel whose gates read only the current token.

    z_t   = sigmoid(W_z h_t + b_z)                      how much of the state is replaced
    u_t   = W_x h_t + b_x;   c_t = u_t + 1/2 (u_t >= 0),  sigmoid(u_t) (u_t < 0)      the candidate
    S_t   = (1 - z_t) S_(t-1) + z_t c_t                 element by element, S_(-1) = 0
    out_t = W_o (S_t * silu(W_g h_t))

Because neither gate reads the state, the three projections of a whole portion are one product, and
the recurrence itself is a scan over float32 numbers: sequential per channel for short portions, in
pieces that run side by side for long ones (S at a piece's end is a S_start + b with a = prod (1 - z)
and b the piece's scan from zero).  A request carries S, float32, in its state slot.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import FixedState
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part

# portions of a request longer than this run in pieces side by side
MINGRU_PIECES_FROM = 64


class MinGRU(Part):
    graph_safe = True

    def __init__(self, width: int, inner: int):
        self.width, self.inner = width, inner
        self.w_in = self.b_in = self.wo = None

    def cache_spec(self):
        return FixedState((self.inner,), torch.float32)

    def tensor_specs(self, prefix):
        E, W = self.width, self.inner
        return [TensorSpec(prefix + ".z", (W, E)), TensorSpec(prefix + ".z.b", (W,), VECTOR), TensorSpec(prefix + ".x", (W, E)),
                TensorSpec(prefix + ".x.b", (W,), VECTOR), TensorSpec(prefix + ".g", (W, E)), TensorSpec(prefix + ".o", (E, W))]

    def bind(self, prefix, tensors, rt):
        t = lambda n: tensors[prefix + n]
        self.w_in = torch.cat([t(".z"), t(".x"), t(".g")], dim=0).contiguous()
        self.b_in = torch.cat([t(".z.b").float(), t(".x.b").float(), torch.zeros_like(t(".z.b"), dtype=torch.float32)]).contiguous()
        self.wo = t(".o")

    def first_weights(self):
        return [self.w_in]

    def forward(self, rt, h, batch, cache):
        proj = rt.linear(h, self.w_in, bias=self.b_in, out_dtype=torch.float32)         # [tokens, z | u | g]
        out = torch.empty((h.shape[0], self.inner), dtype=rt.dtype, device=h.device)
        chunks = chunk_start = None
        if batch.max_q_len > MINGRU_PIECES_FROM:
            chunks, chunk_start = batch.scan_pieces(ops.mingru_chunk_tokens())
        ops.mingru_scan(proj, cache.state, batch.seq_start, batch.slots, out, chunks, chunk_start)
        return rt.linear(out, self.wo, partials_ok=True)


register_part("mixer", "mingru", MinGRU)
