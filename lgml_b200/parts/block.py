"""The arrangement of a layer's parts.

``PreNormBlock`` is the Llama layer (``lua/lgml/transformer.lua:2312-2345``):
x = x + mixer(norm(x)); x = x + ffn(norm(x)).  The residual stream x stays
float32 and every sum into it is a float32 add.  A sum and the norm that follows
it are one kernel, so a block hands its last delta on as ``pending`` and the next
norm (the next block's, or the model's final norm) adds it.

Three things a layer may have on top, each absent by default:

* ``residual_scale`` m: x = x + m * mixer(..), x = x + m * ffn(..);
* ``shift``: a part between the first norm and the mixer that mixes every row with the row of the
  token before it (``parts/token_mix.py``); it keeps that row in the request's state slot, so the
  layer's cache then holds the shift's floats first and the mixer's own state behind them;
* ``side``: a part after the feed-forward that adds something of the token itself to x.  It also adds
  the pending delta, so a block with it hands nothing on.
"""
from __future__ import annotations

import dataclasses

from .. import ops
from ..cache import FixedState
from .base import Part, register_part


class PreNormBlock(Part):
    def __init__(self, mixer_norm, mixer, ffn_norm, ffn, names=None, residual_scale: float = 1.0, shift=None, side=None):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.shift, self.side = shift, side
        self.residual_scale = float(residual_scale)
        # tensor-name stems of the parts under the layer's prefix
        self.names = {"mixer_norm": "input_layernorm", "mixer": "self_attn", "ffn_norm": "post_attention_layernorm", "ffn": "mlp",
                      "shift": "shift", "side": "side"}
        self.names.update(names or {})
        if shift is not None and mixer is None:
            raise ValueError("a shift needs a mixer to feed")

    def _parts(self, prefix):
        for key in ("mixer_norm", "shift", "mixer", "ffn_norm", "ffn", "side"):
            part = getattr(self, key)
            if part is not None:
                yield part, f"{prefix}.{self.names[key]}"

    def tensor_specs(self, prefix):
        return [s for part, p in self._parts(prefix) for s in part.tensor_specs(p)]

    def bind(self, prefix, tensors, rt):
        for part, p in self._parts(prefix):
            part.bind(p, tensors, rt)

    def cache_spec(self):
        own = self.mixer.cache_spec() if self.mixer is not None else None
        if self.shift is None:
            return own
        first = self.shift.cache_spec()
        if own is None:
            return first
        if isinstance(own, FixedState):
            if len(own.shape) != 1 or own.dtype != first.dtype:
                raise TypeError(f"a shift shares a state slot only with a mixer whose state is one row of {first.dtype}, not {own}")
            return FixedState((first.shape[0] + own.shape[0],), first.dtype)
        return (own, first)

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in (self.mixer_norm, self.shift, self.mixer, self.ffn_norm, self.ffn, self.side)
                   if p is not None)

    def forward(self, rt, x, pending, batch, cache):
        m = self.residual_scale
        scaled = {"delta_scale": m} if m != 1.0 else {}
        if self.mixer is not None:
            if self.shift is None:
                h = self.mixer_norm.forward(rt, x, rt.dtype, delta=pending, **scaled)
            else:
                n_shift = self.shift.cache_spec().shape[0]
                h = self.mixer_norm.forward(rt, x, self.shift.input_dtype, delta=pending, **scaled)
                h = self.shift.forward(rt, h, batch, cache.state[:, :n_shift])
                if cache.state.shape[1] > n_shift:
                    cache = dataclasses.replace(cache, state=cache.state[:, n_shift:])
            if self.ffn is not None:
                first = getattr(self.ffn, "first_weights", None)
                if first is not None:
                    rt.ahead(first())       # read after the mixer: L2 may fetch their head meanwhile
            pending = self.mixer.forward(rt, h, batch, cache)
        if self.ffn is not None:
            h = self.ffn_norm.forward(rt, x, rt.dtype, delta=pending, **scaled)
            pending = self.ffn.forward(rt, h)
        if self.side is not None:
            self.side.forward(rt, x, pending, m, batch)
            pending = None
        elif m != 1.0 and pending is not None:
            ops.residual_fold(x, pending, m)        # whoever adds a delta after this block knows no scale
            pending = None
        return x, pending


register_part("block", "pre_norm", PreNormBlock)
