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

import torch

from .. import ops
from ..cache import FixedState
from .base import Part, register_part
from .norm import PendingDelta


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


class SandwichBlock(Part):
    """A layer that norms what a sublayer reads and what it adds:

        x = x + post1(mixer(conv1(pre1(x))));   x = x + post2(ffn(conv2(pre2(x))))

    ``conv1`` / ``conv2`` (``parts/token_mix.py``: ``InputConv``) are optional.  A sum, the norm on what is added and the
    next norm on x are one kernel: the block hands its last result on as a ``PendingDelta`` with the weight of
    the norm it still has to pass, and the next norm (the next block's, or the model's final one, which must
    take such a delta) does both.  The layer's fixed state is one row per request: the convolutions' rows first,
    the mixer's own state behind them."""

    takes_pending_row = True

    def __init__(self, mixer_norm, mixer_post, mixer, ffn_norm, ffn_post, ffn, mixer_conv=None, ffn_conv=None, names=None):
        self.mixer_norm, self.mixer_post, self.mixer = mixer_norm, mixer_post, mixer
        self.ffn_norm, self.ffn_post, self.ffn = ffn_norm, ffn_post, ffn
        self.mixer_conv, self.ffn_conv = mixer_conv, ffn_conv
        self.names = {"mixer_norm": "norm1", "mixer_post": "norm1b", "mixer": "mix", "ffn_norm": "norm2", "ffn_post": "norm2b", "ffn": "mlp",
                      "mixer_conv": "canon1", "ffn_conv": "canon2"}
        self.names.update(names or {})
        if ffn is None and (ffn_norm is not None or ffn_post is not None or ffn_conv is not None):
            raise ValueError("a layer without a feed-forward has no norms or convolution for it")
        paged, own = None, 0
        spec = mixer.cache_spec()
        for sp in (spec if isinstance(spec, (tuple, list)) else (spec,)):
            if isinstance(sp, FixedState):
                if len(sp.shape) != 1 or sp.dtype != torch.float32:
                    raise TypeError(f"the layer's state slot holds rows of float32 only, not {sp}")
                own = sp.shape[0]
            elif sp is not None:
                paged = sp
        conv_floats = [c.cache_spec().shape[0] if c is not None and c.cache_spec() is not None else 0 for c in (mixer_conv, ffn_conv)]
        self._paged, self._floats = paged, (conv_floats[0], conv_floats[1], own)

    def _parts(self, prefix):
        for key in ("mixer_norm", "mixer_post", "mixer_conv", "mixer", "ffn_norm", "ffn_post", "ffn_conv", "ffn"):
            part = getattr(self, key)
            if part is not None:
                yield part, f"{prefix}.{self.names[key]}"

    def tensor_specs(self, prefix):
        return [s for part, p in self._parts(prefix) for s in part.tensor_specs(p)]

    def bind(self, prefix, tensors, rt):
        for part, p in self._parts(prefix):
            part.bind(p, tensors, rt)

    def cache_spec(self):
        total = sum(self._floats)
        both = tuple(s for s in (self._paged, FixedState((total,), torch.float32) if total else None) if s is not None)
        return both if len(both) > 1 else (both[0] if both else None)

    @property
    def graph_safe(self):
        return all(getattr(part, "graph_safe", False) for part, _ in self._parts(""))

    @staticmethod
    def _pend(delta, post):
        return PendingDelta(delta, post.weight, eps=post.eps) if post is not None else PendingDelta(delta)

    def forward(self, rt, x, pending, batch, cache):
        c1, c2, own = self._floats
        state = cache.state

        def read(norm, conv, first, floats, pend):
            if conv is None:
                return norm.forward(rt, x, rt.dtype, delta=pend)
            if batch.max_q_len == 1 and getattr(norm, "takes_pending", False):
                # one token a request: the norm's kernel adds the convolution itself
                return norm.forward(rt, x, rt.dtype, delta=pend, conv=(conv.w_t, state[:, first:first + floats] if floats else None, batch.slots))
            h = norm.forward(rt, x, conv.input_dtype, delta=pend)
            return conv.forward(rt, h, batch, state[:, first:first + floats] if floats else None)

        h = read(self.mixer_norm, self.mixer_conv, 0, c1, pending)
        if self.ffn is not None:
            first = getattr(self.ffn, "first_weights", None)
            if first is not None:
                rt.ahead(first())
        mixer_cache = dataclasses.replace(cache, state=state[:, c1 + c2:c1 + c2 + own] if own else None)
        pending = self._pend(self.mixer.forward(rt, h, batch, mixer_cache), self.mixer_post)
        if self.ffn is not None:
            h = read(self.ffn_norm, self.ffn_conv, c1, c2, pending)
            pending = self._pend(self.ffn.forward(rt, h), self.ffn_post)
        return x, pending


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "sandwich", SandwichBlock)
