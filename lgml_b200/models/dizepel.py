"""The Dizepel decoder: which parts a ``DizepelConfig`` asks for, layer by layer.

The embedding's rows times ``embedding.scale`` are the residual stream x.  Every layer norms what a sublayer
reads and what it adds (layer norms with a weight and no bias): x += norm1b(mixer(conv(norm1(x)))), then, unless
its ``mlp`` is null, x += norm2b(ff(conv(norm2(x)))); ``conv`` adds a short causal convolution over time of the
normed rows to them (``parts/token_mix.py``: ``InputConv``).  The mixer is two mixers side by side on the same
input (``parts/parallel.py``): attention whose values are its keys, with a short convolution on q and k, partly
rotated heads, capped scores and a sink; and a selective state-space recurrence; half the sum of their
unit-normed results.  The feed-forward is two matrices around a polynomial of normed powers
(``parts/mlp.py``: ``PolyNormMLP``).

``loop`` runs a range of layers several times with the same weights; every run of a layer is a schedule entry
with a cache and state of its own, and the first layer of pass t first adds row t of ``loop.step`` to x.

Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``,
``l<i>.canon1``, ``l<i>.canon2``, ``l<i>.mix.left.*``, ``l<i>.mix.right.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import torch

from ..config import DizepelConfig, register_architecture
from ..parts import LMHead, TokenEmbedding, make_part
from .decoder import DecoderModel, LayerCall


def mixer_of(cfg: DizepelConfig, layer: dict):
    left, right = layer["mixer"]["left"], layer["mixer"]["right"]
    rot = left["rot"]
    attention = make_part("mixer", "conv_attention", width=cfg.width, n_heads=left["heads"], n_kv_heads=left["kv_heads"], head_dim=left["dim"],
                          v_head_dim=left["vdim"], taps=left["conv"], scale=left["scale"], softcap=left.get("softcap"), rope_base=rot["base"],
                          rope_dims=rot["dims"], rope_scaling=rot.get("scaling"), sink=True)
    recurrence = make_part("mixer", "state_space_dual", width=cfg.width, n_heads=right["heads"], head_dim=right["vdim"], n_state=right["state"],
                           n_groups=right["groups"], taps=right["conv"], norm_groups=right["norm_groups"], eps=cfg.norm_eps)
    return make_part("mixer", "parallel", width=cfg.width, left=attention, right=recurrence, eps=cfg.norm_eps)


def feed_forward_of(cfg: DizepelConfig, mlp):
    if mlp is None:
        return None
    return make_part("feed_forward", "polynorm_mlp", width=cfg.width, inner=mlp["ff"], eps=cfg.norm_eps)


def build_dizepel(cfg: DizepelConfig) -> DecoderModel:
    norm = lambda: make_part("norm", "layernorm", width=cfg.width, eps=cfg.norm_eps)
    conv = lambda: make_part("token_input", "input_conv", width=cfg.width, taps=cfg.canon_taps) if cfg.canon_taps else None
    blocks = []
    for layer in cfg.layers:
        ffn = feed_forward_of(cfg, layer.get("mlp"))
        blocks.append(make_part("block", "sandwich", mixer_norm=norm(), mixer_post=norm(), mixer=mixer_of(cfg, layer),
                                ffn_norm=norm() if ffn else None, ffn_post=norm() if ffn else None, ffn=ffn,
                                mixer_conv=conv(), ffn_conv=conv() if ffn else None))
    schedule = [LayerCall(i, add_row=t) for i, t in cfg.layer_runs()]
    embedding = TokenEmbedding(cfg.vocab, cfg.width, name="embed")
    head = LMHead(cfg.vocab, cfg.width, name="head")
    return DecoderModel(cfg, embedding, blocks, norm(), head, schedule=schedule, block_prefix="l{}", final_norm_prefix="final.norm",
                        embed_scale=cfg.embed_scale if cfg.embed_scale != 1.0 else None, delta_dtype=torch.float32, pass_rows="loop.step")


register_architecture("Dizepel", DizepelConfig, build_dizepel)
