"""The Konovik decoder: which parts a ``KonovikConfig`` asks for, layer by layer.

The embedding's rows go through the model's norm; that is the residual stream x.  Every layer is
pre-norm with a residual multiplier m: x += m * mixer(shift(norm1(x))), then, unless its ``mlp`` is
null, x += m * ff(norm2(x)), then the layer's token input (``parts/token_mix.py``).  Every norm of
the model is an RMS norm whose weight is one number.  The mixer is chosen per layer by ``type``:
``mingru`` (``parts/mingru.py``) or ``latent_attention`` (``parts/latent_attention.py``, with a
sliding window, stretched rotary frequencies and an output gate); what it reads is first mixed with
the previous token's (``TokenShift``).  The feed-forward is the gated one with SiLU (``dense``) or a
mixture of experts (``moe``): sigmoid scores, a correction on the choice, experts with a squared relu
and no gate, a shared expert behind a gate of its own.

``loop`` runs a range of layers several times with the same weights; every run of a layer is a
schedule entry with a cache and state of its own, and before the first layer of every pass but
the first the model's input (x before layer 0) is added to x.  A looped layer's token input reads
the same slice of the table in every pass.

Tensor names: ``embed``, ``embed.norm``, ``side.embed``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import torch

from ..config import KonovikConfig, register_architecture
from ..parts import LMHead, TokenEmbedding, make_part
from .decoder import DecoderModel, LayerCall

NAMES = {"mixer_norm": "norm1", "mixer": "mix", "ffn_norm": "norm2", "ffn": "mlp", "shift": "shift", "side": "side"}


def mixer_of(cfg: KonovikConfig, layer: dict):
    m = layer["mixer"]
    if layer["type"] == "mingru":
        return make_part("mixer", "mingru", width=cfg.width, inner=m["width"])
    mask = m.get("mask")
    return make_part("mixer", "latent_attention", width=cfg.width, n_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                     v_head_dim=m["vdim"], rank=m["kv_rank"], scale=m["scale"], eps=cfg.norm_eps, rope_base=m["rot"]["base"],
                     rope_dims=m["rot"]["dims"], rope_scaling=m["rot"].get("scaling"), window=mask["size"] if mask else None, out_gate=True)


def feed_forward_of(cfg: KonovikConfig, mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return make_part("feed_forward", "gated_mlp", width=cfg.width, inner=mlp["ff"], names=(".gate", ".up", ".down"))
    shared = mlp.get("shared")
    return make_part("feed_forward", "routed_experts", width=cfg.width, inner=mlp["expert"]["ff"], n_experts=mlp["router"]["experts"],
                     top=mlp["router"]["top"], router="sigmoid", route_scale=mlp["router"].get("scale", 1.0), gated=False,
                     shared_inner=shared["ff"] if shared else 0, bias_name=".correction")


def build_konovik(cfg: KonovikConfig) -> DecoderModel:
    norm = lambda: make_part("norm", "rmsnorm", width=cfg.width, eps=cfg.norm_eps, suffix="", single=True)
    n = len(cfg.layers)
    blocks = []
    for i, layer in enumerate(cfg.layers):
        ffn = feed_forward_of(cfg, layer.get("mlp"))
        side = None
        if cfg.side_dim:
            side = make_part("token_input", "token_side", width=cfg.width, dim=cfg.side_dim, vocab=cfg.vocab, table_name="side.embed",
                             table_cols=n * cfg.side_dim, col0=i * cfg.side_dim, eps=cfg.norm_eps)
        blocks.append(make_part("block", "pre_norm", mixer_norm=norm(), mixer=mixer_of(cfg, layer), ffn_norm=norm() if ffn else None, ffn=ffn,
                                names=NAMES, residual_scale=cfg.residual_mult, shift=make_part("token_input", "token_shift", width=cfg.width),
                                side=side))
    schedule = [LayerCall(i, add_input=again) for i, again in cfg.layer_runs()]
    embedding = TokenEmbedding(cfg.vocab, cfg.width, name="embed")
    head = LMHead(cfg.vocab, cfg.width, name="head")
    return DecoderModel(cfg, embedding, blocks, norm(), head, schedule=schedule, block_prefix="l{}", final_norm_prefix="final.norm",
                        embed_norm=norm(), embed_norm_prefix="embed.norm", delta_dtype=torch.float32)


register_architecture("Konovik", KonovikConfig, build_konovik)
