"""Configuration of the Konovik decoder, from its own ``config.json`` keys.

``architecture`` names it; ``vocab``, ``width``, ``norm.eps`` and ``residual_mult`` (the factor on
everything a layer adds to the residual stream; absent: 1) are the model's own numbers; ``layers``
lists the layers one by one: ``type`` (the mixer: ``mingru`` or ``latent_attention``), ``mixer`` (its
sizes and constants) and ``mlp`` (the feed-forward, or null for a layer without one).  ``loop``
(``start``, ``stop``, ``times``): layers start .. stop - 1 run ``times`` times in a row with the same
weights.  ``token_side.dim``: the width of each layer's slice of the per-layer token table (absent:
no such input).

mingru ``mixer``: ``width`` (the recurrence's channels).

latent_attention ``mixer``: ``heads``, ``dim`` (unrotated per head), ``rot_dim`` (rotated, shared by
the heads on the key side), ``vdim``, ``kv_rank``, ``scale``, ``rot.base`` / ``rot.dims``,
``rot.scaling`` (``factor``, ``original``, ``fast``, ``slow``; absent: the plain frequencies),
``mask.size`` (the window; absent: every earlier token).

``mlp``: ``kind`` ``dense`` with ``ff``, or ``moe`` with ``expert.ff``, ``router.experts``,
``router.top``, ``router.scale`` (absent: 1) and ``shared.ff`` (a shared expert; absent: none).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, ModelConfig
from .gotulorn import _number, _positive_int

MIXERS = ("mingru", "latent_attention")
MLP_KINDS = ("dense", "moe")


@dataclass
class KonovikConfig(ModelConfig):
    architecture: str = "Konovik"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    residual_mult: float = 1.0
    side_dim: int = 0                      # 0: no per-layer token input
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)
    layers: List[Dict[str, Any]] = field(default_factory=list)
    torch_dtype: str = "bfloat16"

    # the names other parts of the engine ask a configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def layer_runs(self) -> List[Tuple[int, bool]]:
        """The layers in the order in which they run, as (layer, is it the first layer of a pass of the
        loop after the first pass?)."""
        n = len(self.layers)
        if not self.loop:
            return [(i, False) for i in range(n)]
        a, b, times = self.loop
        runs = [(i, False) for i in range(a)]
        for r in range(times):
            runs += [(i, r > 0 and i == a) for i in range(a, b)]
        return runs + [(i, False) for i in range(b, n)]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KonovikConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json: '{key}' is missing")
        norm = d["norm"]
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        if not isinstance(d["layers"], list):
            raise ConfigError("config.json: 'layers' must be a list")
        side = d.get("token_side")
        if side is not None and not isinstance(side, dict):
            raise ConfigError("config.json: 'token_side' must be an object with 'dim'")
        loop = d.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: 'loop' must be an object with 'start', 'stop' and 'times'")
            for key in ("start", "stop", "times"):
                v = loop.get(key)
                if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                    raise ConfigError(f"config.json: loop.{key} must be a non-negative integer, not {v!r}")
            loop = (loop["start"], loop["stop"], loop["times"])
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(norm["eps"]),
                   residual_mult=float(d.get("residual_mult", 1.0)), side_dim=_positive_int("token_side", side, "dim") if side else 0,
                   loop=loop, layers=copy.deepcopy(d["layers"]), torch_dtype=str(d.get("torch_dtype", "bfloat16")))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        if self.loop is not None:
            a, b, times = self.loop
            if not (0 <= a < b <= len(self.layers)) or times < 1:
                raise ConfigError(f"config.json: loop must name layers start < stop <= {len(self.layers)} and times >= 1, not {self.loop}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"config.json: {where}.type must be one of {MIXERS}, not {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            mw = where + ".mixer"
            if layer["type"] == "mingru":
                _positive_int(mw, m, "width")
            else:
                for key in ("heads", "dim", "vdim", "rot_dim", "kv_rank"):
                    _positive_int(mw, m, key)
                _number(mw, m, "scale")
                rot = m.get("rot")
                if not isinstance(rot, dict):
                    raise ConfigError(f"config.json: {mw}.rot must be an object with 'base' and 'dims'")
                _number(mw + ".rot", rot, "base")
                dims = _positive_int(mw + ".rot", rot, "dims")
                if dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"config.json: {mw}.rot.dims {dims} must be even and at most rot_dim {m['rot_dim']}")
                sc = rot.get("scaling")
                if sc is not None:
                    if not isinstance(sc, dict):
                        raise ConfigError(f"config.json: {mw}.rot.scaling must be an object")
                    for key in ("factor", "original", "fast", "slow"):
                        if not _number(mw + ".rot.scaling", sc, key) > 0:
                            raise ConfigError(f"config.json: {mw}.rot.scaling.{key} must be positive")
                if m.get("mask") is not None:
                    _positive_int(mw + ".mask", m["mask"], "size")
            mlp = layer.get("mlp")
            if mlp is not None:
                fw = where + ".mlp"
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: {fw}.kind must be one of {MLP_KINDS}")
                if mlp["kind"] == "dense":
                    _positive_int(fw, mlp, "ff")
                else:
                    _positive_int(fw + ".expert", mlp.get("expert"), "ff")
                    n = _positive_int(fw + ".router", mlp.get("router"), "experts")
                    top = _positive_int(fw + ".router", mlp.get("router"), "top")
                    if top > n:
                        raise ConfigError(f"config.json: {fw}.router.top {top} is more than its {n} experts")
                    if "scale" in mlp["router"]:
                        _number(fw + ".router", mlp["router"], "scale")
                    if mlp.get("shared") is not None:
                        _positive_int(fw + ".shared", mlp["shared"], "ff")

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult, "layers": copy.deepcopy(self.layers)}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d
