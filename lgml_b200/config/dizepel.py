"""Configuration of the Dizepel decoder, from its own ``config.json`` keys.

``architecture`` names it; ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (the factor on the embedding's
rows; absent: 1) and ``canon.taps`` (the taps of the convolution on what every sublayer reads; absent: none)
are the model's own numbers.  ``layers`` lists the layers one by one: ``type`` (the mixer: ``parallel``), ``mixer``
(its sizes and constants) and ``mlp`` (the feed-forward, or null for a layer without one).  ``loop`` (``start``,
``stop``, ``times``): layers start .. stop - 1 run ``times`` times in a row with the same weights; every pass adds
its own row of the tensor ``loop.step`` to the residual stream first.

parallel ``mixer``: two sides.  ``left``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps of the
convolution on q and k), ``scale``, ``softcap`` (absent or 0: none), ``rot.base`` / ``rot.dims`` / ``rot.scaling``
(``factor``, ``original``, ``fast``, ``slow``; absent: the plain frequencies).  ``right``: ``heads``, ``vdim``,
``state``, ``groups``, ``conv``, ``norm_groups``.

``mlp``: ``kind`` ``dense`` with ``ff``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, ModelConfig
from .gotulorn import _number, _positive_int

MIXERS = ("parallel",)
MLP_KINDS = ("dense",)


@dataclass
class DizepelConfig(ModelConfig):
    architecture: str = "Dizepel"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    embed_scale: float = 1.0
    canon_taps: int = 0                    # 0: no convolution on what the sublayers read
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

    def layer_runs(self) -> List[Tuple[int, Optional[int]]]:
        """The layers in the order in which they run, as (layer, the number of the pass of the loop that this run
        starts, or None)."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop
        runs: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(a)]
        for r in range(times):
            runs += [(i, r if i == a else None) for i in range(a, b)]
        return runs + [(i, None) for i in range(b, n)]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DizepelConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json: '{key}' is missing")
        norm = d["norm"]
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        if not isinstance(d["layers"], list):
            raise ConfigError("config.json: 'layers' must be a list")
        emb, canon = d.get("embedding"), d.get("canon")
        for key, v in (("embedding", emb), ("canon", canon)):
            if v is not None and not isinstance(v, dict):
                raise ConfigError(f"config.json: '{key}' must be an object")
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
                   embed_scale=float(_number("embedding", emb, "scale")) if emb and "scale" in emb else 1.0,
                   canon_taps=_positive_int("canon", canon, "taps") if canon is not None else 0,
                   loop=loop, layers=copy.deepcopy(d["layers"]), torch_dtype=str(d.get("torch_dtype", "bfloat16")))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        if not 0 <= self.canon_taps <= 8:
            raise ConfigError(f"config.json: canon.taps must be 1 to 8, not {self.canon_taps}")
        if self.loop is not None:
            a, b, times = self.loop
            if not (0 <= a < b <= len(self.layers)) or times < 1:
                raise ConfigError(f"config.json: loop must name layers start < stop <= {len(self.layers)} and times >= 1, not {self.loop}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"config.json: {where}.type must be one of {MIXERS}, not {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict) or not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object with 'left' and 'right'")
            lw, left = where + ".mixer.left", m["left"]
            for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
                _positive_int(lw, left, key)
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"config.json: {lw}.heads {left['heads']} is no multiple of kv_heads {left['kv_heads']}")
            if left["vdim"] > left["dim"]:
                raise ConfigError(f"config.json: {lw}.vdim {left['vdim']} is more than dim {left['dim']}: the values are the keys")
            if left["conv"] > 8:
                raise ConfigError(f"config.json: {lw}.conv must be at most 8")
            _number(lw, left, "scale")
            if left.get("softcap") is not None and not _number(lw, left, "softcap") >= 0:
                raise ConfigError(f"config.json: {lw}.softcap must not be negative")
            rot = left.get("rot")
            if not isinstance(rot, dict):
                raise ConfigError(f"config.json: {lw}.rot must be an object with 'base' and 'dims'")
            _number(lw + ".rot", rot, "base")
            dims = _positive_int(lw + ".rot", rot, "dims")
            if dims % 2 or dims > left["dim"]:
                raise ConfigError(f"config.json: {lw}.rot.dims {dims} must be even and at most dim {left['dim']}")
            sc = rot.get("scaling")
            if sc is not None:
                if not isinstance(sc, dict):
                    raise ConfigError(f"config.json: {lw}.rot.scaling must be an object")
                for key in ("factor", "original", "fast", "slow"):
                    if not _number(lw + ".rot.scaling", sc, key) > 0:
                        raise ConfigError(f"config.json: {lw}.rot.scaling.{key} must be positive")
            rw, right = where + ".mixer.right", m["right"]
            for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                _positive_int(rw, right, key)
            if right["heads"] % right["groups"]:
                raise ConfigError(f"config.json: {rw}.heads {right['heads']} is no multiple of groups {right['groups']}")
            if (right["heads"] * right["vdim"]) % right["norm_groups"]:
                raise ConfigError(f"config.json: {rw}.norm_groups {right['norm_groups']} does not divide heads x vdim")
            if right["conv"] > 8 or right["state"] > 1024:
                raise ConfigError(f"config.json: {rw}.conv must be at most 8 and state at most 1024")
            mlp = layer.get("mlp")
            if mlp is not None:
                fw = where + ".mlp"
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: {fw}.kind must be one of {MLP_KINDS}")
                _positive_int(fw, mlp, "ff")

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embed_scale}, "layers": copy.deepcopy(self.layers)}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d
