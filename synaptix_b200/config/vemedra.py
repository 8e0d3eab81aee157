"""Typed configuration of the Vemedra decoder, read from its config.json.

Keys: ``architecture`` ("Vemedra"), ``vocab``, ``width``, ``norm.eps``, ``canon.taps`` (taps of the short convolution in
front of every sublayer), ``layers`` (a list; each entry has ``type``, the sizes of its mixer under ``mixer`` and its
feed-forward under ``mlp`` or ``null``) and ``loop`` (``start``, ``stop``, ``times``: layers ``start .. stop-1`` run
``times`` times in a row with the same weights).  Layer types:

* ``mingru``: ``mixer.width`` channels of a gated recurrence;
* ``parallel``: ``mixer.left`` (softmax attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap``,
  ``mask.size``, ``rot.dims``, ``rot.base``) beside ``mixer.right`` (retention: ``heads``, ``dim``, ``vdim``, ``decay``
  per head), added as ``left_scale * left + right_scale * right``.

Feed-forward: ``mlp.kind`` = ``dense`` with ``ff`` and ``limit``.  Every size and constant is taken from here; a key
that is required and missing, or a type or kind that is not known, is an error.  ``softcap``, ``mask`` and ``rot`` may be
absent or null: the attention then has no cap, no chunks, no rotation.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take


@dataclasses.dataclass(frozen=True)
class SoftmaxSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    chunk: Optional[int]
    rot_dims: Optional[int]
    rot_base: Optional[float]

    @classmethod
    def from_dict(cls, d, where):
        mask = d.get("mask") or {}
        rot = d.get("rot") or {}
        return cls(heads=take(d, "heads", int, where=where), kv_heads=take(d, "kv_heads", int, where=where),
                   dim=take(d, "dim", int, where=where), vdim=take(d, "vdim", int, where=where),
                   scale=take(d, "scale", float, where=where), softcap=take(d, "softcap", float, None, where=where),
                   chunk=take(mask, "size", int, None, where=where + ".mask"),
                   rot_dims=take(rot, "dims", int, None, where=where + ".rot"),
                   rot_base=take(rot, "base", float, None, where=where + ".rot"))

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        if self.rot_dims is not None:
            d["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        return d

    def validate(self, where):
        if min(self.heads, self.kv_heads, self.dim, self.vdim) <= 0 or self.heads % self.kv_heads:
            raise ConfigError(f"{where}: heads must be a positive multiple of kv_heads, dim and vdim positive")
        if self.chunk is not None and self.chunk <= 0:
            raise ConfigError(f"{where}: mask.size must be > 0")
        if self.rot_dims is not None:
            if self.rot_dims % 2 or not (0 < self.rot_dims <= self.dim) or self.rot_base is None or self.rot_base <= 0:
                raise ConfigError(f"{where}: rot.dims must be even and at most dim, rot.base positive")
        if self.softcap is not None and self.softcap <= 0:
            raise ConfigError(f"{where}: softcap must be > 0")


@dataclasses.dataclass(frozen=True)
class RetentionSpec:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @classmethod
    def from_dict(cls, d, where):
        decay = d.get("decay")
        if not isinstance(decay, list) or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
            raise ConfigError(f"{where}: 'decay' must be a list of numbers")
        return cls(heads=take(d, "heads", int, where=where), dim=take(d, "dim", int, where=where),
                   vdim=take(d, "vdim", int, where=where), decay=tuple(float(x) for x in decay))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}

    def validate(self, where):
        if min(self.heads, self.dim, self.vdim) <= 0 or len(self.decay) != self.heads:
            raise ConfigError(f"{where}: sizes must be positive, with one decay per head")


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    type: str
    mingru_width: Optional[int] = None
    left: Optional[SoftmaxSpec] = None
    right: Optional[RetentionSpec] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    ff: Optional[int] = None              # None: the layer has no feed-forward
    ff_kind: Optional[str] = None
    ff_limit: Optional[float] = None

    @classmethod
    def from_dict(cls, d, i):
        where = f"config.json: layers[{i}]"
        if not isinstance(d, dict):
            raise ConfigError(f"{where} must be an object")
        typ = take(d, "type", str, where=where)
        mixer = d.get("mixer")
        if not isinstance(mixer, dict):
            raise ConfigError(f"{where}: 'mixer' must be an object")
        kw: Dict[str, Any] = {}
        if typ == "mingru":
            kw["mingru_width"] = take(mixer, "width", int, where=where + ".mixer")
        elif typ == "parallel":
            for side in ("left", "right"):
                if not isinstance(mixer.get(side), dict):
                    raise ConfigError(f"{where}.mixer: '{side}' must be an object")
            kw["left"] = SoftmaxSpec.from_dict(mixer["left"], where + ".mixer.left")
            kw["right"] = RetentionSpec.from_dict(mixer["right"], where + ".mixer.right")
            kw["left_scale"] = take(mixer, "left_scale", float, where=where + ".mixer")
            kw["right_scale"] = take(mixer, "right_scale", float, where=where + ".mixer")
        else:
            raise ConfigError(f"{where}: unknown layer type {typ!r} (known: mingru, parallel)")
        mlp = d.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict):
                raise ConfigError(f"{where}: 'mlp' must be an object or null")
            kw["ff_kind"] = take(mlp, "kind", str, where=where + ".mlp")
            if kw["ff_kind"] != "dense":
                raise ConfigError(f"{where}.mlp: unknown kind {kw['ff_kind']!r} (known: dense)")
            kw["ff"] = take(mlp, "ff", int, where=where + ".mlp")
            kw["ff_limit"] = take(mlp, "limit", float, where=where + ".mlp")
        return cls(type=typ, **kw)

    def to_dict(self):
        if self.type == "mingru":
            mixer = {"width": self.mingru_width}
        else:
            mixer = {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                     "right_scale": self.right_scale}
        mlp = None if self.ff is None else {"kind": self.ff_kind, "ff": self.ff, "limit": self.ff_limit}
        return {"type": self.type, "mixer": mixer, "mlp": mlp}

    def validate(self, i):
        where = f"config.json: layers[{i}]"
        if self.type == "mingru":
            if self.mingru_width <= 0:
                raise ConfigError(f"{where}: mixer.width must be > 0")
        else:
            self.left.validate(where + ".mixer.left")
            self.right.validate(where + ".mixer.right")
        if self.ff is not None and (self.ff <= 0 or self.ff_limit <= 0):
            raise ConfigError(f"{where}.mlp: ff and limit must be > 0")


@dataclasses.dataclass(frozen=True)
class VemedraConfig(ModelConfig):
    architectures: ClassVar[Tuple[str, ...]] = ("Vemedra",)
    model_types: ClassVar[Tuple[str, ...]] = ("vemedra",)

    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    canon_taps: int = 1
    layers: Tuple[LayerSpec, ...] = ()
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    has_loop: bool = False

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VemedraConfig":
        norm, canon, loop = d.get("norm"), d.get("canon"), d.get("loop")
        if not isinstance(norm, dict) or not isinstance(canon, dict):
            raise ConfigError("config.json: 'norm' and 'canon' must be objects")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        kw = {}
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: 'loop' must be an object or null")
            kw = dict(loop_start=take(loop, "start", int, where="config.json: loop"),
                      loop_stop=take(loop, "stop", int, where="config.json: loop"),
                      loop_times=take(loop, "times", int, where="config.json: loop"), has_loop=True)
        cfg = cls(vocab=take(d, "vocab", int), width=take(d, "width", int),
                  norm_eps=take(norm, "eps", float, where="config.json: norm"),
                  canon_taps=take(canon, "taps", int, where="config.json: canon"),
                  layers=tuple(LayerSpec.from_dict(x, i) for i, x in enumerate(layers)), **kw)
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architectures[0], "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps},
             "layers": [x.to_dict() for x in self.layers]}
        if self.has_loop:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return d

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: vocab and width must be > 0")
        if self.norm_eps < 0 or self.canon_taps < 1:
            raise ConfigError("config.json: norm.eps must be >= 0 and canon.taps >= 1")
        for i, layer in enumerate(self.layers):
            layer.validate(i)
        if self.has_loop:
            if not (0 <= self.loop_start <= self.loop_stop <= len(self.layers)) or self.loop_times < 1:
                raise ConfigError("config.json: loop needs 0 <= start <= stop <= number of layers and times >= 1")

    # the order in which layers run: (layer, pass) with pass = the number of the loop's pass that the run opens, else None
    def runs(self):
        if not self.has_loop or self.loop_start == self.loop_stop:
            return [(i, None) for i in range(len(self.layers))]
        out = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            out += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, None) for i in range(self.loop_stop, len(self.layers))]
