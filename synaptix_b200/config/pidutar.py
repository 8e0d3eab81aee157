"""Typed configuration of the Pidutar decoder, read from its config.json.

Keys: ``architecture`` ("Pidutar"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (the embedding's rows are
multiplied by it), ``residual_mult`` (a layer adds this multiple of its branches' sum to the stream), ``logit_scale``
(the output head's results are multiplied by it) and ``layers`` (a list; each entry has ``type``, the sizes of its
mixer under ``mixer`` and its feed-forward under ``mlp`` or ``null``).  Layer types:

* ``mlstm``: a matrix memory per head with exponential gates: ``heads``, ``dim`` (queries and keys), ``vdim`` (values),
  ``gate_cap`` (the gates' pre-activations are capped by ``cap * tanh(. / cap)``);
* ``latent_attention``: softmax attention whose keys and values are made from a cached latent: ``heads``, ``dim``
  (unrotated query/key elements a head), ``rot_dim`` (rotated ones, the key's shared by all heads), ``vdim``,
  ``q_rank`` and ``kv_rank`` (sizes of the two latents), ``scale``, ``mask.size`` (a sliding window; absent: every
  earlier key is seen), ``rot.dims`` / ``rot.base`` (pairs of neighbouring elements rotated; absent: no rotation) and
  ``kv_from`` (the layer has no key/value latent of its own and reads the cache of that earlier layer).

Feed-forward: ``mlp.kind`` = ``moe`` with ``expert.ff``, ``router.experts``, ``router.top``, ``router.scale``.  Every
size and constant is taken from here; a key that is required and missing, or a type or kind that is not known, is an
error.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take


@dataclasses.dataclass(frozen=True)
class MatrixMemorySpec:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, d, where):
        return cls(heads=take(d, "heads", int, where=where), dim=take(d, "dim", int, where=where),
                   vdim=take(d, "vdim", int, where=where), gate_cap=take(d, "gate_cap", float, where=where))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}

    def validate(self, where):
        if min(self.heads, self.dim, self.vdim) <= 0 or self.gate_cap <= 0:
            raise ConfigError(f"{where}: heads, dim, vdim and gate_cap must be > 0")


@dataclasses.dataclass(frozen=True)
class LatentAttentionSpec:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot_dims: Optional[int]
    rot_base: Optional[float]
    kv_from: Optional[int]

    @classmethod
    def from_dict(cls, d, where):
        mask = d.get("mask") or {}
        rot = d.get("rot") or {}
        return cls(heads=take(d, "heads", int, where=where), dim=take(d, "dim", int, where=where),
                   rot_dim=take(d, "rot_dim", int, where=where), vdim=take(d, "vdim", int, where=where),
                   q_rank=take(d, "q_rank", int, where=where), kv_rank=take(d, "kv_rank", int, where=where),
                   scale=take(d, "scale", float, where=where),
                   window=take(mask, "size", int, None, where=where + ".mask"),
                   rot_dims=take(rot, "dims", int, None, where=where + ".rot"),
                   rot_base=take(rot, "base", float, None, where=where + ".rot"),
                   kv_from=take(d, "kv_from", int, None, where=where))

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "q_rank": self.q_rank,
             "kv_rank": self.kv_rank, "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.rot_dims is not None:
            d["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d

    def validate(self, where):
        if min(self.heads, self.vdim, self.q_rank, self.kv_rank) <= 0 or self.dim < 0 or self.rot_dim < 0 \
                or self.dim + self.rot_dim <= 0:
            raise ConfigError(f"{where}: heads, vdim, q_rank and kv_rank must be > 0, dim + rot_dim > 0")
        if self.window is not None and self.window <= 0:
            raise ConfigError(f"{where}: mask.size must be > 0")
        if self.rot_dims is not None:
            if self.rot_dims % 2 or not (0 < self.rot_dims <= self.rot_dim) or self.rot_base is None or self.rot_base <= 0:
                raise ConfigError(f"{where}: rot.dims must be even and at most rot_dim, rot.base positive")


@dataclasses.dataclass(frozen=True)
class ExpertsSpec:
    ff: int
    experts: int
    top: int
    scale: float

    @classmethod
    def from_dict(cls, d, where):
        kind = take(d, "kind", str, where=where)
        if kind != "moe":
            raise ConfigError(f"{where}: unknown kind {kind!r} (known: moe)")
        expert, router = d.get("expert"), d.get("router")
        if not isinstance(expert, dict) or not isinstance(router, dict):
            raise ConfigError(f"{where}: 'expert' and 'router' must be objects")
        return cls(ff=take(expert, "ff", int, where=where + ".expert"),
                   experts=take(router, "experts", int, where=where + ".router"),
                   top=take(router, "top", int, where=where + ".router"),
                   scale=take(router, "scale", float, where=where + ".router"))

    def to_dict(self):
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top, "scale": self.scale}}

    def validate(self, where):
        if self.ff <= 0 or not (0 < self.top <= self.experts):
            raise ConfigError(f"{where}: expert.ff must be > 0 and 0 < router.top <= router.experts")


@dataclasses.dataclass(frozen=True)
class PidutarLayer:
    type: str
    memory: Optional[MatrixMemorySpec] = None
    attention: Optional[LatentAttentionSpec] = None
    mlp: Optional[ExpertsSpec] = None            # None: the layer has no feed-forward

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
        if typ == "mlstm":
            kw["memory"] = MatrixMemorySpec.from_dict(mixer, where + ".mixer")
        elif typ == "latent_attention":
            kw["attention"] = LatentAttentionSpec.from_dict(mixer, where + ".mixer")
        else:
            raise ConfigError(f"{where}: unknown layer type {typ!r} (known: mlstm, latent_attention)")
        mlp = d.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict):
                raise ConfigError(f"{where}: 'mlp' must be an object or null")
            kw["mlp"] = ExpertsSpec.from_dict(mlp, where + ".mlp")
        return cls(type=typ, **kw)

    def to_dict(self):
        mixer = self.memory.to_dict() if self.type == "mlstm" else self.attention.to_dict()
        return {"type": self.type, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclasses.dataclass(frozen=True)
class PidutarConfig(ModelConfig):
    architectures: ClassVar[Tuple[str, ...]] = ("Pidutar",)
    model_types: ClassVar[Tuple[str, ...]] = ("pidutar",)

    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    layers: Tuple[PidutarLayer, ...] = ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PidutarConfig":
        norm, emb = d.get("norm"), d.get("embedding")
        if not isinstance(norm, dict) or not isinstance(emb, dict):
            raise ConfigError("config.json: 'norm' and 'embedding' must be objects")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        cfg = cls(vocab=take(d, "vocab", int), width=take(d, "width", int),
                  norm_eps=take(norm, "eps", float, where="config.json: norm"),
                  embedding_scale=take(emb, "scale", float, where="config.json: embedding"),
                  residual_mult=take(d, "residual_mult", float), logit_scale=take(d, "logit_scale", float),
                  layers=tuple(PidutarLayer.from_dict(x, i) for i, x in enumerate(layers)))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architectures[0], "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
                "layers": [x.to_dict() for x in self.layers]}

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: vocab and width must be > 0")
        if self.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        for i, layer in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            if layer.type == "mlstm":
                layer.memory.validate(where + ".mixer")
            else:
                a = layer.attention
                a.validate(where + ".mixer")
                if a.kv_from is not None:
                    j = a.kv_from
                    if not (0 <= j < i) or self.layers[j].type != "latent_attention" \
                            or self.layers[j].attention.kv_from is not None:
                        raise ConfigError(f"{where}.mixer: kv_from must name an earlier latent attention layer that "
                                          "has a key/value latent of its own")
                    b = self.layers[j].attention
                    if (a.kv_rank, a.rot_dim, a.rot_dims, a.rot_base) != (b.kv_rank, b.rot_dim, b.rot_dims, b.rot_base):
                        raise ConfigError(f"{where}.mixer: kv_rank, rot_dim and rot must equal those of layer {j}")
            if layer.mlp is not None:
                layer.mlp.validate(where + ".mlp")
