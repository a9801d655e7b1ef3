"""Typed configuration of the Sumevik decoder, read from config.json.

The file is nested.  Top level: ``architecture`` ("Sumevik"), ``vocab``, ``width``, ``norm.eps`` (of every RMS norm of
the model), ``logit_scale`` (a factor on the logits; absent: 1) and ``layers``, a list in which every entry gives
``type`` ("rglru" or "parallel"), the sizes and constants of its ``mixer`` and its ``mlp`` (null: the layer has no
feed-forward).

  rglru mixer:     width (channels of the recurrence), blocks (of the block-diagonal gate matrices), conv (taps)
  parallel mixer:  left  = heads, kv_heads, dim, vdim, scale, mask.size (the chunk; absent: every earlier key is seen),
                           rot (dims, base; absent: nothing rotates)
                   right = heads, dim, vdim, tau
                   left_scale, right_scale
  mlp:             kind "dense" with ff, or kind "moe" with expert (ff, limit) and router (experts, identity, top,
                   groups: count, keep)

Every size and constant that can differ between two models of the design is read from here and from nowhere else;
what the design fixes (the factor -8 of the recurrence's decay, the 1.702 of the experts' gate, the pair layout of the
rotation) is written where the plan is made or in the kernels' parameters.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from ..errors import ConfigError, UnsupportedError
from .json_file import read_config_json
from .kugilix import _of


@dataclass(frozen=True)
class SumevikRecurrent:
    width: int
    blocks: int
    conv: int

    def to_dict(self) -> dict:
        return {"blocks": self.blocks, "conv": self.conv, "width": self.width}


@dataclass(frozen=True)
class SumevikAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int] = None
    rot_dims: int = 0
    rot_base: float = 10000.0

    def to_dict(self) -> dict:
        d: dict = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class SumevikLinearAttention:
    heads: int
    dim: int
    vdim: int
    tau: float

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "tau": self.tau, "vdim": self.vdim}


@dataclass(frozen=True)
class SumevikParallel:
    left: SumevikAttention
    right: SumevikLinearAttention
    left_scale: float
    right_scale: float

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class SumevikDense:
    ff: int

    def to_dict(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class SumevikExperts:
    ff: int
    limit: float
    experts: int  # experts with weights
    identity: int  # router outputs after those that stand for "the input itself"
    top: int
    group_count: int = 1
    group_keep: int = 1

    def to_dict(self) -> dict:
        return {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe",
                "router": {"experts": self.experts, "groups": {"count": self.group_count, "keep": self.group_keep},
                           "identity": self.identity, "top": self.top}}


@dataclass(frozen=True)
class SumevikLayer:
    type: str  # "rglru" or "parallel"
    mixer: Any  # SumevikRecurrent or SumevikParallel
    mlp: Any  # SumevikDense, SumevikExperts or None

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


@dataclass(frozen=True)
class SumevikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple  # of SumevikLayer
    logit_scale: float = 1.0
    architecture: str = "Sumevik"

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        for name in ("vocab", "width"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be > 0, found {getattr(self, name)}")
        if not (self.norm_eps >= 0.0):
            raise ConfigError(f"config.json: norm.eps must be >= 0, found {self.norm_eps}")
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            m = layer.mixer
            if layer.type == "rglru":
                if m.width <= 0 or m.blocks <= 0 or m.width % m.blocks:
                    raise ConfigError(f"config.json: {where}.mixer: {m.width} channels in {m.blocks} equal blocks")
                if m.conv < 1:
                    raise ConfigError(f"config.json: {where}.mixer.conv must be >= 1, found {m.conv}")
            else:
                a, g = m.left, m.right
                if a.heads <= 0 or a.kv_heads <= 0 or a.heads % a.kv_heads:
                    raise ConfigError(f"config.json: {where}.mixer.left: {a.heads} heads cannot share {a.kv_heads} kv heads")
                if a.dim <= 0 or a.vdim <= 0 or g.heads <= 0 or g.dim <= 0 or g.vdim <= 0:
                    raise ConfigError(f"config.json: {where}.mixer: head sizes must be > 0")
                if a.rot_dims < 0 or a.rot_dims % 2 or a.rot_dims > a.dim:
                    raise ConfigError(f"config.json: {where}.mixer.left.rot.dims = {a.rot_dims} must be even and at most dim = {a.dim}")
                if a.rot_dims and not (a.rot_base > 0.0):
                    raise ConfigError(f"config.json: {where}.mixer.left.rot.base must be > 0, found {a.rot_base}")
                if a.chunk is not None and a.chunk <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.left.mask.size must be > 0")
                if not (g.tau > 0.0):
                    raise ConfigError(f"config.json: {where}.mixer.right.tau must be > 0, found {g.tau}")
            e = layer.mlp
            if isinstance(e, SumevikDense) and e.ff <= 0:
                raise ConfigError(f"config.json: {where}.mlp.ff must be > 0")
            if isinstance(e, SumevikExperts):
                n = e.experts + e.identity
                if e.ff <= 0 or e.experts < 0 or e.identity < 0 or n <= 0 or not (1 <= e.top <= n):
                    raise ConfigError(f"config.json: {where}.mlp: ff = {e.ff}, {e.top} of {e.experts} + {e.identity} experts")
                if not (e.limit > 0.0):
                    raise ConfigError(f"config.json: {where}.mlp.expert.limit must be > 0, found {e.limit}")
                if e.group_count <= 0 or n % e.group_count or not (1 <= e.group_keep <= e.group_count):
                    raise ConfigError(f"config.json: {where}.mlp.router.groups: {n} router outputs in {e.group_count} "
                                      f"groups of which {e.group_keep} stay")
                if e.top > e.group_keep * (n // e.group_count):
                    raise ConfigError(f"config.json: {where}.mlp.router: {e.top} experts cannot be chosen from "
                                      f"{e.group_keep} groups of {n // e.group_count}")

    # --------------------------------------------------------------------- I/O
    @classmethod
    def from_dict(cls, d: dict) -> "SumevikConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != "Sumevik":
            raise UnsupportedError(f"architecture {name!r} is not read by SumevikConfig")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list):
            raise ConfigError("config.json: 'layers' must be a list")
        layers = []
        for i, e in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(e, dict) or not isinstance(e.get("type"), str):
                raise ConfigError(f"config.json: {where} must be an object with a 'type'")
            kind = e["type"]
            m = _of(e, "mixer", dict, where)
            mw = where + ".mixer"
            if kind == "rglru":
                mixer = SumevikRecurrent(_of(m, "width", int, mw), _of(m, "blocks", int, mw, default=1, required=False),
                                         _of(m, "conv", int, mw, default=1, required=False))
            elif kind == "parallel":
                left, right = _of(m, "left", dict, mw), _of(m, "right", dict, mw)
                lw, rw = mw + ".left", mw + ".right"
                mask = _of(left, "mask", dict, lw, required=False)
                rot = _of(left, "rot", dict, lw, required=False)
                heads, dim = _of(left, "heads", int, lw), _of(left, "dim", int, lw)
                attention = SumevikAttention(
                    heads, _of(left, "kv_heads", int, lw, default=heads, required=False), dim,
                    _of(left, "vdim", int, lw, default=dim, required=False), _of(left, "scale", float, lw),
                    chunk=None if mask is None else _of(mask, "size", int, lw + ".mask"),
                    rot_dims=0 if rot is None else _of(rot, "dims", int, lw + ".rot"),
                    rot_base=10000.0 if rot is None else _of(rot, "base", float, lw + ".rot"))
                rdim = _of(right, "dim", int, rw)
                linear = SumevikLinearAttention(_of(right, "heads", int, rw), rdim,
                                                _of(right, "vdim", int, rw, default=rdim, required=False),
                                                _of(right, "tau", float, rw))
                mixer = SumevikParallel(attention, linear, _of(m, "left_scale", float, mw, default=1.0, required=False),
                                        _of(m, "right_scale", float, mw, default=1.0, required=False))
            else:
                raise UnsupportedError(f"config.json: {where}.type '{kind}' is not a mixer of this design")
            raw = e.get("mlp")
            mlp = None
            if raw is not None:
                fw = where + ".mlp"
                if not isinstance(raw, dict) or raw.get("kind") not in ("dense", "moe"):
                    raise UnsupportedError(f"config.json: {fw} must be null or of kind 'dense' or 'moe'")
                if raw["kind"] == "dense":
                    mlp = SumevikDense(_of(raw, "ff", int, fw))
                else:
                    ex, router = _of(raw, "expert", dict, fw), _of(raw, "router", dict, fw)
                    groups = _of(router, "groups", dict, fw + ".router", required=False)
                    mlp = SumevikExperts(
                        _of(ex, "ff", int, fw + ".expert"), _of(ex, "limit", float, fw + ".expert"),
                        _of(router, "experts", int, fw + ".router"),
                        _of(router, "identity", int, fw + ".router", default=0, required=False),
                        _of(router, "top", int, fw + ".router"),
                        group_count=1 if groups is None else _of(groups, "count", int, fw + ".router.groups"),
                        group_keep=1 if groups is None else _of(groups, "keep", int, fw + ".router.groups"))
            layers.append(SumevikLayer(kind, mixer, mlp))
        norm = _of(d, "norm", dict, "the top level")
        cfg = cls(
            vocab=_of(d, "vocab", int, "the top level"),
            width=_of(d, "width", int, "the top level"),
            norm_eps=_of(norm, "eps", float, "norm"),
            layers=tuple(layers),
            logit_scale=_of(d, "logit_scale", float, "the top level", default=1.0, required=False),
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict[str, Any]:
        return {
            "architecture": self.architecture,
            "layers": [layer.to_dict() for layer in self.layers],
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }

    @classmethod
    def from_json(cls, path: str) -> "SumevikConfig":
        return cls.from_dict(read_config_json(path))
