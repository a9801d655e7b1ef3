"""Typed configuration of the Netinex decoder, read from config.json.

The file is nested.  Top level: ``architecture`` ("Netinex"), ``vocab``, ``width``, ``norm.eps`` (of the RMS norms
inside the mixers; the layers' own norm, a dynamic tanh, uses none), ``logit_softcap`` (absent or null: logits are not
capped) and ``layers``, a list in which every entry gives ``type`` ("retention" or "attention"), the sizes and constants
of its ``mixer`` and its ``mlp`` (``kind`` "moe" with ``expert.ff``, ``router.experts`` and ``router.top``, or null for
a layer without a feed-forward).

  retention mixer:  heads, dim, vdim, decay (one per head), rot (dims, base[, scaling])
  attention mixer:  heads, kv_heads, dim, vdim (the values are the keys, so vdim = dim), scale, mask.size (the chunk),
                    rot (dims, base, scaling: factor, original, fast, slow)

Every size and constant that can differ between two models of the design is read from here and from nowhere else;
what the design fixes (pair layouts of the rotations, the key factor of the retention, activations) is written where
the plan is made.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from ..errors import ConfigError, UnsupportedError
from .json_file import read_config_json
from .kugilix import _of


@dataclass(frozen=True)
class NetinexRotation:
    dims: int
    base: float
    scaling: Optional[tuple] = None  # (factor, original, fast, slow)

    def to_dict(self) -> dict:
        d: dict = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            factor, original, fast, slow = self.scaling
            d["scaling"] = {"factor": factor, "fast": fast, "original": original, "slow": slow}
        return d

    def scaling_dict(self) -> Optional[dict]:
        if self.scaling is None:
            return None
        factor, original, fast, slow = self.scaling
        return {"factor": factor, "original": original, "fast": fast, "slow": slow}

    @classmethod
    def from_dict(cls, d, where) -> Optional["NetinexRotation"]:
        if d is None:
            return None
        sc = _of(d, "scaling", dict, where, required=False)
        scaling = None
        if sc is not None:
            w = where + ".scaling"
            original = sc.get("original")
            if isinstance(original, bool) or not isinstance(original, (int, float)) or original <= 0:
                raise ConfigError(f"config.json: {w}.original must be a positive number, found {original!r}")
            scaling = (_of(sc, "factor", float, w), original, _of(sc, "fast", float, w), _of(sc, "slow", float, w))
        return cls(_of(d, "dims", int, where), _of(d, "base", float, where), scaling)


@dataclass(frozen=True)
class NetinexMixer:
    type: str  # "retention" or "attention"
    heads: int
    dim: int
    vdim: int
    rot: Optional[NetinexRotation] = None
    decay: tuple = ()  # retention, one per head
    kv_heads: int = 0  # attention
    scale: float = 0.0  # attention
    chunk: Optional[int] = None  # attention: mask.size (None: every earlier key is seen)

    def to_dict(self) -> dict:
        d: dict = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        if self.type == "retention":
            d["decay"] = list(self.decay)
        else:
            d["kv_heads"], d["scale"] = self.kv_heads, self.scale
            if self.chunk is not None:
                d["mask"] = {"size": self.chunk}
        return d


@dataclass(frozen=True)
class NetinexExperts:
    ff: int
    experts: int
    top: int

    def to_dict(self) -> dict:
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class NetinexLayer:
    mixer: NetinexMixer
    mlp: Optional[NetinexExperts]  # None: no feed-forward

    def to_dict(self) -> dict:
        return {"type": self.mixer.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class NetinexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple  # of NetinexLayer
    logit_softcap: Optional[float] = None
    architecture: str = "Netinex"

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        for name in ("vocab", "width"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be > 0, found {getattr(self, name)}")
        if not (self.norm_eps >= 0.0):
            raise ConfigError(f"config.json: norm.eps must be >= 0, found {self.norm_eps}")
        if self.logit_softcap is not None and not (self.logit_softcap > 0.0):
            raise ConfigError(f"config.json: logit_softcap must be > 0, found {self.logit_softcap}")
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        for i, layer in enumerate(self.layers):
            m, where = layer.mixer, f"layers[{i}]"
            if m.heads <= 0 or m.dim <= 0 or m.vdim <= 0:
                raise ConfigError(f"config.json: {where}.mixer sizes must be > 0")
            if m.rot is not None:
                if m.rot.dims < 0 or m.rot.dims % 2 or m.rot.dims > m.dim:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims = {m.rot.dims} must be even and at most dim = {m.dim}")
                if not (m.rot.base > 1.0):
                    raise ConfigError(f"config.json: {where}.mixer.rot.base must be > 1, found {m.rot.base}")
                if m.rot.scaling is not None and any(not (x > 0) for x in m.rot.scaling):
                    raise ConfigError(f"config.json: {where}.mixer.rot.scaling must hold positive numbers")
            if m.type == "attention":
                if m.kv_heads <= 0 or m.heads % m.kv_heads:
                    raise ConfigError(f"config.json: {where}: {m.heads} heads cannot share {m.kv_heads} kv heads")
                if m.vdim != m.dim:
                    raise ConfigError(f"config.json: {where}: the values are the keys, so vdim = {m.vdim} must equal dim = {m.dim}")
                if m.chunk is not None and m.chunk <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.mask.size must be > 0")
            elif m.type == "retention":
                if len(m.decay) != m.heads:
                    raise ConfigError(f"config.json: {where}: {len(m.decay)} decays for {m.heads} heads")
            if layer.mlp is not None:
                e = layer.mlp
                if e.ff <= 0 or e.experts <= 0 or not (1 <= e.top <= e.experts):
                    raise ConfigError(f"config.json: {where}.mlp: ff = {e.ff}, {e.top} of {e.experts} experts")

    # --------------------------------------------------------------------- I/O
    @classmethod
    def from_dict(cls, d: dict) -> "NetinexConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != "Netinex":
            raise UnsupportedError(f"architecture {name!r} is not read by NetinexConfig")
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
            rot = NetinexRotation.from_dict(_of(m, "rot", dict, mw, required=False), mw + ".rot")
            heads = _of(m, "heads", int, mw)
            if kind == "retention":
                decay = m.get("decay")
                if not isinstance(decay, list) or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
                    raise ConfigError(f"config.json: {mw}.decay must be a list of numbers")
                mixer = NetinexMixer("retention", heads, _of(m, "dim", int, mw), _of(m, "vdim", int, mw), rot,
                                     decay=tuple(float(x) for x in decay))
            elif kind == "attention":
                mask = _of(m, "mask", dict, mw, required=False)
                dim = _of(m, "dim", int, mw)
                mixer = NetinexMixer("attention", heads, dim, _of(m, "vdim", int, mw, default=dim, required=False), rot,
                                     kv_heads=_of(m, "kv_heads", int, mw, default=heads, required=False),
                                     scale=_of(m, "scale", float, mw),
                                     chunk=None if mask is None else _of(mask, "size", int, mw + ".mask"))
            else:
                raise UnsupportedError(f"config.json: {where}.type '{kind}' is not a mixer of this design")
            mlp = e.get("mlp")
            experts = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    raise UnsupportedError(f"config.json: {where}.mlp must be null or of kind 'moe'")
                router = _of(mlp, "router", dict, where + ".mlp")
                experts = NetinexExperts(_of(_of(mlp, "expert", dict, where + ".mlp"), "ff", int, where + ".mlp.expert"),
                                         _of(router, "experts", int, where + ".mlp.router"),
                                         _of(router, "top", int, where + ".mlp.router"))
            layers.append(NetinexLayer(mixer, experts))
        norm = _of(d, "norm", dict, "the top level")
        cfg = cls(
            vocab=_of(d, "vocab", int, "the top level"),
            width=_of(d, "width", int, "the top level"),
            norm_eps=_of(norm, "eps", float, "norm"),
            layers=tuple(layers),
            logit_softcap=_of(d, "logit_softcap", float, "the top level", required=False),
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict[str, Any]:
        d: dict = {
            "architecture": self.architecture,
            "vocab": self.vocab,
            "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [layer.to_dict() for layer in self.layers],
        }
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d

    @classmethod
    def from_json(cls, path: str) -> "NetinexConfig":
        return cls.from_dict(read_config_json(path))
