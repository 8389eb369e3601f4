"""Typed configuration of the Figalix decoder.

config.json of this design is nested: ``architecture`` (a string), ``width``, ``vocab``, ``norm.eps``,
``residual_mult`` (the factor on what every sub-layer adds to the stream), ``logit_softcap`` and ``layers``.  Every
entry of ``layers`` has ``type`` (the kind of mixer), ``mixer`` (its sizes and constants) and ``mlp`` (null for a layer
without feed-forward).  The kinds of mixer:

* ``parallel``: two mixers on the same rows, ``left`` and ``right``.  ``left`` is attention: ``heads``, ``kv_heads``,
  ``dim`` (query/key size of a head), ``vdim`` (its value size), ``scale`` (the factor on the scores), ``rot``
  (``base``, ``dims`` = how many leading columns of a head are rotated, optionally ``scaling`` with ``factor``,
  ``original``, ``fast``, ``slow``) and ``mask`` (``size`` of the window, ``keep_first`` = how many first tokens of a
  sequence every later position still sees).  ``right`` is a matrix memory: ``heads``, ``dim``, ``vdim``, ``gate_cap``.
* ``mamba2``: a state-space mixer: ``heads``, ``vdim`` (columns of a head), ``state`` (rows of a head's state),
  ``groups`` (of heads that share B and C), ``conv`` (taps of the short convolution), ``norm_groups`` (equal parts of
  the row that the output norm takes one by one).

The kinds of feed-forward: ``dense`` with ``ff``; ``moe`` with ``router`` (``experts``, ``top``), ``expert`` (``ff``)
and optionally ``shared`` (``ff``), a branch that runs for every token.  Every size and constant that a model of the
design may set is read from there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, optional_int, required_float, required_int

_FAMILY = "figalix"
MIXER_KINDS = ("parallel", "mamba2")
MLP_KINDS = ("dense", "moe")


def _mapping(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError.unsupported(f"{_FAMILY} config {where} missing {key}")
    return value


def _number(value: float):
    return int(value) if float(value).is_integer() and abs(value) < 2 ** 53 else value


@dataclass(frozen=True)
class IndexScaling:
    """Frequencies stretched by their index between the wavelengths that make ``fast`` and ``slow`` turns over
    ``original`` positions."""

    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self) -> dict:
        return {"factor": self.factor, "fast": self.fast, "original": _number(self.original), "slow": self.slow}


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[IndexScaling] = None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "Rotation":
        scaling = None
        if raw.get("scaling") is not None:
            sc = _mapping(raw, "scaling", where)
            scaling = IndexScaling(*(required_float(sc, key, _FAMILY) for key in ("factor", "original", "fast", "slow")))
            if min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0.0:
                raise ConfigError.invalid(f"{_FAMILY} config {where}.scaling needs positive constants")
        dims = required_int(raw, "dims", _FAMILY, minimum=0)
        if dims % 2:
            raise ConfigError.invalid(f"{_FAMILY} config {where}.dims must be even, got {dims}")
        base = required_float(raw, "base", _FAMILY)
        if base <= 1.0:
            raise ConfigError.invalid(f"{_FAMILY} config {where}.base must be above one, got {base}")
        return cls(base=base, dims=dims, scaling=scaling)

    def to_dict(self) -> dict:
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = self.scaling.to_dict()
        return out


@dataclass(frozen=True)
class WindowedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation
    window: Optional[int]
    keep_first: int

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "WindowedAttention":
        heads, kv_heads = required_int(m, "heads", _FAMILY), required_int(m, "kv_heads", _FAMILY)
        if heads % kv_heads:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        dim = required_int(m, "dim", _FAMILY)
        rot = Rotation.from_dict(_mapping(m, "rot", where), where + ".rot")
        if rot.dims > dim:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: rot.dims {rot.dims} exceeds dim {dim}")
        window, keep_first = None, 0
        if m.get("mask") is not None:
            mask = _mapping(m, "mask", where)
            window = required_int(mask, "size", _FAMILY)
            keep_first = optional_int(mask, "keep_first", _FAMILY, 0)
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=required_int(m, "vdim", _FAMILY),
                   scale=required_float(m, "scale", _FAMILY), rot=rot, window=window, keep_first=keep_first)

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "rot": self.rot.to_dict(), "scale": self.scale,
               "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"keep_first": self.keep_first, "size": self.window}
        return out


@dataclass(frozen=True)
class MatrixMemoryMixer:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "MatrixMemoryMixer":
        cap = required_float(m, "gate_cap", _FAMILY)
        if cap <= 0.0:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: gate_cap must be positive, got {cap}")
        return cls(heads=required_int(m, "heads", _FAMILY), dim=required_int(m, "dim", _FAMILY),
                   vdim=required_int(m, "vdim", _FAMILY), gate_cap=cap)

    def to_dict(self) -> dict:
        return {"dim": self.dim, "gate_cap": self.gate_cap, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelMixer:
    left: WindowedAttention
    right: MatrixMemoryMixer

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class StateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "StateSpace":
        out = cls(heads=required_int(m, "heads", _FAMILY), vdim=required_int(m, "vdim", _FAMILY),
                  state=required_int(m, "state", _FAMILY), groups=required_int(m, "groups", _FAMILY),
                  conv=required_int(m, "conv", _FAMILY), norm_groups=required_int(m, "norm_groups", _FAMILY))
        if out.heads % out.groups:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: {out.heads} heads are not a multiple of {out.groups} groups")
        if (out.heads * out.vdim) % out.norm_groups:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: {out.heads * out.vdim} columns do not split into "
                                      f"{out.norm_groups} equal parts")
        return out

    def to_dict(self) -> dict:
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}


@dataclass(frozen=True)
class DenseMLP:
    ff: int

    def to_dict(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class ExpertsMLP:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int] = None

    def to_dict(self) -> dict:
        out = {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class FigalixLayer:
    kind: str
    mixer: object
    mlp: object  # DenseMLP, ExpertsMLP or None


def _mlp(mlp, where: str):
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, Mapping) else mlp
    if kind not in MLP_KINDS:
        raise ConfigError.unsupported(f"{_FAMILY} config {where}: feed-forward kind {kind!r} is unsupported; known: {', '.join(MLP_KINDS)}")
    if kind == "dense":
        return DenseMLP(ff=required_int(mlp, "ff", _FAMILY))
    router = _mapping(mlp, "router", where)
    experts, top = required_int(router, "experts", _FAMILY), required_int(router, "top", _FAMILY)
    if top > experts:
        raise ConfigError.invalid(f"{_FAMILY} config {where}: every token uses {top} of {experts} experts")
    shared = None
    if mlp.get("shared") is not None:
        shared = required_int(_mapping(mlp, "shared", where), "ff", _FAMILY)
    return ExpertsMLP(experts=experts, top=top, ff=required_int(_mapping(mlp, "expert", where), "ff", _FAMILY), shared_ff=shared)


@dataclass(frozen=True)
class FigalixConfig:
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    logit_softcap: Optional[float]
    layers: Tuple[FigalixLayer, ...]

    architecture = "Figalix"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FigalixConfig":
        if raw.get("architecture") != cls.architecture:
            raise ConfigError.unsupported(f"config is not a {cls.architecture} model: architecture={raw.get('architecture')!r}")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError.unsupported(f"{_FAMILY} config missing layers")
        layers = []
        for index, entry in enumerate(entries):
            where = f"layers[{index}]"
            if not isinstance(entry, Mapping):
                raise ConfigError.invalid(f"{_FAMILY} config {where} must be an object")
            kind = entry.get("type")
            if kind not in MIXER_KINDS:
                raise ConfigError.unsupported(f"{_FAMILY} config {where}: layer type {kind!r} is unsupported; known: {', '.join(MIXER_KINDS)}")
            m = _mapping(entry, "mixer", where)
            if kind == "parallel":
                mixer = ParallelMixer(WindowedAttention.from_dict(_mapping(m, "left", where + ".mixer"), where + ".mixer.left"),
                                      MatrixMemoryMixer.from_dict(_mapping(m, "right", where + ".mixer"), where + ".mixer.right"))
            else:
                mixer = StateSpace.from_dict(m, where + ".mixer")
            layers.append(FigalixLayer(kind, mixer, _mlp(entry.get("mlp"), where + ".mlp")))
        eps = required_float(_mapping(raw, "norm", "root"), "eps", _FAMILY)
        if eps < 0.0:
            raise ConfigError.invalid(f"{_FAMILY} config norm.eps must be non-negative")
        softcap = None
        if raw.get("logit_softcap") is not None:
            softcap = required_float(raw, "logit_softcap", _FAMILY)
            if softcap <= 0.0:
                raise ConfigError.invalid(f"{_FAMILY} config logit_softcap must be positive, got {softcap}")
        mult = 1.0 if raw.get("residual_mult") is None else required_float(raw, "residual_mult", _FAMILY)
        return cls(width=required_int(raw, "width", _FAMILY), vocab=required_int(raw, "vocab", _FAMILY), norm_eps=eps,
                   residual_mult=mult, logit_softcap=softcap, layers=tuple(layers))

    def to_dict(self) -> dict:
        """The config.json content that parses back to this configuration."""
        layers = [{"type": layer.kind, "mixer": layer.mixer.to_dict(), "mlp": None if layer.mlp is None else layer.mlp.to_dict()}
                  for layer in self.layers]
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.norm_eps},
               "residual_mult": self.residual_mult, "layers": layers}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out
