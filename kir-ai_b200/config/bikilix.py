"""Typed configuration of the Bikilix decoder.

config.json of this design is nested: ``architecture`` (a string), ``width``, ``vocab``, ``norm.eps``,
``embedding.scale``, ``layers`` and optionally ``loop``.  Every entry of ``layers`` has ``type`` (the kind of mixer),
``mixer`` (its sizes and constants) and ``mlp`` (null for a layer without feed-forward).  The kinds of mixer:

* ``attention``: ``heads``, ``kv_heads``, ``dim`` (query/key size of a head), ``vdim`` (its value size), ``scale``
  (the factor on the scores), ``rot`` (``base``, ``dims`` = how many leading columns of a head are rotated) and
  ``mask.size`` (a position sees itself and the ``size`` - 1 positions before it; without ``mask`` every earlier one);
* ``latent_attention``: ``heads``, ``dim`` (unrotated) and ``rot_dim`` (rotated query/key columns of a head),
  ``vdim``, ``q_rank`` and ``kv_rank`` (sizes of the two latents), ``scale``, ``rot`` (``base``; ``dims`` equals
  ``rot_dim``; optionally ``scaling`` with ``factor``, ``original``, ``fast``, ``slow``).

The kinds of feed-forward: ``dense`` with ``ff``; ``moe`` with ``expert`` (``ff``, ``limit``) and ``router``
(``experts``, ``top``, and ``groups`` with ``count`` and ``keep``).

``loop`` = {``start``, ``stop``, ``times``}: layers start .. stop - 1 run ``times`` times in a row with the same
weights before the rest follows.  Every size and constant that a model of the design may set is read from there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, optional_int, required_float, required_int

_FAMILY = "bikilix"
MIXER_KINDS = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


def _mapping(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError.unsupported(f"{_FAMILY} config {where} missing {key}")
    return value


def _whole(value: float):
    return int(value) if float(value).is_integer() else value


@dataclass(frozen=True)
class IndexScaling:
    """Frequencies stretched by their index (see ``parts.rope``)."""

    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self) -> dict:
        return {"factor": self.factor, "fast": self.fast, "original": _whole(self.original), "slow": self.slow}


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
        dims = required_int(raw, "dims", _FAMILY)
        if dims % 2:
            raise ConfigError.invalid(f"{_FAMILY} config {where}.dims must be even, got {dims}")
        base = required_float(raw, "base", _FAMILY)
        if base <= 1.0:
            raise ConfigError.invalid(f"{_FAMILY} config {where}.base must exceed one, got {base}")
        return cls(base=base, dims=dims, scaling=scaling)

    def to_dict(self) -> dict:
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = self.scaling.to_dict()
        return out


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation
    window: Optional[int] = None

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "rot": self.rot.to_dict(), "scale": self.scale,
               "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Rotation

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "rot": self.rot.to_dict(),
                "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class DenseMLP:
    ff: int

    def to_dict(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class ExpertsMLP:
    ff: int
    limit: float
    experts: int
    top: int
    groups: int
    keep: int

    def to_dict(self) -> dict:
        return {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe",
                "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.keep}, "top": self.top}}


@dataclass(frozen=True)
class BikilixLayer:
    kind: str
    mixer: object
    mlp: object  # DenseMLP, ExpertsMLP or None


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


def _mixer(kind: str, m: Mapping[str, Any], where: str):
    rot = Rotation.from_dict(_mapping(m, "rot", where), where + ".rot")
    if kind == "attention":
        heads, kv_heads = required_int(m, "heads", _FAMILY), required_int(m, "kv_heads", _FAMILY)
        if heads % kv_heads:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        dim = required_int(m, "dim", _FAMILY)
        if rot.dims > dim:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: rot.dims {rot.dims} exceeds dim {dim}")
        if rot.scaling is not None:
            raise ConfigError.unsupported(f"{_FAMILY} config {where}: stretched frequencies belong to latent attention")
        window = None if m.get("mask") is None else required_int(_mapping(m, "mask", where), "size", _FAMILY)
        return AttentionMixer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=required_int(m, "vdim", _FAMILY),
                              scale=required_float(m, "scale", _FAMILY), rot=rot, window=window)
    rot_dim = required_int(m, "rot_dim", _FAMILY)
    if rot.dims != rot_dim:
        raise ConfigError.invalid(f"{_FAMILY} config {where}: rot.dims {rot.dims} must equal rot_dim {rot_dim}")
    return LatentMixer(heads=required_int(m, "heads", _FAMILY), dim=required_int(m, "dim", _FAMILY), rot_dim=rot_dim,
                       vdim=required_int(m, "vdim", _FAMILY), q_rank=required_int(m, "q_rank", _FAMILY),
                       kv_rank=required_int(m, "kv_rank", _FAMILY), scale=required_float(m, "scale", _FAMILY), rot=rot)


def _mlp(mlp, where: str):
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, Mapping) else mlp
    if kind not in MLP_KINDS:
        raise ConfigError.unsupported(f"{_FAMILY} config {where}: feed-forward kind {kind!r} is unsupported; known: {', '.join(MLP_KINDS)}")
    if kind == "dense":
        return DenseMLP(ff=required_int(mlp, "ff", _FAMILY))
    expert, router = _mapping(mlp, "expert", where), _mapping(mlp, "router", where)
    experts, top = required_int(router, "experts", _FAMILY), required_int(router, "top", _FAMILY)
    groups, keep = 1, 1
    if router.get("groups") is not None:
        g = _mapping(router, "groups", where + ".router")
        groups, keep = required_int(g, "count", _FAMILY), required_int(g, "keep", _FAMILY)
    if experts % groups or not 0 < keep <= groups:
        raise ConfigError.invalid(f"{_FAMILY} config {where}: {experts} experts in {groups} equal groups of which {keep} stay open")
    if not 0 < top <= keep * (experts // groups):
        raise ConfigError.invalid(f"{_FAMILY} config {where}: a token uses {top} experts, {keep} groups of {experts // groups} are open")
    limit = required_float(expert, "limit", _FAMILY)
    if limit <= 0.0:
        raise ConfigError.invalid(f"{_FAMILY} config {where}: expert.limit must be positive, got {limit}")
    return ExpertsMLP(ff=required_int(expert, "ff", _FAMILY), limit=limit, experts=experts, top=top, groups=groups, keep=keep)


@dataclass(frozen=True)
class BikilixConfig:
    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[BikilixLayer, ...]
    loop: Optional[Loop] = None

    architecture = "Bikilix"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def passes(self):
        """The runs of layers in order, as (pass number or None, (layer indices)): every pass of the looped stretch is
        an entry with its number, the layers ahead of and behind the stretch are entries without one."""
        count = len(self.layers)
        if self.loop is None:
            return ((None, tuple(range(count))),)
        out = []
        if self.loop.start:
            out.append((None, tuple(range(self.loop.start))))
        out += [(t, tuple(range(self.loop.start, self.loop.stop))) for t in range(self.loop.times)]
        if self.loop.stop < count:
            out.append((None, tuple(range(self.loop.stop, count))))
        return tuple(out)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "BikilixConfig":
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
            layers.append(BikilixLayer(kind, _mixer(kind, _mapping(entry, "mixer", where), where + ".mixer"),
                                       _mlp(entry.get("mlp"), where + ".mlp")))
        eps = required_float(_mapping(raw, "norm", "root"), "eps", _FAMILY)
        if eps < 0.0:
            raise ConfigError.invalid(f"{_FAMILY} config norm.eps must be non-negative")
        scale = 1.0
        if raw.get("embedding") is not None:
            scale = required_float(_mapping(raw, "embedding", "root"), "scale", _FAMILY)
        loop = None
        if raw.get("loop") is not None:
            lp = _mapping(raw, "loop", "root")
            loop = Loop(start=optional_int(lp, "start", _FAMILY, 0), stop=required_int(lp, "stop", _FAMILY, minimum=0),
                        times=required_int(lp, "times", _FAMILY))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError.invalid(f"{_FAMILY} config loop {loop.start}..{loop.stop} does not lie inside {len(layers)} layers")
        return cls(width=required_int(raw, "width", _FAMILY), vocab=required_int(raw, "vocab", _FAMILY), norm_eps=eps,
                   embedding_scale=scale, layers=tuple(layers), loop=loop)

    def to_dict(self) -> dict:
        """The config.json content that parses back to this configuration."""
        layers = [{"type": layer.kind, "mixer": layer.mixer.to_dict(), "mlp": None if layer.mlp is None else layer.mlp.to_dict()}
                  for layer in self.layers]
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out
