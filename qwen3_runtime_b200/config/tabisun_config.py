"""Typed configuration of the Tabisun design, read from its own ``config.json`` keys.

The file lists the layers one by one: each entry names its mixer (``type``) with the mixer's sizes and
constants (``mixer``) and its feed-forward (``mlp``, or null for none).  An entry with ``weights_of: j`` has
no stored tensors: it runs layer j's mixer, feed-forward and norms on a cache layer of its own.  Every size
and constant that can differ between two models of the design is a field here; nothing is assumed equal
between layers.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .logesun_config import _positive_int
from .model_config import ConfigError, _require


def _positive(where: str, raw: Mapping[str, Any], key: str) -> float:
    value = float(_require(raw, key))
    if not value > 0:
        raise ConfigError(f"{where}: {key} must be positive, got {value!r}")
    return value


@dataclass(frozen=True)
class RotaryConfig:
    """``dims`` leading dimensions of a head turn by position * base^(-2i / dims), rescaled by ``scaling``
    (a tuple of (key, value) pairs; which keys it has depends on the mixer)."""

    dims: int
    base: float
    scaling: tuple[tuple[str, float], ...] = ()

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any], keys: tuple[str, ...], limit: int) -> "RotaryConfig":
        dims = _positive_int(where, raw, "dims")
        if dims % 2 or dims > limit:
            raise ConfigError(f"{where}: dims={dims} must be even and at most {limit}")
        scaling = raw.get("scaling")
        pairs: tuple[tuple[str, float], ...] = ()
        if scaling:
            pairs = tuple((k, _positive(where + ".scaling", scaling, k)) for k in keys)
        return cls(dims=dims, base=_positive(where, raw, "base"), scaling=pairs)

    def to_raw(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(base=self.base, dims=self.dims)
        if self.scaling:
            out["scaling"] = dict(self.scaling)
        return out


def _heads(where: str, raw: Mapping[str, Any]) -> tuple[int, int]:
    heads, kv_heads = _positive_int(where, raw, "heads"), _positive_int(where, raw, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"{where}: heads={heads} must be a multiple of kv_heads={kv_heads}")
    return heads, kv_heads


@dataclass(frozen=True)
class DifferentialConfig:
    """``attention``: two score maps per head over shared values, chunked mask, no positions."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    chunk: int | None

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "DifferentialConfig":
        heads, kv_heads = _heads(where, raw)
        mask = raw.get("mask") or {}
        chunk = int(mask["size"]) if mask.get("size") else None
        if chunk is not None and chunk < 1:
            raise ConfigError(f"{where}: mask.size must be positive")
        return cls(heads=heads, kv_heads=kv_heads, dim=_positive_int(where, raw, "dim"),
                   vdim=_positive_int(where, raw, "vdim"), scale=_positive(where, raw, "scale"),
                   diff=float(_require(raw, "diff")), chunk=chunk)

    def to_raw(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                                   scale=self.scale, diff=self.diff)
        if self.chunk is not None:
            out["mask"] = dict(size=self.chunk)
        return out


@dataclass(frozen=True)
class KeyValueConfig:
    """``attention_2``: grouped heads whose values are the projected keys; rotary on interleaved pairs with a
    wavelength-dependent rescaling; capped scores; causal."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    rot: RotaryConfig | None

    SCALING_KEYS = ("factor", "low", "high", "original")

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "KeyValueConfig":
        heads, kv_heads = _heads(where, raw)
        dim = _positive_int(where, raw, "dim")
        vdim = int(raw.get("vdim", dim))
        if vdim != dim:
            raise ConfigError(f"{where}: the values are the keys, so vdim={vdim} must equal dim={dim}")
        rot = raw.get("rot")
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=_positive(where, raw, "scale"),
                   softcap=_positive(where, raw, "softcap") if raw.get("softcap") else None,
                   rot=RotaryConfig.from_raw(where + ".rot", rot, cls.SCALING_KEYS, dim) if rot else None)

    def to_raw(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                                   scale=self.scale)
        if self.softcap is not None:
            out["softcap"] = self.softcap
        if self.rot is not None:
            out["rot"] = self.rot.to_raw()
        return out


@dataclass(frozen=True)
class LatentConfig:
    """``latent_attention``: keys and values through a normed latent, one rotated key part for all heads
    (halves pairing, ramped rescaling), a sink per head, a sigmoid gate on the heads' outputs; causal."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig

    SCALING_KEYS = ("factor", "original", "fast", "slow")

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "LatentConfig":
        rot_dim = _positive_int(where, raw, "rot_dim")
        return cls(heads=_positive_int(where, raw, "heads"), dim=_positive_int(where, raw, "dim"), rot_dim=rot_dim,
                   vdim=_positive_int(where, raw, "vdim"), kv_rank=_positive_int(where, raw, "kv_rank"),
                   scale=_positive(where, raw, "scale"),
                   rot=RotaryConfig.from_raw(where + ".rot", _require(raw, "rot"), cls.SCALING_KEYS, rot_dim))

    def to_raw(self) -> dict[str, Any]:
        return dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, kv_rank=self.kv_rank,
                    scale=self.scale, rot=self.rot.to_raw())


MIXER_CONFIGS = {"attention": DifferentialConfig, "attention_2": KeyValueConfig, "latent_attention": LatentConfig}


@dataclass(frozen=True)
class TabisunLayerConfig:
    type: str
    mixer: Any
    ff: int | None  # width of the dense gated feed-forward; None: the layer has none
    weights_of: int | None = None  # the layer whose tensors this one runs with


@dataclass(frozen=True)
class TabisunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[TabisunLayerConfig, ...]
    logit_softcap: float | None = None
    extra: dict = field(default_factory=dict, compare=False, repr=False)

    architecture = "Tabisun"

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps!r}")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        for i, layer in enumerate(self.layers):
            if layer.weights_of is None:
                continue
            owner = self.layers[self.owner_of(i)]
            if (owner.type, owner.mixer, owner.ff) != (layer.type, layer.mixer, layer.ff):
                raise ConfigError(f"layer {i}: its entry differs from layer {self.owner_of(i)}'s, whose weights it uses")

    def owner_of(self, i: int) -> int:
        """The layer whose stored tensors layer ``i`` runs with (itself, or where its ``weights_of`` leads)."""
        seen = {i}
        while self.layers[i].weights_of is not None:
            j = self.layers[i].weights_of
            if not 0 <= j < len(self.layers) or j in seen:
                raise ConfigError(f"layer {i}: weights_of={j} must lead to another layer that has tensors of its own")
            seen.add(j)
            i = j
        return i

    @classmethod
    def from_hf_config(cls, raw: Mapping[str, Any]) -> "TabisunConfig":
        names = [raw.get("architecture"), *(raw.get("architectures") or [])]
        if cls.architecture not in names:
            raise ConfigError(f"unsupported architecture: {names}")
        layers = []
        for i, entry in enumerate(_require(raw, "layers")):
            kind = _require(entry, "type")
            if kind not in MIXER_CONFIGS:
                raise ConfigError(f"layer {i}: unknown layer type {kind!r} (known: {sorted(MIXER_CONFIGS)})")
            mixer = MIXER_CONFIGS[kind].from_raw(f"layer {i} mixer", _require(entry, "mixer"))
            mlp = entry.get("mlp")
            ff = None
            if mlp:
                if _require(mlp, "kind") != "dense":
                    raise ConfigError(f"layer {i} mlp: unknown feed-forward kind {mlp['kind']!r}")
                ff = _positive_int(f"layer {i} mlp", mlp, "ff")
            owner = entry.get("weights_of")
            layers.append(TabisunLayerConfig(kind, mixer, ff, int(owner) if owner is not None else None))
        cap = raw.get("logit_softcap")
        return cls(vocab=int(_require(raw, "vocab")), width=int(_require(raw, "width")),
                   norm_eps=float(_require(_require(raw, "norm"), "eps")), layers=tuple(layers),
                   logit_softcap=float(cap) if cap else None)

    def to_hf_config(self) -> dict[str, Any]:
        """The ``config.json`` dictionary that :meth:`from_hf_config` reads back."""
        out: dict[str, Any] = dict(architecture=self.architecture, vocab=self.vocab, width=self.width,
                                   norm=dict(eps=self.norm_eps))
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        out["layers"] = []
        for layer in self.layers:
            entry = dict(type=layer.type, mixer=layer.mixer.to_raw(),
                         mlp=dict(kind="dense", ff=layer.ff) if layer.ff else None)
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            out["layers"].append(entry)
        return copy.deepcopy(out)
