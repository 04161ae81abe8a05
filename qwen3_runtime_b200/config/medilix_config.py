"""Typed configuration of the Medilix design, read from its own ``config.json`` keys.

The file lists the layers one by one: each entry names its mixer (``type``: ``mlstm``, ``attention``
or ``wkv``) with the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``: ``kind``
``dense`` or ``moe``, or null for none).  ``embedding`` gives the scale of the token rows and the
hash of the bigram table, ``norm`` the eps and the number of groups of every norm, ``loop`` the run
of layers that is repeated with the same weights.  Every size and constant that can differ between
two models of the design is a field here; nothing is assumed equal between layers.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Mapping

from .model_config import ConfigError, _require


def _positive_int(where: str, raw: Mapping[str, Any], key: str) -> int:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"{where}: missing key {key!r}")
    value = raw[key]
    if int(value) != value or int(value) < 1:
        raise ConfigError(f"{where}: {key} must be a positive integer, got {value!r}")
    return int(value)


@dataclass(frozen=True)
class BigramConfig:
    """Row ``(previous * mul_prev + token * mul_cur) mod buckets`` of a table of ``buckets + 1`` rows is
    added to the token's embedding; a sequence's first token takes the last row."""

    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class MlstmConfig:
    """A matrix memory with exponential input and forget gates whose logits are capped smoothly."""

    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class GatedAttentionConfig:
    """Softmax attention with grouped key/value heads, unit-normed q and k, a window that also keeps the
    sequence's first ``keep_first`` tokens (``window`` None: every earlier token is seen), one added to
    the softmax's denominator and a sigmoid gate on the heads' outputs."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None
    keep_first: int


@dataclass(frozen=True)
class WkvConfig:
    """Token-shifted inputs and a decayed matrix state with a bonus for the present token.  ``decay_rank``:
    rows of the decay's first matrix; config.json does not say: 0 until the stored tensor's shape has been
    read (:meth:`MedilixConfig.with_tensor_shapes`)."""

    heads: int
    dim: int
    decay_rank: int = 0


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeConfig:
    """``experts`` stored experts of ``ff`` rows and ``identity`` further router outputs that stand for
    experts returning their input; ``top`` are chosen per token, only from the best ``groups_keep`` of
    ``groups`` equal groups of neighbouring router outputs."""

    experts: int
    identity: int
    top: int
    ff: int
    groups: int
    groups_keep: int


def _mixer_from_raw(where: str, kind: str, raw: Mapping[str, Any]):
    if kind == "mlstm":
        cfg = MlstmConfig(heads=_positive_int(where, raw, "heads"), dim=_positive_int(where, raw, "dim"),
                          vdim=_positive_int(where, raw, "vdim"), gate_cap=float(_require(raw, "gate_cap")))
        if not cfg.gate_cap > 0:
            raise ConfigError(f"{where}: gate_cap must be positive")
        return cfg
    if kind == "attention":
        mask = raw.get("mask") or {}
        window = mask.get("size")
        cfg = GatedAttentionConfig(
            heads=_positive_int(where, raw, "heads"), kv_heads=_positive_int(where, raw, "kv_heads"),
            dim=_positive_int(where, raw, "dim"), vdim=_positive_int(where, raw, "vdim"),
            scale=float(_require(raw, "scale")), window=int(window) if window else None,
            keep_first=int(mask.get("keep_first") or 0) if window else 0)
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"{where}: heads={cfg.heads} is no multiple of kv_heads={cfg.kv_heads}")
        if cfg.keep_first < 0 or (cfg.window is not None and cfg.window < 1):
            raise ConfigError(f"{where}: mask.size must be positive and mask.keep_first not negative")
        return cfg
    if kind == "wkv":
        return WkvConfig(heads=_positive_int(where, raw, "heads"), dim=_positive_int(where, raw, "dim"),
                         decay_rank=int(raw.get("decay_rank") or 0))  # an optional key: a model yet to be written
    raise ConfigError(f"{where}: unknown layer type {kind!r} (mlstm, attention or wkv)")


def _mixer_to_raw(m) -> dict[str, Any]:
    if isinstance(m, MlstmConfig):
        return dict(heads=m.heads, dim=m.dim, vdim=m.vdim, gate_cap=m.gate_cap)
    if isinstance(m, GatedAttentionConfig):
        out = dict(heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale)
        if m.window:
            out["mask"] = dict(size=m.window, keep_first=m.keep_first)
        return out
    return dict(heads=m.heads, dim=m.dim, decay_rank=m.decay_rank)


def _mlp_from_raw(where: str, raw: Mapping[str, Any] | None):
    if not raw:
        return None
    kind = raw.get("kind")
    if kind == "dense":
        cfg = DenseConfig(ff=_positive_int(where, raw, "ff"), limit=float(_require(raw, "limit")))
        if not cfg.limit > 0:
            raise ConfigError(f"{where}: limit must be positive")
        return cfg
    if kind == "moe":
        router = _require(raw, "router")
        groups = router.get("groups") or {}
        cfg = MoeConfig(experts=_positive_int(where + ".router", router, "experts"),
                        identity=int(router.get("identity") or 0), top=_positive_int(where + ".router", router, "top"),
                        ff=_positive_int(where + ".expert", _require(raw, "expert"), "ff"),
                        groups=int(groups.get("count") or 1), groups_keep=int(groups.get("keep") or groups.get("count") or 1))
        total = cfg.experts + cfg.identity
        if cfg.identity < 0 or cfg.top > total:
            raise ConfigError(f"{where}: top={cfg.top} of {total} router outputs")
        if cfg.groups < 1 or total % cfg.groups or not 1 <= cfg.groups_keep <= cfg.groups:
            raise ConfigError(f"{where}: {total} router outputs do not form {cfg.groups} equal groups "
                              f"of which {cfg.groups_keep} are kept")
        if cfg.groups_keep * (total // cfg.groups) < cfg.top:
            raise ConfigError(f"{where}: the kept groups hold fewer than top={cfg.top} router outputs")
        return cfg
    raise ConfigError(f"{where}: unknown feed-forward kind {kind!r} (dense or moe)")


def _mlp_to_raw(f) -> dict[str, Any] | None:
    if f is None:
        return None
    if isinstance(f, DenseConfig):
        return dict(kind="dense", ff=f.ff, limit=f.limit)
    return dict(kind="moe", expert=dict(ff=f.ff),
                router=dict(experts=f.experts, identity=f.identity, top=f.top,
                            groups=dict(count=f.groups, keep=f.groups_keep)))


@dataclass(frozen=True)
class MedilixLayerConfig:
    kind: str  # mlstm | attention | wkv
    mixer: Any
    mlp: Any  # DenseConfig | MoeConfig | None


@dataclass(frozen=True)
class MedilixConfig:
    architecture = "Medilix"

    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    embed_scale: float
    bigram: BigramConfig | None
    layers: tuple[MedilixLayerConfig, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0  # 0: no loop

    def __post_init__(self) -> None:
        if not self.layers:
            raise ConfigError("Medilix: at least one layer")
        if self.norm_groups < 1 or self.width % self.norm_groups:
            raise ConfigError(f"Medilix: width={self.width} does not split into norm.groups={self.norm_groups} equal parts")
        if self.loop_times and not 0 <= self.loop_start < self.loop_stop <= len(self.layers):
            raise ConfigError(f"Medilix: loop {self.loop_start}..{self.loop_stop} lies outside the "
                              f"{len(self.layers)} layers")

    @classmethod
    def from_hf_config(cls, raw: Mapping[str, Any]) -> "MedilixConfig":
        emb = raw.get("embedding") or {}
        big = emb.get("bigram")
        bigram = None
        if big:
            bigram = BigramConfig(buckets=_positive_int("embedding.bigram", big, "buckets"),
                                  mul_prev=int(_require(big, "mul_prev")), mul_cur=int(_require(big, "mul_cur")))
        norm = _require(raw, "norm")
        layers = []
        for i, entry in enumerate(_require(raw, "layers")):
            where = f"layers[{i}]"
            kind = _require(entry, "type")
            layers.append(MedilixLayerConfig(kind, _mixer_from_raw(where + ".mixer", kind, _require(entry, "mixer")),
                                             _mlp_from_raw(where + ".mlp", entry.get("mlp"))))
        loop = raw.get("loop") or {}
        times = int(loop.get("times") or 0)
        return cls(vocab=_positive_int("config", raw, "vocab"), width=_positive_int("config", raw, "width"),
                   norm_eps=float(_require(norm, "eps")), norm_groups=int(norm.get("groups") or 1),
                   embed_scale=float(emb.get("scale", 1.0)), bigram=bigram, layers=tuple(layers),
                   loop_start=int(loop.get("start") or 0) if times else 0,
                   loop_stop=int(loop.get("stop") or 0) if times else 0, loop_times=times)

    def to_hf_config(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(
            architecture=self.architecture, vocab=self.vocab, width=self.width,
            norm=dict(eps=self.norm_eps, groups=self.norm_groups),
            embedding=dict(scale=self.embed_scale),
            layers=[dict(type=layer.kind, mixer=_mixer_to_raw(layer.mixer), mlp=_mlp_to_raw(layer.mlp))
                    for layer in self.layers])
        if self.bigram is not None:
            out["embedding"]["bigram"] = dict(buckets=self.bigram.buckets, mul_prev=self.bigram.mul_prev,
                                              mul_cur=self.bigram.mul_cur)
        if self.loop_times:
            out["loop"] = dict(start=self.loop_start, stop=self.loop_stop, times=self.loop_times)
        return out

    def with_tensor_shapes(self, shape_of) -> "MedilixConfig":
        """The sizes that only a stored tensor gives: the rank of a wkv layer's decay product is the
        row count of ``l<i>.mix.w1``.  ``shape_of(name)`` returns a stored tensor's shape."""
        layers = []
        for i, layer in enumerate(self.layers):
            if isinstance(layer.mixer, WkvConfig) and not layer.mixer.decay_rank:
                rank = int(shape_of(f"l{i}.mix.w1")[0])
                layer = dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, decay_rank=rank))
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    def run_order(self) -> list[tuple[int, bool]]:
        """``(layer, a pass of the loop starts here)`` in the order the layers run."""
        n = len(self.layers)
        if not self.loop_times:
            return [(i, False) for i in range(n)]
        order = [(i, False) for i in range(self.loop_start)]
        for _ in range(self.loop_times):
            order += [(i, i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, False) for i in range(self.loop_stop, n)]
