"""Typed configuration of the Pevolorn design, read from its own config.json keys.

config.json carries ``architecture`` (the name), ``vocab``, ``width``, ``norm.eps``, ``postln_alpha`` and
``layers``: per layer ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (its feed-forward,
or null for a layer without one).  Layer types:

``latent_attention``  attention over one compressed vector per token: ``heads``, ``dim`` (unrotated query/key
                      elements per head), ``rot_dim`` (rotated ones), ``vdim``, ``kv_rank``, ``scale``, ``rot.base``,
                      ``rot.dims``; with ``kv_from``: j the layer has no compression of its own and reads layer j's
                      cache.
``parallel``          two mixers side by side, ``mixer.left`` (grouped-query attention: ``heads``, ``kv_heads``,
                      ``dim``, ``vdim``, ``scale``, ``softcap``, ``rot.base``, ``rot.dims``) and ``mixer.right`` (a
                      selective state space: ``heads``, ``vdim``, ``state``, ``groups``, ``conv``, ``norm_groups``),
                      mixed with ``mixer.left_scale`` and ``mixer.right_scale``.

Feed-forward ``moe``: ``expert.ff``, ``router.experts``, ``router.top``, ``router.identity``, ``router.groups.count``,
``router.groups.keep``, and ``shared.ff`` (or no ``shared``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple, Union

from .base import ConfigError, ModelConfig, coerce, optional, require

ARCHITECTURE = "Pevolorn"


def _section(raw: Dict[str, Any], key: str, where: str, needed: bool = True) -> Optional[Dict[str, Any]]:
    value = raw.get(key)
    if value is None:
        if needed:
            raise ConfigError(f"config.json: {where}{key!r} is missing")
        return None
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return value


def _positive(obj, names, where: str) -> None:
    for name in names:
        if not getattr(obj, name) > 0:
            raise ConfigError(f"config.json: {where}{name} must be positive")


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, raw, where):
        rot = _section(raw, "rot", where)
        rot_dim = require(raw, "rot_dim")
        kv_from = raw.get("kv_from")
        return cls(heads=require(raw, "heads"), dim=require(raw, "dim"), rot_dim=rot_dim,
                   vdim=optional(raw, "vdim", raw.get("dim")), kv_rank=require(raw, "kv_rank"),
                   scale=require(raw, "scale", float), rot_base=require(rot, "base", float),
                   rot_dims=optional(rot, "dims", rot_dim),
                   kv_from=None if kv_from is None else coerce(kv_from, where + "kv_from", int))

    def to_dict(self):
        out = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank,
               "rot": {"base": self.rot_base, "dims": self.rot_dims}, "rot_dim": self.rot_dim, "scale": self.scale,
               "vdim": self.vdim}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out

    def validate(self, where):
        _positive(self, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "rot_base"), where)
        if self.rot_dims % 2 or not 0 < self.rot_dims <= self.rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most rot_dim")


@dataclass(frozen=True)
class GroupedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    rot_base: float
    rot_dims: int

    @classmethod
    def from_dict(cls, raw, where):
        heads, dim = require(raw, "heads"), require(raw, "dim")
        rot = _section(raw, "rot", where)
        cap = raw.get("softcap")
        return cls(heads=heads, kv_heads=optional(raw, "kv_heads", heads), dim=dim, vdim=optional(raw, "vdim", dim),
                   scale=require(raw, "scale", float), softcap=None if cap is None else coerce(cap, where + "softcap", float),
                   rot_base=require(rot, "base", float), rot_dims=optional(rot, "dims", dim))

    def to_dict(self):
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
               "rot": {"base": self.rot_base, "dims": self.rot_dims}, "scale": self.scale, "vdim": self.vdim}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        return out

    def validate(self, where):
        _positive(self, ("heads", "kv_heads", "dim", "vdim", "rot_base"), where)
        if self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        if self.rot_dims % 2 or not 0 < self.rot_dims <= self.dim:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim")
        if self.softcap is not None and not self.softcap > 0:
            raise ConfigError(f"config.json: {where}softcap must be positive")


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, raw, where):
        return cls(heads=require(raw, "heads"), vdim=require(raw, "vdim"), state=require(raw, "state"),
                   groups=optional(raw, "groups", 1), conv=require(raw, "conv"), norm_groups=optional(raw, "norm_groups", 1))

    def to_dict(self):
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}

    def validate(self, where):
        _positive(self, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), where)
        if self.heads % self.groups:
            raise ConfigError(f"config.json: {where}heads must be a multiple of groups")
        if (self.heads * self.vdim) % self.norm_groups:
            raise ConfigError(f"config.json: {where}heads * vdim must be a multiple of norm_groups")


@dataclass(frozen=True)
class PairConfig:
    """Two mixers side by side and the weights their outputs are mixed with."""
    left: GroupedAttentionConfig
    right: StateSpaceConfig
    left_scale: float
    right_scale: float

    def to_dict(self):
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}

    def validate(self, where):
        self.left.validate(where + "left.")
        self.right.validate(where + "right.")


@dataclass(frozen=True)
class MixtureConfig:
    expert_ff: int
    experts: int
    top: int
    identity: int
    group_count: int
    group_keep: int
    shared_ff: Optional[int]

    @classmethod
    def from_dict(cls, raw, where):
        kind = optional(raw, "kind", "moe", str)
        if kind != "moe":
            raise ConfigError(f"config.json: {where}kind {kind!r} is not 'moe'")
        router = _section(raw, "router", where)
        groups = _section(router, "groups", where + "router.", needed=False) or {}
        shared = _section(raw, "shared", where, needed=False)
        return cls(expert_ff=require(_section(raw, "expert", where), "ff"), experts=require(router, "experts"),
                   top=require(router, "top"), identity=optional(router, "identity", 0),
                   group_count=optional(groups, "count", 1), group_keep=optional(groups, "keep", optional(groups, "count", 1)),
                   shared_ff=None if shared is None else require(shared, "ff"))

    def to_dict(self):
        out = {"expert": {"ff": self.expert_ff}, "kind": "moe",
               "router": {"experts": self.experts, "groups": {"count": self.group_count, "keep": self.group_keep},
                          "identity": self.identity, "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out

    def validate(self, where):
        _positive(self, ("expert_ff", "experts", "top", "group_count", "group_keep"), where)
        total = self.experts + self.identity
        if self.identity < 0 or total % self.group_count or self.group_keep > self.group_count:
            raise ConfigError(f"config.json: {where}router: {self.group_count} groups (keep {self.group_keep}) over "
                              f"{self.experts} + {self.identity} experts")
        if self.top > self.group_keep * (total // self.group_count):
            raise ConfigError(f"config.json: {where}router.top exceeds the experts of the groups that are kept")
        if self.shared_ff is not None and self.shared_ff <= 0:
            raise ConfigError(f"config.json: {where}shared.ff must be positive")


LAYER_TYPES = ("latent_attention", "parallel")


@dataclass(frozen=True)
class PevolornLayerConfig:
    type: str
    mixer: Union[LatentConfig, PairConfig]
    mlp: Optional[MixtureConfig]


@dataclass(frozen=True)
class PevolornConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    layers: Tuple[PevolornLayerConfig, ...]
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architecture: str = field(default=ARCHITECTURE)

    MAX_POSITIONS = 1 << 20       # the design has no table that bounds the context; the cache's size does

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return self.MAX_POSITIONS

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PevolornConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = require(entry, "type", str)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type {kind!r} is not a layer of this design {list(LAYER_TYPES)}")
            m = _section(entry, "mixer", where)
            if kind == "parallel":
                mixer = PairConfig(GroupedAttentionConfig.from_dict(_section(m, "left", where + "mixer."), where + "mixer.left."),
                                   StateSpaceConfig.from_dict(_section(m, "right", where + "mixer."), where + "mixer.right."),
                                   optional(m, "left_scale", 1.0, float), optional(m, "right_scale", 1.0, float))
            else:
                mixer = LatentConfig.from_dict(m, where + "mixer.")
            mlp_raw = _section(entry, "mlp", where, needed=False)
            mlp = None if mlp_raw is None else MixtureConfig.from_dict(mlp_raw, where + "mlp.")
            layers.append(PevolornLayerConfig(kind, mixer, mlp))
        norm = _section(raw, "norm", "")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(coerce(x, "eos_token_id[]", int) for x in eos)
        else:
            eos_ids = (coerce(eos, "eos_token_id", int),)
        bos = raw.get("bos_token_id")
        return cls(vocab=require(raw, "vocab"), width=require(raw, "width"), norm_eps=require(norm, "eps", float),
                   postln_alpha=optional(raw, "postln_alpha", 1.0, float), layers=tuple(layers),
                   eos_token_ids=eos_ids, bos_token_id=None if bos is None else coerce(bos, "bos_token_id", int))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(), "type": l.type}
                       for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "postln_alpha": self.postln_alpha,
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            layer.mixer.validate(where + "mixer.")
            if layer.mlp is not None:
                layer.mlp.validate(where + "mlp.")
            m = layer.mixer
            if isinstance(m, LatentConfig) and m.kv_from is not None:
                j = m.kv_from
                src = self.layers[j].mixer if 0 <= j < len(self.layers) else None
                if j >= i or not isinstance(src, LatentConfig) or src.kv_from is not None:
                    raise ConfigError(f"config.json: {where}mixer.kv_from must name an earlier latent_attention layer "
                                      "that has a compression of its own")
                if (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base) != (m.kv_rank, m.rot_dim, m.rot_dims, m.rot_base):
                    raise ConfigError(f"config.json: {where}mixer: kv_rank, rot_dim and rot must equal layer {j}'s")
        for tok in self.eos_token_ids:
            if not 0 <= tok < self.vocab:
                raise ConfigError(f"config.json: eos_token_id {tok} is outside the vocabulary")
