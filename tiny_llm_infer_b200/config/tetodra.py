"""Typed configuration of the Tetodra design, read from its own config.json keys.

config.json carries ``architecture`` (the name), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``residual_mult`` and ``layers``: per layer ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp``
(its feed-forward, or null for a layer without one).  Layer types:

``parallel``    two mixers side by side, ``mixer.left`` (attention whose values are its keys: ``heads``,
                ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``bias_max``, ``q_temp.coef``, ``q_temp.every``) and
                ``mixer.right`` (a matrix memory: ``heads``, ``dim``, ``vdim``, ``gate_cap``), mixed with
                ``mixer.left_scale`` and ``mixer.right_scale``.
``parallel_2``  ``mixer.left`` (attention with a rotation: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
                ``rot.base``, ``rot.dims``) and ``mixer.right`` (gated linear attention: ``heads``, ``dim``,
                ``vdim``, ``tau``), mixed the same way.
``delta``       the delta rule with a decay per head: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``.

Feed-forward ``dense``: ``ff``.  Two sizes come from the shapes of the checkpoint's tensors: the rows of the
attention's table of distance biases (``l<i>.mix.left.rel``) and the rank of the gated linear attention's decay
projection (``l<i>.mix.right.a1``).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Dict, Optional, Tuple, Union

from .base import ConfigError, ModelConfig, coerce, optional, require

ARCHITECTURE = "Tetodra"
DEFAULT_BIAS_ROWS = 16        # where no checkpoint says them (random weights)


def _section(raw: Dict[str, Any], key: str, where: str, needed: bool = True) -> Optional[Dict[str, Any]]:
    value = raw.get(key)
    if value is None:
        if needed:
            raise ConfigError(f"config.json: {where}{key!r} is missing")
        return None
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return value


def default_rank(width: int) -> int:
    return max(8, width // 64 * 4)


def _positive(obj, names, where: str) -> None:
    for name in names:
        if not getattr(obj, name) > 0:
            raise ConfigError(f"config.json: {where}{name} must be positive")


@dataclass(frozen=True)
class KeyValueAttentionConfig:
    """Attention whose values are its keys, with normed queries and keys, a query temperature, a table of distance
    biases and a learned sink."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: float
    temp_coef: float
    temp_every: int
    bias_rows: Optional[int] = None       # not a key of config.json: rows of the table in the checkpoint

    @classmethod
    def from_dict(cls, raw, where):
        heads = require(raw, "heads")
        temp = _section(raw, "q_temp", where)
        return cls(heads=heads, kv_heads=optional(raw, "kv_heads", heads), dim=require(raw, "dim"),
                   vdim=optional(raw, "vdim", raw.get("dim")), scale=require(raw, "scale", float),
                   bias_max=require(raw, "bias_max", float), temp_coef=require(temp, "coef", float),
                   temp_every=require(temp, "every"))

    def to_dict(self):
        return {"bias_max": self.bias_max, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "q_temp": {"coef": self.temp_coef, "every": self.temp_every}, "scale": self.scale, "vdim": self.vdim}

    def validate(self, where):
        _positive(self, ("heads", "kv_heads", "dim", "vdim", "bias_max", "temp_every"), where)
        if self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        if self.vdim != self.dim:
            raise ConfigError(f"config.json: {where}vdim must equal dim where the values are the keys")
        rows = self.bias_rows or DEFAULT_BIAS_ROWS
        if rows < 2 or not self.bias_max > rows // 2:
            raise ConfigError(f"config.json: {where}bias_max must exceed half the table's {rows} rows")


@dataclass(frozen=True)
class RotaryAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int

    @classmethod
    def from_dict(cls, raw, where):
        heads = require(raw, "heads")
        rot = _section(raw, "rot", where)
        dim = require(raw, "dim")
        return cls(heads=heads, kv_heads=optional(raw, "kv_heads", heads), dim=dim,
                   vdim=optional(raw, "vdim", dim), scale=require(raw, "scale", float),
                   rot_base=require(rot, "base", float), rot_dims=optional(rot, "dims", dim))

    def to_dict(self):
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}, "scale": self.scale, "vdim": self.vdim}

    def validate(self, where):
        _positive(self, ("heads", "kv_heads", "dim", "vdim", "rot_base", "rot_dims"), where)
        if self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim")


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, raw, where):
        return cls(heads=require(raw, "heads"), dim=require(raw, "dim"), vdim=optional(raw, "vdim", raw.get("dim")),
                   gate_cap=require(raw, "gate_cap", float))

    def to_dict(self):
        return {"dim": self.dim, "gate_cap": self.gate_cap, "heads": self.heads, "vdim": self.vdim}

    def validate(self, where):
        _positive(self, ("heads", "dim", "vdim", "gate_cap"), where)


@dataclass(frozen=True)
class GatedLinearConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: Optional[int] = None      # not a key of config.json: rows of the decay's first projection

    @classmethod
    def from_dict(cls, raw, where):
        return cls(heads=require(raw, "heads"), dim=require(raw, "dim"), vdim=optional(raw, "vdim", raw.get("dim")),
                   tau=require(raw, "tau", float))

    def to_dict(self):
        return {"dim": self.dim, "heads": self.heads, "tau": self.tau, "vdim": self.vdim}

    def validate(self, where):
        _positive(self, ("heads", "dim", "vdim", "tau"), where)


@dataclass(frozen=True)
class GatedDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, raw, where):
        heads = require(raw, "heads")
        return cls(heads=heads, kv_heads=optional(raw, "kv_heads", heads), dim=require(raw, "dim"),
                   vdim=optional(raw, "vdim", raw.get("dim")), conv=require(raw, "conv"))

    def to_dict(self):
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}

    def validate(self, where):
        _positive(self, ("heads", "kv_heads", "dim", "vdim", "conv"), where)
        if self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")


@dataclass(frozen=True)
class PairConfig:
    """Two mixers side by side and the weights their outputs are mixed with."""
    left: Union[KeyValueAttentionConfig, RotaryAttentionConfig]
    right: Union[MatrixMemoryConfig, GatedLinearConfig]
    left_scale: float
    right_scale: float

    def to_dict(self):
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}

    def validate(self, where):
        self.left.validate(where + "left.")
        self.right.validate(where + "right.")


PAIRS = {"parallel": (KeyValueAttentionConfig, MatrixMemoryConfig), "parallel_2": (RotaryAttentionConfig, GatedLinearConfig)}
LAYER_TYPES = ("parallel", "parallel_2", "delta")


@dataclass(frozen=True)
class DenseConfig:
    ff: int

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class TetodraLayerConfig:
    type: str
    mixer: Union[PairConfig, GatedDeltaConfig]
    mlp: Optional[DenseConfig]


@dataclass(frozen=True)
class TetodraConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    residual_mult: float
    layers: Tuple[TetodraLayerConfig, ...]
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
    def from_dict(cls, raw: Dict[str, Any]) -> "TetodraConfig":
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
            if kind in PAIRS:
                left_cls, right_cls = PAIRS[kind]
                mixer = PairConfig(left_cls.from_dict(_section(m, "left", where + "mixer."), where + "mixer.left."),
                                   right_cls.from_dict(_section(m, "right", where + "mixer."), where + "mixer.right."),
                                   optional(m, "left_scale", 1.0, float), optional(m, "right_scale", 1.0, float))
            else:
                mixer = GatedDeltaConfig.from_dict(m, where + "mixer.")
            mlp_raw = _section(entry, "mlp", where, needed=False)
            mlp = None
            if mlp_raw is not None:
                ff_kind = optional(mlp_raw, "kind", "dense", str)
                if ff_kind != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {ff_kind!r} is not 'dense'")
                mlp = DenseConfig(require(mlp_raw, "ff"))
            layers.append(TetodraLayerConfig(kind, mixer, mlp))
        embedding = _section(raw, "embedding", "", needed=False) or {}
        norm = _section(raw, "norm", "")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(coerce(x, "eos_token_id[]", int) for x in eos)
        else:
            eos_ids = (coerce(eos, "eos_token_id", int),)
        bos = raw.get("bos_token_id")
        return cls(vocab=require(raw, "vocab"), width=require(raw, "width"),
                   embedding_scale=optional(embedding, "scale", 1.0, float), norm_eps=require(norm, "eps", float),
                   residual_mult=optional(raw, "residual_mult", 1.0, float), layers=tuple(layers),
                   eos_token_ids=eos_ids, bos_token_id=None if bos is None else coerce(bos, "bos_token_id", int))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(), "type": l.type}
                       for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "TetodraConfig":
        """The sizes that only the checkpoint gives: the rows of a table of distance biases and the rank of a decay
        projection."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if isinstance(m, PairConfig):
                left, right = m.left, m.right
                rel, a1 = shapes.get(f"l{i}.mix.left.rel"), shapes.get(f"l{i}.mix.right.a1")
                if isinstance(left, KeyValueAttentionConfig) and rel:
                    left = replace(left, bias_rows=int(rel[0]))
                if isinstance(right, GatedLinearConfig) and a1:
                    right = replace(right, decay_rank=int(a1[0]))
                m = replace(m, left=left, right=right)
            layers.append(replace(layer, mixer=m))
        return replace(self, layers=tuple(layers))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            layer.mixer.validate(f"layers[{i}].mixer.")
            if layer.mlp is not None and layer.mlp.ff <= 0:
                raise ConfigError(f"config.json: layers[{i}].mlp.ff must be positive")
        for tok in self.eos_token_ids:
            if not 0 <= tok < self.vocab:
                raise ConfigError(f"config.json: eos_token_id {tok} is outside the vocabulary")
