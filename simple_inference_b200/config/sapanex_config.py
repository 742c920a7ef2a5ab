"""Typed configuration of the Sapanex design, read from its ``config.json``.

The file names the design with one string (``"architecture": "Sapanex"``) and lists its
layers one by one: each entry gives the kind of mixer (``type``), the mixer's sizes and
constants (``mixer``) and the feed-forward (``mlp``, or null for a layer without one).  Every
size and constant that can differ between two models of the design is a field here; what
the design fixes (activation functions, the decay's constant, the unit key's epsilon) lives
with the part that computes it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .model_config import ConfigError, ModelConfig


def _need(d: dict[str, Any], keys: tuple[str, ...], where: str) -> None:
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks keys {missing}")


def _positive_int(v: Any, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class YarnScaling:
    """``rot.scaling``: stretch ``factor``, the length the model was made for (``original``)
    and the two turn counts between which frequencies blend (``fast``, ``slow``)."""

    factor: float
    original: float
    fast: float
    slow: float

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "YarnScaling":
        _need(d, ("factor", "original", "fast", "slow"), "rot.scaling")
        out = cls(float(d["factor"]), float(d["original"]), float(d["fast"]), float(d["slow"]))
        if out.factor <= 0 or out.original <= 0 or out.fast <= 0 or out.slow <= 0:
            raise ConfigError(f"rot.scaling needs positive numbers, got {d}")
        return out

    def to_dict(self) -> dict[str, Any]:
        original = int(self.original) if float(self.original).is_integer() else self.original
        return {"factor": self.factor, "fast": self.fast, "original": original, "slow": self.slow}


@dataclass(frozen=True)
class Rotary:
    """``rot``: rotated dimensions per head, base, optional YaRN scaling."""

    dims: int
    base: float
    scaling: YarnScaling | None = None

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "Rotary":
        _need(d, ("dims", "base"), "mixer.rot")
        scaling = YarnScaling.from_dict(d["scaling"]) if d.get("scaling") else None
        dims = _positive_int(d["dims"], "rot.dims")
        if dims % 2 != 0:
            raise ConfigError(f"rot.dims must be even, got {dims}")
        if not float(d["base"]) > 1.0:
            raise ConfigError(f"rot.base must exceed 1, got {d['base']!r}")
        return cls(dims, float(d["base"]), scaling)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = self.scaling.to_dict()
        return out


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int          # size of a query or key head
    vdim: int         # size of a value head
    scale: float
    rot: Rotary | None
    window: int | None    # mask.size
    pool: int | None      # mask.pool

    kind = "attention"

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "AttentionMixerConfig":
        _need(d, ("heads", "kv_heads", "dim", "vdim", "scale"), "an attention mixer")
        heads = _positive_int(d["heads"], "heads")
        kv_heads = _positive_int(d["kv_heads"], "kv_heads")
        dim, vdim = _positive_int(d["dim"], "dim"), _positive_int(d["vdim"], "vdim")
        if heads % kv_heads != 0:
            raise ConfigError(f"{heads} query heads do not divide into {kv_heads} key/value heads")
        rot = Rotary.from_dict(d["rot"]) if d.get("rot") else None
        if rot is not None and rot.dims > dim:
            raise ConfigError(f"rot.dims {rot.dims} exceeds the head size {dim}")
        if rot is not None and vdim % 2 != 0:
            raise ConfigError(f"values are rotated in pairs: vdim must be even, got {vdim}")
        mask = d.get("mask") or {}
        window = _positive_int(mask["size"], "mask.size") if mask.get("size") else None
        pool = _positive_int(mask["pool"], "mask.pool") if mask.get("pool") else None
        if pool is not None and window is None:
            raise ConfigError("mask.pool needs mask.size: blocks are pooled once they left a window")
        return cls(heads, kv_heads, dim, vdim, float(d["scale"]), rot, window, pool)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads}
        if self.window is not None:
            out["mask"] = {"size": self.window}
            if self.pool is not None:
                out["mask"] = {"pool": self.pool, "size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        out["scale"] = self.scale
        out["vdim"] = self.vdim
        return out


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    dim: int
    # inner width of the decay's two-matrix projection.  A checkpoint's config.json does not
    # carry it (the tensor's shape says it); the random-weights mode may name it here.
    decay_rank: int | None = None

    kind = "general_delta"

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "DeltaMixerConfig":
        _need(d, ("heads", "dim"), "a general_delta mixer")
        rank = _positive_int(d["decay_rank"], "decay_rank") if d.get("decay_rank") else None
        return cls(_positive_int(d["heads"], "heads"), _positive_int(d["dim"], "dim"), rank)

    def to_dict(self) -> dict[str, Any]:
        out = {"dim": self.dim, "heads": self.heads}
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        return out


_MIXERS = {"attention": AttentionMixerConfig, "general_delta": DeltaMixerConfig}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str
    ff: int

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "FeedForwardConfig":
        _need(d, ("kind", "ff"), "mlp")
        if d["kind"] != "dense":
            raise ConfigError(f"mlp.kind {d['kind']!r}: only 'dense' is built")
        return cls(str(d["kind"]), _positive_int(d["ff"], "mlp.ff"))

    def to_dict(self) -> dict[str, Any]:
        return {"ff": self.ff, "kind": self.kind}


@dataclass(frozen=True)
class SapanexLayer:
    type: str
    mixer: AttentionMixerConfig | DeltaMixerConfig
    mlp: FeedForwardConfig | None

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "SapanexLayer":
        _need(d, ("type", "mixer"), "a layer")
        if d["type"] not in _MIXERS:
            raise ConfigError(f"layer type {d['type']!r}: known mixers are {sorted(_MIXERS)}")
        mlp = FeedForwardConfig.from_dict(d["mlp"]) if d.get("mlp") else None
        return cls(str(d["type"]), _MIXERS[d["type"]].from_dict(d["mixer"]), mlp)

    def to_dict(self) -> dict[str, Any]:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None,
                "type": self.type}


# positions are float32 in the kernels: every integer up to 2^24 is exact there
_MAX_POSITIONS = 1 << 24


@dataclass(kw_only=True)
class SapanexConfig(ModelConfig):
    """config.json of the Sapanex design."""

    vocab: int
    width: int
    layers: list = field(default_factory=list)
    embedding: dict = field(default_factory=dict)   # {"scale": s}
    norm: dict = field(default_factory=dict)        # {"eps": e}
    postln_alpha: float = 1.0
    architecture: str = "Sapanex"
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "SapanexConfig":
        _need(d, ("vocab", "width", "layers", "embedding", "norm", "postln_alpha"), "the model")
        cfg = cls(vocab=d["vocab"], width=d["width"],
                  layers=[x if isinstance(x, SapanexLayer) else SapanexLayer.from_dict(x)
                          for x in d["layers"]],
                  embedding=dict(d["embedding"]), norm=dict(d["norm"]),
                  postln_alpha=d["postln_alpha"],
                  architecture=str(d.get("architecture", "Sapanex")),
                  torch_dtype=str(d.get("torch_dtype", "bfloat16")))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        if not self.layers:
            raise ConfigError("the model has no layers")
        _need(self.embedding, ("scale",), "embedding")
        _need(self.norm, ("eps",), "norm")
        if not float(self.norm["eps"]) > 0.0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm['eps']!r}")
        self.postln_alpha = float(self.postln_alpha)
        if self.torch_dtype not in ("bfloat16", "float16", "float32"):
            raise ConfigError(f"torch_dtype {self.torch_dtype!r} is not a dtype a checkpoint is stored in")

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "embedding": dict(self.embedding),
                "layers": [layer.to_dict() for layer in self.layers], "norm": dict(self.norm),
                "postln_alpha": self.postln_alpha, "vocab": self.vocab, "width": self.width}

    # the names the command line and the engine use for every architecture
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def max_position_embeddings(self) -> int:
        return _MAX_POSITIONS

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding["scale"])
