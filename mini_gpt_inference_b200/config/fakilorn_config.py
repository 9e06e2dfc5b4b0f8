"""Typed configuration of the Fakilorn decoder, read from its ``config.json``.

The file is nested: ``vocab``, ``width``, ``logit_scale``, ``embedding.scale``, ``norm.eps`` and a
list ``layers``; each entry has ``type`` (the mixer's kind), ``mixer`` (its sizes and constants) and
``mlp`` (the feed-forward, or null for none).  Every size and constant is read from the file; a
missing key is an error, a key that this engine does not know a warning.
"""

from __future__ import annotations

import json
import warnings
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .model_config import ConfigError


def _positive_int(value, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {value!r}")
    return value


def _number(value, what: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{what} must be a number, got {value!r}")
    return float(value)


def _keys(raw: Mapping[str, Any], required, optional, what: str) -> None:
    if not isinstance(raw, Mapping):
        raise ConfigError(f"{what} must be an object, got {raw!r}")
    missing = [k for k in required if k not in raw]
    unknown = [k for k in raw if k not in required and k not in optional]
    if unknown:
        warnings.warn(f"{what}: keys not used by this architecture: " + ", ".join(sorted(unknown)), stacklevel=3)
    if missing:
        raise ConfigError(f"{what}: missing " + ", ".join(missing))


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int                 # features of a query or key head
    vdim: int                # features of a value head
    scale: float             # factor on q . k
    v_mix: bool              # whether the layer takes part in the blending of values

    @classmethod
    def from_dict(cls, raw, what: str) -> "AttentionMixerConfig":
        _keys(raw, ("heads", "kv_heads", "dim", "vdim", "scale"), ("v_mix",), what)
        heads = _positive_int(raw["heads"], what + ".heads")
        kv_heads = _positive_int(raw["kv_heads"], what + ".kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{what}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        return cls(heads, kv_heads, _positive_int(raw["dim"], what + ".dim"),
                   _positive_int(raw["vdim"], what + ".vdim"), _number(raw["scale"], what + ".scale"),
                   bool(raw.get("v_mix", False)))

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                "v_mix": self.v_mix, "vdim": self.vdim}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                          # "dense" | "moe"
    ff: int = 0                        # dense: hidden width; moe: hidden width of an expert
    experts: int = 0
    top: int = 0
    shared_ff: int | None = None       # hidden width of the expert that every token uses

    @classmethod
    def from_dict(cls, raw, what: str) -> "FeedForwardConfig":
        if not isinstance(raw, Mapping) or "kind" not in raw:
            raise ConfigError(f"{what} must be an object with a 'kind'")
        kind = raw["kind"]
        if kind == "dense":
            _keys(raw, ("kind", "ff"), (), what)
            return cls("dense", _positive_int(raw["ff"], what + ".ff"))
        if kind == "moe":
            _keys(raw, ("kind", "expert", "router"), ("shared",), what)
            _keys(raw["expert"], ("ff",), (), what + ".expert")
            _keys(raw["router"], ("experts", "top"), (), what + ".router")
            experts = _positive_int(raw["router"]["experts"], what + ".router.experts")
            top = _positive_int(raw["router"]["top"], what + ".router.top")
            if top > experts:
                raise ConfigError(f"{what}: top ({top}) exceeds experts ({experts})")
            shared = raw.get("shared")
            if shared is not None:
                _keys(shared, ("ff",), (), what + ".shared")
                shared = _positive_int(shared["ff"], what + ".shared.ff")
            return cls("moe", _positive_int(raw["expert"]["ff"], what + ".expert.ff"), experts, top, shared)
        raise ConfigError(f"{what}.kind {kind!r} is not known (dense, moe)")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        out = {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class FakilornLayerConfig:
    type: str
    mixer: AttentionMixerConfig
    mlp: FeedForwardConfig | None

    @classmethod
    def from_dict(cls, raw, what: str) -> "FakilornLayerConfig":
        _keys(raw, ("type", "mixer"), ("mlp",), what)
        if raw["type"] != "attention":
            raise ConfigError(f"{what}.type {raw['type']!r} is not a mixer of this design (attention)")
        mlp = raw.get("mlp")
        return cls("attention", AttentionMixerConfig.from_dict(raw["mixer"], what + ".mixer"),
                   None if mlp is None else FeedForwardConfig.from_dict(mlp, what + ".mlp"))

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclass(frozen=True)
class FakilornConfig:
    vocab: int
    width: int
    layers: tuple[FakilornLayerConfig, ...]
    embedding_scale: float
    logit_scale: float
    norm_eps: float
    architecture: str = "Fakilorn"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], architecture: str | None = None) -> "FakilornConfig":
        _keys(raw, ("vocab", "width", "layers", "embedding", "norm", "logit_scale"),
              ("architecture", "architectures", "model_type", "dtype", "torch_dtype"), "config.json")
        _keys(raw["embedding"], ("scale",), (), "embedding")
        _keys(raw["norm"], ("eps",), (), "norm")
        if not isinstance(raw["layers"], (list, tuple)) or not raw["layers"]:
            raise ConfigError("layers must be a list with at least one layer")
        layers = tuple(FakilornLayerConfig.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(raw["layers"]))
        eps = _number(raw["norm"]["eps"], "norm.eps")
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps!r}")
        blending = [layer.mixer for layer in layers if layer.mixer.v_mix]
        if any((m.kv_heads, m.vdim) != (blending[0].kv_heads, blending[0].vdim) for m in blending):
            raise ConfigError("layers that blend values (v_mix) must agree in kv_heads and vdim")
        return cls(_positive_int(raw["vocab"], "vocab"), _positive_int(raw["width"], "width"), layers,
                   _number(raw["embedding"]["scale"], "embedding.scale"),
                   _number(raw["logit_scale"], "logit_scale"), eps, architecture or "Fakilorn")

    @classmethod
    def from_json(cls, path: str | Path) -> "FakilornConfig":
        from .model_config import read_config_json

        path = Path(path)
        return cls.from_dict(read_config_json(path / "config.json" if path.is_dir() else path))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                "layers": [layer.to_dict() for layer in self.layers], "logit_scale": self.logit_scale,
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def num_parameters(self) -> int:
        c = self.width
        total = self.vocab * c + 2 * c
        for layer in self.layers:
            m = layer.mixer
            total += 2 * c + c * (m.heads * m.dim + m.kv_heads * (m.dim + m.vdim) + 2 * m.heads * m.vdim)
            total += 1 if m.v_mix else 0
            f = layer.mlp
            if f is None:
                continue
            total += 2 * c
            if f.kind == "dense":
                total += 2 * c * f.ff
            else:
                total += f.experts * (c + 3 * c * f.ff)
                total += 0 if f.shared_ff is None else 3 * c * f.shared_ff + c
        return total

    def save(self, model_dir: str | Path) -> Path:
        model_dir = Path(model_dir)
        model_dir.mkdir(parents=True, exist_ok=True)
        path = model_dir / "config.json"
        path.write_text(json.dumps(self.to_dict(), indent=1) + "\n")
        return path
