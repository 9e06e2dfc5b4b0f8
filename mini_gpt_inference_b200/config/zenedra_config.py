"""Typed configuration of the Zenedra decoder, read from its ``config.json``.

The file is nested: ``vocab``, ``width``, ``max_positions``, ``norm.eps``, ``embedding.bigram``
(``buckets``, ``mul_prev``, ``mul_cur``), an optional ``loop`` (``start``, ``stop``, ``times``) and a
list ``layers``; each entry has ``type`` (the mixer's kind: ``gla``, ``attention`` or ``mlstm``),
``mixer`` (its sizes and constants) and ``mlp`` (the feed-forward, or null for none).  Every size and
constant is read from the file; a missing key is an error, a key that this engine does not know a
warning.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .fakilorn_config import _keys, _number, _positive_int
from .model_config import ConfigError

MIXER_TYPES = ("gla", "attention", "mlstm")


@dataclass(frozen=True)
class ZenedraMixerConfig:
    """Sizes and constants of one mixer; fields that a kind does not have are None."""

    kind: str
    heads: int
    dim: int                          # features of a query or key head
    vdim: int                         # features of a value head
    kv_heads: int | None = None       # attention
    scale: float | None = None        # attention: factor on q . k
    mask_size: int | None = None      # attention: positions see only their own block of this many
    tau: float | None = None          # gla: decay = sigmoid(z) ** (1 / tau)
    gate_cap: float | None = None     # mlstm: soft cap of the gates' pre-activations

    @classmethod
    def from_dict(cls, kind: str, raw, what: str) -> "ZenedraMixerConfig":
        if kind == "gla":
            _keys(raw, ("heads", "dim", "vdim", "tau"), (), what)
            tau = _number(raw["tau"], what + ".tau")
            if tau <= 0:
                raise ConfigError(f"{what}.tau must be positive, got {tau!r}")
            return cls(kind, _positive_int(raw["heads"], what + ".heads"), _positive_int(raw["dim"], what + ".dim"),
                       _positive_int(raw["vdim"], what + ".vdim"), tau=tau)
        if kind == "mlstm":
            _keys(raw, ("heads", "dim", "vdim", "gate_cap"), (), what)
            cap = _number(raw["gate_cap"], what + ".gate_cap")
            if cap <= 0:
                raise ConfigError(f"{what}.gate_cap must be positive, got {cap!r}")
            return cls(kind, _positive_int(raw["heads"], what + ".heads"), _positive_int(raw["dim"], what + ".dim"),
                       _positive_int(raw["vdim"], what + ".vdim"), gate_cap=cap)
        _keys(raw, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"), (), what)
        _keys(raw["mask"], ("size",), (), what + ".mask")
        heads = _positive_int(raw["heads"], what + ".heads")
        kv_heads = _positive_int(raw["kv_heads"], what + ".kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{what}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim, vdim = _positive_int(raw["dim"], what + ".dim"), _positive_int(raw["vdim"], what + ".vdim")
        if vdim != dim:
            raise ConfigError(f"{what}: the values are the keys, so vdim ({vdim}) must equal dim ({dim})")
        return cls(kind, heads, dim, vdim, kv_heads=kv_heads, scale=_number(raw["scale"], what + ".scale"),
                   mask_size=_positive_int(raw["mask"]["size"], what + ".mask.size"))

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.kind == "gla":
            out["tau"] = self.tau
        elif self.kind == "mlstm":
            out["gate_cap"] = self.gate_cap
        else:
            out.update(kv_heads=self.kv_heads, scale=self.scale, mask={"size": self.mask_size})
        return out


@dataclass(frozen=True)
class ZenedraFeedForwardConfig:
    kind: str                          # "dense" | "moe"
    ff: int = 0                        # dense: hidden width; moe: hidden width of an expert
    limit: float = 0.0                 # moe: clamp of an expert's hidden features
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0           # factor on the chosen experts' scores
    group_count: int | None = None     # experts form this many groups of neighbours ...
    group_keep: int | None = None      # ... of which the best this many can be chosen from
    shared_ff: int | None = None       # hidden width of the expert that every token uses
    shared_limit: float | None = None

    @classmethod
    def from_dict(cls, raw, what: str) -> "ZenedraFeedForwardConfig":
        if not isinstance(raw, Mapping) or "kind" not in raw:
            raise ConfigError(f"{what} must be an object with a 'kind'")
        kind = raw["kind"]
        if kind == "dense":
            _keys(raw, ("kind", "ff"), (), what)
            return cls("dense", _positive_int(raw["ff"], what + ".ff"))
        if kind != "moe":
            raise ConfigError(f"{what}.kind {kind!r} is not known (dense, moe)")
        _keys(raw, ("kind", "expert", "router"), ("shared",), what)
        _keys(raw["expert"], ("ff", "limit"), (), what + ".expert")
        _keys(raw["router"], ("experts", "top", "scale"), ("groups",), what + ".router")
        experts = _positive_int(raw["router"]["experts"], what + ".router.experts")
        top = _positive_int(raw["router"]["top"], what + ".router.top")
        if top > experts:
            raise ConfigError(f"{what}: top ({top}) exceeds experts ({experts})")
        count = keep = None
        groups = raw["router"].get("groups")
        if groups is not None:
            _keys(groups, ("count", "keep"), (), what + ".router.groups")
            count = _positive_int(groups["count"], what + ".router.groups.count")
            keep = _positive_int(groups["keep"], what + ".router.groups.keep")
            if experts % count or keep > count:
                raise ConfigError(f"{what}: {experts} experts do not form {count} equal groups of which {keep} are kept")
            if keep * (experts // count) < top:
                raise ConfigError(f"{what}: {keep} groups of {experts // count} experts cannot give {top} choices")
        shared_ff = shared_limit = None
        shared = raw.get("shared")
        if shared is not None:
            _keys(shared, ("ff", "limit"), (), what + ".shared")
            shared_ff = _positive_int(shared["ff"], what + ".shared.ff")
            shared_limit = _number(shared["limit"], what + ".shared.limit")
        return cls("moe", _positive_int(raw["expert"]["ff"], what + ".expert.ff"),
                   _number(raw["expert"]["limit"], what + ".expert.limit"), experts, top,
                   _number(raw["router"]["scale"], what + ".router.scale"), count, keep, shared_ff, shared_limit)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        router: dict[str, Any] = {"experts": self.experts, "scale": self.route_scale, "top": self.top}
        if self.group_count is not None:
            router["groups"] = {"count": self.group_count, "keep": self.group_keep}
        out: dict[str, Any] = {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe", "router": router}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out


@dataclass(frozen=True)
class ZenedraLayerConfig:
    type: str
    mixer: ZenedraMixerConfig
    mlp: ZenedraFeedForwardConfig | None

    @classmethod
    def from_dict(cls, raw, what: str) -> "ZenedraLayerConfig":
        _keys(raw, ("type", "mixer"), ("mlp",), what)
        if raw["type"] not in MIXER_TYPES:
            raise ConfigError(f"{what}.type {raw['type']!r} is not a mixer of this design ({', '.join(MIXER_TYPES)})")
        mlp = raw.get("mlp")
        return cls(raw["type"], ZenedraMixerConfig.from_dict(raw["type"], raw["mixer"], what + ".mixer"),
                   None if mlp is None else ZenedraFeedForwardConfig.from_dict(mlp, what + ".mlp"))

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclass(frozen=True)
class ZenedraConfig:
    vocab: int
    width: int
    max_positions: int
    layers: tuple[ZenedraLayerConfig, ...]
    norm_eps: float
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    loop_start: int = 0                # layers loop_start .. loop_stop-1 run loop_times times in a row;
    loop_stop: int = 0                 # loop_times 0: the file names no loop
    loop_times: int = 0
    architecture: str = "Zenedra"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], architecture: str | None = None) -> "ZenedraConfig":
        _keys(raw, ("vocab", "width", "max_positions", "layers", "embedding", "norm"),
              ("loop", "architecture", "architectures", "model_type", "dtype", "torch_dtype"), "config.json")
        _keys(raw["embedding"], ("bigram",), (), "embedding")
        _keys(raw["embedding"]["bigram"], ("buckets", "mul_prev", "mul_cur"), (), "embedding.bigram")
        _keys(raw["norm"], ("eps",), (), "norm")
        if not isinstance(raw["layers"], (list, tuple)) or not raw["layers"]:
            raise ConfigError("layers must be a list with at least one layer")
        layers = tuple(ZenedraLayerConfig.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(raw["layers"]))
        eps = _number(raw["norm"]["eps"], "norm.eps")
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps!r}")
        b = raw["embedding"]["bigram"]
        for key in ("mul_prev", "mul_cur"):
            if not isinstance(b[key], int) or isinstance(b[key], bool) or b[key] < 0:
                raise ConfigError(f"embedding.bigram.{key} must be a non-negative integer, got {b[key]!r}")
        start = stop = times = 0
        loop = raw.get("loop")
        if loop is not None:
            _keys(loop, ("start", "stop", "times"), (), "loop")
            start, stop = loop["start"], loop["stop"]
            times = _positive_int(loop["times"], "loop.times")
            if not (isinstance(start, int) and isinstance(stop, int) and 0 <= start < stop <= len(layers)):
                raise ConfigError(f"loop: layers {start!r} .. {stop!r} are not a range of the {len(layers)} layers")
        return cls(_positive_int(raw["vocab"], "vocab"), _positive_int(raw["width"], "width"),
                   _positive_int(raw["max_positions"], "max_positions"), layers, eps,
                   _positive_int(b["buckets"], "embedding.bigram.buckets"), b["mul_prev"], b["mul_cur"],
                   start, stop, times, architecture or "Zenedra")

    @classmethod
    def from_json(cls, path: str | Path) -> "ZenedraConfig":
        from .model_config import read_config_json

        path = Path(path)
        return cls.from_dict(read_config_json(path / "config.json" if path.is_dir() else path))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture,
               "embedding": {"bigram": {"buckets": self.bigram_buckets, "mul_cur": self.bigram_mul_cur,
                                        "mul_prev": self.bigram_mul_prev}},
               "layers": [layer.to_dict() for layer in self.layers], "max_positions": self.max_positions,
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.loop_times:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out

    def run_order(self) -> list[tuple[int, int | None]]:
        """``(layer, pass)`` in the order the layers run; ``pass`` is None outside the loop."""
        n = len(self.layers)
        if not self.loop_times:
            return [(i, None) for i in range(n)]
        order: list[tuple[int, int | None]] = [(i, None) for i in range(self.loop_start)]
        for p in range(self.loop_times):
            order += [(i, p) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, None) for i in range(self.loop_stop, n)]

    def num_parameters(self) -> int:
        c = self.width
        total = self.vocab * c * 2 + (self.bigram_buckets + 1) * c + self.max_positions * c + c
        if self.loop_times:
            total += 2 * c * c + self.loop_times * c
        for layer in self.layers:
            m = layer.mixer
            total += c
            if m.kind == "attention":
                total += (m.heads + m.kv_heads) * m.dim * (c + 1) + 2 * m.dim + c * (m.heads * m.dim + 1)
            else:
                total += c * (2 * m.heads * m.dim + 3 * m.heads * m.vdim)
                if m.kind == "gla":
                    total += m.vdim      # plus the two decay matrices, whose rank the checkpoint gives
                else:
                    total += m.heads * m.vdim + 2 * m.heads * (c + 1)
            f = layer.mlp
            if f is None:
                continue
            total += c
            if f.kind == "dense":
                total += 3 * c * f.ff
            else:
                total += f.experts * (c + 1 + 3 * c * f.ff)
                total += 0 if f.shared_ff is None else 3 * c * f.shared_ff
        return total

    def save(self, model_dir: str | Path) -> Path:
        model_dir = Path(model_dir)
        model_dir.mkdir(parents=True, exist_ok=True)
        path = model_dir / "config.json"
        path.write_text(json.dumps(self.to_dict(), indent=1) + "\n")
        return path
