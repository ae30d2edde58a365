"""Configuration of the Sunosun decoder, from its ``config.json``.

``config.json`` lists the layers one by one (``layers``: ``type``, the mixer's sizes and
constants under ``mixer``, the feed-forward under ``mlp`` or null), and model-wide ``vocab``,
``width``, ``norm.eps``, ``embedding.scale``, ``logit_softcap`` and ``loop`` (``start``, ``stop``,
``times``: the layers start .. stop - 1 run ``times`` times in a row).  Layer types: ``gla`` (a gated
linear attention) and ``parallel`` (a softmax attention under ``left`` beside a gated linear
attention under ``right``, each with a factor).  Feed-forwards: ``dense`` (``ff``) or ``moe``
(``expert.ff``, ``router``: ``experts``, ``top``, ``scale``, ``groups``: ``count``, ``keep``; ``shared.ff``).
Nothing here has a default that stands for a size: what the file does not give is an error, except
the options a model may leave out (``mlp``, ``loop``, ``logit_softcap``, ``router.groups``, ``shared``).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import ConfigError, ModelConfig


def _num(j: Any, key: str, where: str, kind=float, positive: bool = True):
    v = j.get(key) if isinstance(j, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and int(v) != v) or not math.isfinite(v):
        raise ConfigError(f"config.json: {where}{key} is missing or no number")
    if positive and v <= 0:
        raise ConfigError(f"config.json: {where}{key} must be positive")
    return kind(v)


@dataclasses.dataclass(frozen=True)
class SunosunAttention:
    heads: int
    kv_heads: int
    dim: int                               # size of a query / key head
    vdim: int                              # size of a value head
    scale: float

    @classmethod
    def from_json(cls, j: Any, where: str) -> "SunosunAttention":
        if not isinstance(j, Mapping):
            raise ConfigError(f"config.json: {where[:-1]} is missing")
        a = cls(heads=_num(j, "heads", where, int), kv_heads=_num(j, "kv_heads", where, int), dim=_num(j, "dim", where, int),
                vdim=_num(j, "vdim", where, int), scale=_num(j, "scale", where))
        if a.heads % a.kv_heads != 0:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        return a

    def to_json(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


@dataclasses.dataclass(frozen=True)
class SunosunLinearAttention:
    heads: int
    dim: int                               # key channels of a head
    vdim: int                              # value numbers of a head
    tau: float                             # the decay is sigmoid(.)^(1 / tau)
    rank: int = 0                          # of the decay's two-step projection; 0: whatever the checkpoint's tensors have

    @classmethod
    def from_json(cls, j: Any, where: str) -> "SunosunLinearAttention":
        if not isinstance(j, Mapping):
            raise ConfigError(f"config.json: {where[:-1]} is missing")
        return cls(heads=_num(j, "heads", where, int), dim=_num(j, "dim", where, int), vdim=_num(j, "vdim", where, int),
                   tau=_num(j, "tau", where), rank=_num(j, "rank", where, int) if j.get("rank") is not None else 0)

    def to_json(self) -> Dict[str, Any]:
        j = dataclasses.asdict(self)
        if not self.rank:
            del j["rank"]
        return j


@dataclasses.dataclass(frozen=True)
class SunosunParallel:
    left: SunosunAttention
    right: SunosunLinearAttention
    left_scale: float
    right_scale: float

    @classmethod
    def from_json(cls, j: Any, where: str) -> "SunosunParallel":
        if not isinstance(j, Mapping):
            raise ConfigError(f"config.json: {where[:-1]} is missing")
        return cls(SunosunAttention.from_json(j.get("left"), where + "left."),
                   SunosunLinearAttention.from_json(j.get("right"), where + "right."),
                   _num(j, "left_scale", where, positive=False), _num(j, "right_scale", where, positive=False))

    def to_json(self) -> Dict[str, Any]:
        return {"left": self.left.to_json(), "right": self.right.to_json(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclasses.dataclass(frozen=True)
class SunosunMLP:
    kind: str                              # "dense" or "moe"
    ff: int                                # inner size (of every expert, for "moe")
    experts: int = 0
    top: int = 0
    scale: float = 1.0                     # factor of the chosen experts' weights
    group_count: int = 0                   # 0: the experts form no groups
    group_keep: int = 0
    shared_ff: int = 0                     # 0: no expert that every token uses

    @classmethod
    def from_json(cls, j: Mapping[str, Any], where: str) -> "SunosunMLP":
        kind = j.get("kind") if isinstance(j, Mapping) else None
        if kind == "dense":
            return cls("dense", _num(j, "ff", where, int))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}kind {kind!r} is not known (dense, moe)")
        r = j.get("router")
        g = r.get("groups") if isinstance(r, Mapping) else None
        sh = j.get("shared")
        m = cls("moe", _num(j.get("expert"), "ff", where + "expert.", int), experts=_num(r, "experts", where + "router.", int),
                top=_num(r, "top", where + "router.", int), scale=_num(r, "scale", where + "router.", positive=False),
                group_count=_num(g, "count", where + "router.groups.", int) if g is not None else 0,
                group_keep=_num(g, "keep", where + "router.groups.", int) if g is not None else 0,
                shared_ff=_num(sh, "ff", where + "shared.", int) if sh is not None else 0)
        if m.top > m.experts:
            raise ConfigError(f"config.json: {where}router.top is larger than the number of experts")
        if m.group_count:
            if m.experts % m.group_count != 0 or m.group_keep > m.group_count:
                raise ConfigError(f"config.json: {where}router.groups: {m.experts} experts do not form {m.group_count} equal groups "
                                  f"of which {m.group_keep} are kept")
            if m.group_keep * (m.experts // m.group_count) < m.top:
                raise ConfigError(f"config.json: {where}router.groups keeps fewer experts than router.top chooses")
        return m

    def to_json(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        r: Dict[str, Any] = {"experts": self.experts, "top": self.top, "scale": self.scale}
        if self.group_count:
            r["groups"] = {"count": self.group_count, "keep": self.group_keep}
        j: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff}, "router": r}
        if self.shared_ff:
            j["shared"] = {"ff": self.shared_ff}
        return j


@dataclasses.dataclass(frozen=True)
class SunosunLayer:
    type: str                                              # "gla" or "parallel"
    mixer: Any                                             # SunosunLinearAttention or SunosunParallel
    mlp: Optional[SunosunMLP]


@dataclasses.dataclass(frozen=True)
class SunosunLoop:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class SunosunConfig(ModelConfig):
    vocab_size: int = 0
    width: int = 0
    layers: Tuple[SunosunLayer, ...] = ()
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_softcap: Optional[float] = None
    loop: Optional[SunosunLoop] = None

    @property
    def vocab(self) -> int:
        return self.vocab_size

    @property
    def max_position(self) -> int:
        return 1 << 24                     # (positions enter a float32 angle: integers are exact up to here)

    def run_order(self) -> Tuple[Tuple[int, Optional[int]], ...]:
        """(layer, the number of the pass that begins with this run or None) for every layer run, in order."""
        n = len(self.layers)
        if self.loop is None:
            return tuple((i, None) for i in range(n))
        a, b = self.loop.start, self.loop.stop
        order = [(i, None) for i in range(a)]
        for t in range(self.loop.times):
            order += [(i, t if i == a else None) for i in range(a, b)]
        return tuple(order + [(i, None) for i in range(b, n)])

    def param_count(self, tied: Optional[bool] = None) -> int:
        """Number of parameters (every expert counted, a looped layer once)."""
        w = self.width
        n = self.vocab_size * w + w + (self.loop.times * w if self.loop is not None else 0)

        def linear_attention(m: SunosunLinearAttention, rank: int) -> int:
            return w * (2 * m.heads * m.dim + 3 * m.heads * m.vdim) + m.vdim + rank * (w + m.heads * m.dim) + m.heads * m.dim

        for L in self.layers:
            n += w
            if L.type == "gla":
                n += linear_attention(L.mixer, L.mixer.rank or 16)
            else:
                a = L.mixer.left
                n += (w + 1) * (a.heads * a.dim + a.kv_heads * (a.dim + a.vdim)) + w * a.heads * a.vdim
                n += linear_attention(L.mixer.right, L.mixer.right.rank or 16)
            if L.mlp is not None:
                n += w
                if L.mlp.kind == "dense":
                    n += 3 * w * L.mlp.ff
                else:
                    n += 2 * w * L.mlp.ff * L.mlp.experts + (w + 1) * L.mlp.experts + (2 * w * L.mlp.shared_ff + w if L.mlp.shared_ff else 0)
        return n

    @classmethod
    def from_json(cls, j: Mapping[str, Any], architecture: str) -> "SunosunConfig":
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: layers is missing or empty")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            kind = L.get("type") if isinstance(L, Mapping) else L
            if kind == "gla":
                mixer = SunosunLinearAttention.from_json(L.get("mixer"), where + "mixer.")
            elif kind == "parallel":
                mixer = SunosunParallel.from_json(L.get("mixer"), where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not known (gla, parallel)")
            mlp = L.get("mlp")
            layers.append(SunosunLayer(kind, mixer, SunosunMLP.from_json(mlp, where + "mlp.") if mlp is not None else None))
        loop = j.get("loop")
        if loop is not None:
            loop = SunosunLoop(_num(loop, "start", "loop.", int, positive=False), _num(loop, "stop", "loop.", int),
                               _num(loop, "times", "loop.", int))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop.start .. loop.stop must be a range of the {len(layers)} layers")
        emb = j.get("embedding")
        cap = j.get("logit_softcap")
        return cls(architecture=architecture, vocab_size=_num(j, "vocab", "", int), width=_num(j, "width", "", int),
                   layers=tuple(layers), norm_eps=_num(j.get("norm"), "eps", "norm."),
                   embedding_scale=_num(emb, "scale", "embedding.", positive=False) if emb is not None else 1.0,
                   logit_softcap=_num(j, "logit_softcap", "") if cap is not None else None, loop=loop)

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = {
            "architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": L.type, "mixer": L.mixer.to_json(), "mlp": L.mlp.to_json() if L.mlp is not None else None}
                       for L in self.layers],
            "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.width}
        if self.logit_softcap is not None:
            j["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            j["loop"] = dataclasses.asdict(self.loop)
        return j
