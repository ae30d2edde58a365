"""Configuration of the Fasunex decoder, from its ``config.json``.

``config.json`` lists the layers one by one (``layers``: ``type``, the mixer's sizes and
constants under ``mixer``, the feed-forward under ``mlp`` or null), and model-wide ``vocab``,
``width``, ``norm.eps`` and ``loop`` (``start``, ``stop``, ``times``: the layers start .. stop - 1
run ``times`` times in a row).  Layer types: ``attention`` (keys double as values) and
``parallel`` (a chunked attention under ``left`` beside a state-space recurrence under ``right``,
each with a factor).  Nothing here has a default that stands for a size: what the file does not
give is an error, except the options a layer may leave out (``mask``, ``rot``, ``router.identity``,
``mlp``, ``loop``).
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
class FasunexAttention:
    heads: int
    kv_heads: int
    dim: int                               # size of a query / key head
    vdim: int                              # size of a value head
    scale: float
    mask_size: Optional[int] = None        # positions per chunk; None: every earlier key
    rot_dims: int = 0                      # turned elements per head; 0: no rotation
    rot_base: float = 10000.0

    @classmethod
    def from_json(cls, j: Any, where: str, keys_are_values: bool) -> "FasunexAttention":
        if not isinstance(j, Mapping):
            raise ConfigError(f"config.json: {where[:-1]} is missing")
        mask, rot = (None, None) if keys_are_values else (j.get("mask"), j.get("rot"))
        a = cls(heads=_num(j, "heads", where, int), kv_heads=_num(j, "kv_heads", where, int), dim=_num(j, "dim", where, int),
                vdim=_num(j, "vdim", where, int), scale=_num(j, "scale", where),
                mask_size=_num(mask, "size", where + "mask.", int) if mask is not None else None,
                rot_dims=_num(rot, "dims", where + "rot.", int) if rot is not None else 0,
                rot_base=_num(rot, "base", where + "rot.") if rot is not None else 10000.0)
        if a.heads % a.kv_heads != 0:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        if a.rot_dims % 2 != 0 or a.rot_dims > a.dim:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim")
        if keys_are_values and a.vdim != a.dim:
            raise ConfigError(f"config.json: {where}vdim must equal dim where the keys are the values")
        return a

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale)
        if self.mask_size is not None:
            j["mask"] = {"size": self.mask_size}
        if self.rot_dims:
            j["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return j


@dataclasses.dataclass(frozen=True)
class FasunexStateSpace:
    heads: int
    vdim: int                              # numbers per head
    state: int                             # state size N
    groups: int                            # groups that share B and C
    conv: int                              # taps of the short convolution
    norm_groups: int                       # equal parts the gated result is normed in

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def channels(self) -> int:             # what passes the convolution: x, B, C
        return self.inner + 2 * self.groups * self.state

    @classmethod
    def from_json(cls, j: Any, where: str) -> "FasunexStateSpace":
        if not isinstance(j, Mapping):
            raise ConfigError(f"config.json: {where[:-1]} is missing")
        s = cls(**{k: _num(j, k, where, int) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")})
        if s.heads % s.groups != 0:
            raise ConfigError(f"config.json: {where}heads must be a multiple of groups")
        if s.inner % s.norm_groups != 0:
            raise ConfigError(f"config.json: {where}heads * vdim must be a multiple of norm_groups")
        return s

    def to_json(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


@dataclasses.dataclass(frozen=True)
class FasunexParallel:
    left: FasunexAttention
    right: FasunexStateSpace
    left_scale: float
    right_scale: float

    @classmethod
    def from_json(cls, j: Any, where: str) -> "FasunexParallel":
        if not isinstance(j, Mapping):
            raise ConfigError(f"config.json: {where[:-1]} is missing")
        return cls(FasunexAttention.from_json(j.get("left"), where + "left.", False),
                   FasunexStateSpace.from_json(j.get("right"), where + "right."),
                   _num(j, "left_scale", where, positive=False), _num(j, "right_scale", where, positive=False))

    def to_json(self) -> Dict[str, Any]:
        return {"left": self.left.to_json(), "right": self.right.to_json(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclasses.dataclass(frozen=True)
class FasunexMoE:
    ff: int                                # inner size of every expert
    experts: int                           # experts with matrices
    top: int
    identity: int = 0                      # further router outputs whose expert returns its input

    @classmethod
    def from_json(cls, j: Mapping[str, Any], where: str) -> "FasunexMoE":
        if j.get("kind") != "moe":
            raise ConfigError(f"config.json: {where}kind {j.get('kind')!r} is not known (moe)")
        r = j.get("router")
        ident = r.get("identity") if isinstance(r, Mapping) else None
        m = cls(ff=_num(j.get("expert"), "ff", where + "expert.", int), experts=_num(r, "experts", where + "router.", int),
                top=_num(r, "top", where + "router.", int),
                identity=_num(r, "identity", where + "router.", int, positive=False) if ident is not None else 0)
        if m.identity < 0 or m.top > m.experts + m.identity:
            raise ConfigError(f"config.json: {where}router.top is larger than the router's outputs")
        return m

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}


@dataclasses.dataclass(frozen=True)
class FasunexLayer:
    type: str                                              # "attention" or "parallel"
    mixer: Any                                             # FasunexAttention or FasunexParallel
    mlp: Optional[FasunexMoE]


@dataclasses.dataclass(frozen=True)
class FasunexLoop:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class FasunexConfig(ModelConfig):
    vocab_size: int = 0
    width: int = 0
    layers: Tuple[FasunexLayer, ...] = ()
    norm_eps: float = 1e-6
    loop: Optional[FasunexLoop] = None

    @property
    def vocab(self) -> int:
        return self.vocab_size

    @property
    def max_position(self) -> int:
        return 1 << 30                     # (the design names no limit; positions are 32-bit integers)

    def run_order(self) -> Tuple[Tuple[int, bool], ...]:
        """(layer, whether a pass of the loop begins with it) for every layer run, in order."""
        n = len(self.layers)
        if self.loop is None:
            return tuple((i, False) for i in range(n))
        a, b = self.loop.start, self.loop.stop
        order = [(i, False) for i in range(a)]
        for _ in range(self.loop.times):
            order += [(i, i == a) for i in range(a, b)]
        return tuple(order + [(i, False) for i in range(b, n)])

    def param_count(self, tied: Optional[bool] = None) -> int:
        """Number of parameters (every expert counted, a looped layer once)."""
        w = self.width
        n = 2 * self.vocab_size * w + w + (2 * w * w if self.loop is not None else 0)

        def attention(m: FasunexAttention, own_values: bool) -> int:
            q, k, v = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim
            return w * (q + k + (v if own_values else 0)) + 2 * w * m.heads * m.vdim + m.heads + (0 if own_values else 2 * m.dim)

        for L in self.layers:
            n += 2 * w
            if L.type == "attention":
                n += attention(L.mixer, False)
            else:
                r = L.mixer.right
                n += attention(L.mixer.left, True)
                n += w * (2 * r.inner + 2 * r.groups * r.state + r.heads) + r.channels * (r.conv + 1) + 3 * r.heads + r.inner + w * r.inner
            if L.mlp is not None:
                n += 2 * w + 3 * w * L.mlp.ff * L.mlp.experts + (w + 1) * (L.mlp.experts + L.mlp.identity)
        return n

    @classmethod
    def from_json(cls, j: Mapping[str, Any], architecture: str) -> "FasunexConfig":
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: layers is missing or empty")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            kind = L.get("type") if isinstance(L, Mapping) else L
            if kind == "attention":
                mixer = FasunexAttention.from_json(L.get("mixer"), where + "mixer.", True)
            elif kind == "parallel":
                mixer = FasunexParallel.from_json(L.get("mixer"), where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not known (attention, parallel)")
            mlp = L.get("mlp")
            layers.append(FasunexLayer(kind, mixer, FasunexMoE.from_json(mlp, where + "mlp.") if mlp is not None else None))
        loop = j.get("loop")
        if loop is not None:
            loop = FasunexLoop(_num(loop, "start", "loop.", int, positive=False), _num(loop, "stop", "loop.", int),
                               _num(loop, "times", "loop.", int))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop.start .. loop.stop must be a range of the {len(layers)} layers")
        return cls(architecture=architecture, vocab_size=_num(j, "vocab", "", int), width=_num(j, "width", "", int),
                   layers=tuple(layers), norm_eps=_num(j.get("norm"), "eps", "norm."), loop=loop)

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [{"type": L.type, "mixer": L.mixer.to_json(), "mlp": L.mlp.to_json() if L.mlp is not None else None}
                       for L in self.layers],
            "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.width}
        if self.loop is not None:
            j["loop"] = dataclasses.asdict(self.loop)
        return j
