"""Attention with options, and a rotation of chosen pairs.

=============  ======================  ==========================================
category       kind                    params
=============  ======================  ==========================================
position       ``rotary_pairs``        head_dim, dims (rotated elements of each
                                       head, from the first; default head_dim),
                                       theta, pairing (``neighbours``: elements
                                       2i and 2i+1 turn together; ``halves``:
                                       i and i + dims/2), scaling (None, or
                                       {"kind": "wavelength", factor, low, high,
                                       original}, or {"kind": "ramp", factor,
                                       original, fast, slow})
mixer          ``attention``           width, heads, kv_heads, head_dim, v_dim
                                       (default head_dim), bias, scale,
                                       qk_norm (None, ``head`` or ``projection``),
                                       eps, position (PartSpec), mask (None or
                                       {"kind": "block" | "window", "size": n}),
                                       sink, sink_value (a fixed score of the
                                       sink instead of learned ones),
                                       value_blend (None or {"role":
                                       "source" | "blend", "group": key}),
                                       qk_norm_weight (default True),
                                       qk_norm_after_rotation (default False),
                                       values (``own`` or ``keys``), gate,
                                       names (q, k, v, o, q_bias, k_bias, v_bias,
                                       q_norm, k_norm, sink, blend, gate -> local
                                       names)
=============  ======================  ==========================================

The mixer, for a token at position p with input h (n tokens, H query heads of size d, G
key/value heads, values of size e):

* q = Wq h (+ bq), k = Wk h (+ bk), v = Wv h (+ bv), one matrix product;
* ``qk_norm``: RMS norm of q and of k with a weight vector, either per head (a weight of
  size d shared by the heads) or over the whole projection at once (weights of size H d and
  G d), before the rotation; without ``qk_norm_weight`` the span is divided by its root mean
  square and no more (no tensors); with ``qk_norm_after_rotation`` the norm follows the rotation;
* the position encoding turns q and k;
* ``values`` = ``keys``: there is no value matrix; a head's value is its key as projected,
  before norm and rotation (so e = d);
* ``value_blend``: the layer with the role ``source`` leaves its values (per token) in the
  step's memo under ``group``; a layer with the role ``blend`` replaces its own values by
  (1 - b) v + b v_source with its learned number b; what is cached is the blended value;
* scores s_j = (q . k_j) * scale over the keys j <= p that the mask lets through: all of
  them, those in p's own block of ``size`` positions (blocks counted from position 0 of the
  sequence, wherever a prompt was cut), or the last ``size``;
* weights exp(s_j) / (sum_j exp(s_j) + exp(sink_h)): the learned sink of a head adds to the
  denominator only; with ``sink_value`` c every head's sink has the score c and there is no tensor
  (c = 0: one is added to the denominator);
* ``gate``: the heads' results, side by side, are multiplied element by element by
  sigmoid(Wg h), a matrix of H e rows that reads the mixer's own input (float32 sigmoid);
* the heads' results, side by side, go through Wo.

Everything after the projection up to the product with Wo is float32 except the stored q, k
and v, which have the compute dtype.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from .. import ops
from ..models.spec import PartSpec
from .base import CacheNeed, Mixer, Position, TensorSpec, build_part, register_part
from .linear import Linear
from .standard import NoPosition


def scaled_frequencies(dims: int, theta: float, scaling) -> Tuple[List[float], float]:
    """The frequencies f_i = theta^(-2i/dims), i < dims/2, changed by ``scaling``, and the
    factor of cos and sin (1 unless the scaling has one); float64 arithmetic.

    ``wavelength`` (the Llama 3.1 rule): with l = 2 pi / f, a frequency stays where
    l < original / high, is divided by ``factor`` where l > original / low, and between the
    two is (1 - s) f / factor + s f with s = (original / l - low) / (high - low).

    ``ramp`` (the YaRN rule): with index(t) = dims ln(original / (2 pi t)) / (2 ln theta),
    lo = max(floor(index(fast)), 0), hi = min(ceil(index(slow)), dims - 1) and
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency becomes
    f_i / factor * r_i + f_i (1 - r_i), and cos and sin are multiplied by 0.1 ln(factor) + 1."""
    freqs = [theta ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return freqs, 1.0
    sc, kind = dict(scaling), dict(scaling).get("kind")
    if kind == "wavelength":
        out = []
        for f in freqs:
            l = 2.0 * math.pi / f
            if l > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif l >= sc["original"] / sc["high"]:
                t = (sc["original"] / l - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - t) * f / sc["factor"] + t * f
            out.append(f)
        return out, 1.0
    if kind == "ramp":
        def index(turns):
            return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
        lo, hi = max(math.floor(index(sc["fast"])), 0), min(math.ceil(index(sc["slow"])), dims - 1)
        out = []
        for i, f in enumerate(freqs):
            r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / sc["factor"] * r + f * (1.0 - r))
        return out, 0.1 * math.log(sc["factor"]) + 1.0
    raise ValueError(f"unknown frequency scaling {kind!r} (wavelength, ramp)")


class RotaryPairs(Position):
    """Pairs of the first ``dims`` elements of every head turn by ``position * theta^(-2i/dims)``,
    i counting the pairs; the other elements pass.  The frequencies (after ``scaling``, see
    :func:`scaled_frequencies`) are evaluated in float64 and rounded to float32 once; the angle
    is their float32 product with the position."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.head_dim = int(params["head_dim"])
        self.dims = int(params.get("dims") or self.head_dim)
        self.theta = float(params["theta"])
        self.pairing = str(params.get("pairing", "neighbours"))
        if self.pairing not in ops.PAIRINGS:
            raise ValueError(f"unknown pairing {self.pairing} ({', '.join(ops.PAIRINGS)})")
        if self.dims % 2 != 0 or not 0 < self.dims <= self.head_dim:
            raise ValueError(f"{self.dims} rotated elements of a head of {self.head_dim}")
        sc = params.get("scaling")
        self.scaling = tuple(sorted(dict(sc).items())) if sc else ()
        inv, self.amplitude = scaled_frequencies(self.dims, self.theta, sc)
        self.inv_freq = torch.tensor(inv, dtype=torch.float64).to(torch.float32).to(ctx.device)

    def rotary_inv_freq(self):
        return None                      # (not the whole-head half-split form that the fused q/k kernel knows)

    def tables(self, batch):
        """cos/sin [tokens, dims/2] of this step, computed once and shared by every layer that turns alike."""
        key = ("rotary_pairs", self.dims, self.theta, self.scaling)
        t = batch.memo.get(key)
        if t is None:
            t = batch.memo[key] = ops.rope_table(batch.positions, self.inv_freq, self.amplitude)
        return t

    def apply(self, q, k, positions):
        cos, sin = ops.rope_table(positions, self.inv_freq, self.amplitude)
        half = self.dims // 2
        for x in (q, k):
            r = x[..., :self.dims]
            if self.pairing == "neighbours":
                u, v = r[..., 0::2], r[..., 1::2]
            else:
                u, v = r[..., :half], r[..., half:]
            c, s = cos[:, None, :], sin[:, None, :]
            nu, nv = u * c - v * s, v * c + u * s
            u.copy_(nu)
            v.copy_(nv)


class Attention(Mixer):
    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.width, self.heads, self.kv_heads = int(p["width"]), int(p["heads"]), int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.v_dim = int(p.get("v_dim") or self.head_dim)
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads != 0:
            raise ValueError("heads must be a positive multiple of kv_heads")
        if self.v_dim > 256:
            raise ValueError(f"the attention kernel takes values of up to 256 elements, not {self.v_dim}")
        self.q_dim, self.k_dim, self.v_all = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.kv_heads * self.v_dim
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.head_dim ** -0.5
        self.bias = bool(p.get("bias", False))
        self.qk_norm = p.get("qk_norm")
        if self.qk_norm not in (None, "head", "projection"):
            raise ValueError(f"qk_norm is None, 'head' or 'projection', not {self.qk_norm!r}")
        self.qk_norm_weight = bool(p.get("qk_norm_weight", True))
        self.norm_after_rotation = bool(p.get("qk_norm_after_rotation", False))
        self.values = str(p.get("values", "own"))
        if self.values not in ("own", "keys"):
            raise ValueError(f"values are 'own' or 'keys', not {self.values!r}")
        self.keys_are_values = self.values == "keys"
        if self.keys_are_values and self.v_dim != self.head_dim:
            raise ValueError("keys that are the values have the values' size")
        self.has_gate = bool(p.get("gate", False))
        self.eps = float(p.get("eps", 0.0))
        mask = p.get("mask")
        self.mask, self.mask_size = "causal", 0
        if mask is not None:
            self.mask, self.mask_size = str(mask["kind"]), int(mask["size"])
            if self.mask not in ("block", "window") or self.mask_size <= 0:
                raise ValueError(f"a mask is a block or a window of a positive size, not {mask}")
        self.sink_value = float(p["sink_value"]) if p.get("sink_value") is not None else None
        self.has_sink = bool(p.get("sink", False)) and self.sink_value is None
        self.blend = p.get("value_blend")
        if self.blend is not None and self.blend.get("role") not in ("source", "blend"):
            raise ValueError(f"value_blend's role is 'source' or 'blend', not {self.blend}")
        if self.keys_are_values:
            if self.blend is not None or self.bias:
                raise ValueError("keys that are the values are neither blended nor biased")
            self.v_all = 0                       # (no rows of the projection)
        self.gate_dim = self.heads * self.v_dim if self.has_gate else 0
        self.position = build_part("position", p.get("position") or PartSpec("none"), ctx)
        if not isinstance(self.position, (RotaryPairs, NoPosition)):
            raise ValueError("this mixer's kernel turns pairs (rotary_pairs) or nothing")
        names = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight", q_bias="q_proj.bias",
                     k_bias="k_proj.bias", v_bias="v_proj.bias", q_norm="q_norm.weight", k_norm="k_norm.weight",
                     sink="sinks", blend="value_blend", gate="gate_proj.weight")
        names.update(p.get("names") or {})
        self.names = names
        self.qkv = Linear(self.q_dim + self.k_dim + self.v_all + self.gate_dim, self.width, ctx)   # rows: q, k, v, gate
        self.o = Linear(self.width, self.heads * self.v_dim, ctx)
        self.qkv_bias = self.q_weight = self.k_weight = self.sink = self.blend_factor = None

    # ---- tensors ----
    def _norm_sizes(self):
        return (self.head_dim, self.head_dim) if self.qk_norm == "head" else (self.q_dim, self.k_dim)

    def tensor_specs(self):
        nm = self.names
        specs = [TensorSpec(nm["q"], (self.q_dim, self.width)), TensorSpec(nm["k"], (self.k_dim, self.width))]
        if not self.keys_are_values:
            specs.append(TensorSpec(nm["v"], (self.v_all, self.width)))
        if self.has_gate:
            specs.append(TensorSpec(nm["gate"], (self.gate_dim, self.width)))
        specs.append(TensorSpec(nm["o"], (self.width, self.heads * self.v_dim)))
        if self.bias:
            specs += [TensorSpec(nm["q_bias"], (self.q_dim,), "vector", init="around_zero"),
                      TensorSpec(nm["k_bias"], (self.k_dim,), "vector", init="around_zero"),
                      TensorSpec(nm["v_bias"], (self.v_all,), "vector", init="around_zero")]
        if self.qk_norm is not None and self.qk_norm_weight:
            qn, kn = self._norm_sizes()
            specs += [TensorSpec(nm["q_norm"], (qn,), "vector"), TensorSpec(nm["k_norm"], (kn,), "vector")]
        if self.has_sink:
            specs.append(TensorSpec(nm["sink"], (self.heads,), "vector", init="around_zero"))
        if self.blend is not None:
            # (the source layer's number exists in a checkpoint too; it is loaded and never used)
            specs.append(TensorSpec(nm["blend"], (), "vector", init="unit_interval"))
        return specs

    def load(self, fetch):
        nm, hold = self.names, self.ctx.hold
        self.qkv.load_rows([fetch(nm["q"]), fetch(nm["k"])] + ([] if self.keys_are_values else [fetch(nm["v"])])
                           + ([fetch(nm["gate"])] if self.has_gate else []))
        self.o.load_rows([fetch(nm["o"])])
        if self.bias:
            self.qkv_bias = torch.cat([hold(fetch(nm[k]), "vector") for k in ("q_bias", "k_bias", "v_bias")])
        if self.qk_norm is not None and self.qk_norm_weight:
            self.q_weight, self.k_weight = hold(fetch(nm["q_norm"]), "vector"), hold(fetch(nm["k_norm"]), "vector")
        if self.has_sink:
            self.sink = hold(fetch(nm["sink"]), "vector")
        elif self.sink_value is not None:
            self.sink = torch.full((self.heads,), self.sink_value, dtype=torch.float32, device=self.ctx.device)
        if self.blend is not None:
            self.blend_factor = hold(fetch(nm["blend"]), "vector").reshape(1)

    def tensor(self, name):
        nm, q, k = self.names, self.q_dim, self.k_dim
        if name == nm["q"]:
            return self.qkv.rows(0, q)
        if name == nm["k"]:
            return self.qkv.rows(q, q + k)
        if name == nm["v"] and not self.keys_are_values:
            return self.qkv.rows(q + k, q + k + self.v_all)
        if self.has_gate and name == nm["gate"]:
            return self.qkv.rows(q + k + self.v_all, q + k + self.v_all + self.gate_dim)
        if name == nm["o"]:
            return self.o.rows(0, self.width)
        if self.bias and name in (nm["q_bias"], nm["k_bias"], nm["v_bias"]):
            lo, hi = {nm["q_bias"]: (0, q), nm["k_bias"]: (q, q + k), nm["v_bias"]: (q + k, q + k + self.v_all)}[name]
            return self.qkv_bias[lo:hi].contiguous()
        if self.q_weight is not None and name == nm["q_norm"]:
            return self.q_weight
        if self.k_weight is not None and name == nm["k_norm"]:
            return self.k_weight
        if self.has_sink and name == nm["sink"]:
            return self.sink
        if self.blend is not None and name == nm["blend"]:
            return self.blend_factor.reshape(())
        return None

    def cache_need(self):
        return CacheNeed("paged_kv", kv_heads=self.kv_heads, head_dim=self.head_dim,
                         v_head_dim=None if self.v_dim == self.head_dim else self.v_dim)

    def weight_bytes(self):
        return self.qkv.weight_bytes() + self.o.weight_bytes()

    # ---- forward ----
    def forward(self, x, batch, cache, write_cache):
        n = x.shape[0]
        parts = self.qkv.forward_delta(x)                 # float32 [splits, n, H d + G d + G e + gate's H e]
        q_span, k_span = self._norm_sizes() if self.qk_norm is not None else (0, 0)
        v_keep, v_mode = None, 0
        if self.blend is not None:
            key = ("value_blend", self.blend.get("group"))
            if self.blend["role"] == "source":
                v_keep = batch.memo[key] = torch.empty((n, self.v_all), dtype=torch.float32, device=x.device)
                v_mode = 1
            else:
                v_keep = batch.memo.get(key)
                if v_keep is None:
                    raise RuntimeError(f"no layer before this one left its values under {key[1]!r}")
                v_mode = 2
        rot = self.position if isinstance(self.position, RotaryPairs) else None
        cos, sin = rot.tables(batch) if rot else (None, None)
        q = ops.qkv_finish(
            parts, self.heads, self.kv_heads, self.head_dim, self.v_dim, dtype=self.ctx.dtype, bias=self.qkv_bias,
            q_weight=self.q_weight, k_weight=self.k_weight, eps=self.eps,
            cos=cos, sin=sin, rot_dims=rot.dims if rot else 0,
            pairing=rot.pairing if rot else "neighbours", v_keep=v_keep, v_mode=v_mode, blend=self.blend_factor,
            kv=cache.kv, page_table=batch.page_table, seq_of_token=batch.seq_of_token, positions=batch.positions,
            write_kv=write_cache, q_span=q_span, k_span=k_span, norm_after_rotation=self.norm_after_rotation,
            keys_are_values=self.keys_are_values)
        att = ops.attention_masked(q, cache.kv, batch, self.scale, n_kv=self.kv_heads, v_dim=self.v_dim, mask=self.mask,
                                   mask_size=self.mask_size, sink=self.sink)
        att = att.view(n, self.heads * self.v_dim)
        if self.has_gate:
            ops.gate_rows_(att, parts, self.q_dim + self.k_dim + self.v_all)
        return self.o.forward_delta(att)


register_part("position", "rotary_pairs", RotaryPairs)
register_part("mixer", "attention", Attention)
