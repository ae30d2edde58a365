"""The parts the Qwen3 dense decoder is put together from.

Each class takes its sizes and constants from ``params`` and nothing else:

=============  ======================  ==========================================
category       kind                    params
=============  ======================  ==========================================
norm           ``rms``                 width, eps, offset (added to the stored
                                       weight, default 0), tensor (its local
                                       name, default "weight"), optional
norm           ``tanh``                width, tensor, names (bias, alpha ->
                                       local names), optional
position       ``rotary_half_split``   head_dim, theta
position       ``none``                —
mixer          ``gqa_attention``       width, heads, kv_heads, head_dim,
                                       qk_norm (PartSpec or None),
                                       position (PartSpec), scale (or None)
ffn            ``gated_mlp``           width, intermediate, activation ("silu"),
                                       names (gate, up, down -> local names)
block          ``prenorm_residual``    width and layer_scale (mixer, ffn -> local
                                       names of the two factors) where the
                                       sublayers' results are scaled; post_norm
                                       (mixer, ffn -> local names, eps) where
                                       they are normed before the sum
block          ``postnorm_residual``   alpha
embedding      ``table``               vocab, width, tensor, scale (a factor of
                                       the rows, default 1), position (None or
                                       {"kind": "sinusoid", "base": b}: a vector
                                       per position that is added)
head           ``linear``              vocab, width, tied, tensor, soft_cap
=============  ======================  ==========================================

Further mixers and position encodings live in ``parts/attention.py``, further
feed-forwards in ``parts/feedforward.py``.

Formulas and their place in wick: RMS norm ``src/kernels.rs:343-357``; rotation
``src/model.rs:404-414`` with ``inv_freq`` from ``src/config.rs:162-167``;
attention ``src/model.rs:452-487,520-553``; SwiGLU MLP ``src/model.rs:490-503``;
output head ``src/model.rs:508-515`` with the tie rule of ``src/model.rs:190``.
"""
from __future__ import annotations

import math
from typing import Any, List, Mapping, Optional

import torch

from .. import ops
from ..models.spec import PartSpec
from .base import (Block, BuildContext, CacheNeed, Embedding, FeedForward, Fetch, Head, Hidden, Mixer,
                   Norm, Part, Position, TensorSpec, as_splits, build_part, register_part)
from .linear import Linear


# ---------------------------------------------------------------------------
class RMSNorm(Norm):
    """x / sqrt(mean(x^2) + eps) * (offset + w).  ``offset`` 1 is the form whose weight is
    stored as its distance from one; the sum is made once, in float32, when the weight is
    loaded.  ``optional``: the tensor may be absent; the norm then has no weight and must
    not be run (its owner asks :attr:`present`)."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.offset = float(params.get("offset", 0.0))
        self.name = str(params.get("tensor", "weight"))
        self.optional = bool(params.get("optional", False))
        self.stored: Optional[torch.Tensor] = None      # as the checkpoint has it
        self.weight: Optional[torch.Tensor] = None      # offset + stored: the factor

    @property
    def present(self) -> bool:
        return self.weight is not None

    def tensor_specs(self):
        init = "absent" if self.optional else ("around_zero" if self.offset else "")
        return [TensorSpec(self.name, (self.width,), "vector", optional=self.optional, init=init)]

    def load(self, fetch):
        w = fetch(self.name)
        if w is None and self.optional:
            self.stored = self.weight = None
            return
        self.stored = self.ctx.hold(w, "vector")
        self.weight = self.stored + self.offset if self.offset else self.stored

    def tensor(self, name):
        return self.stored if name == self.name else None

    def forward(self, x, out_dtype, rows=None):
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, rows=rows)

    def add_forward(self, x, delta, out_dtype, rows=None, *, scale=None, rms=None):
        if scale is not None or rms is not None:              # (the stream's own kernel: the sum's factor or norm, then this norm)
            return ops.stream_update(x, delta, scale=scale, rms=rms, norm=("rms", self.weight, self.eps),
                                     out_dtype=out_dtype, rows=rows)
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, delta=delta, rows=rows)

    def scaled_add_forward(self, x, delta, alpha, out_dtype):
        return ops.scaled_add_rmsnorm(x, delta, alpha, self.weight, self.eps, out_dtype)

    def weight_bytes(self):
        return self.width * 4


class TanhNorm(Norm):
    """tanh(alpha x) * w + b with one learned number alpha: a norm that computes no mean and
    no variance.  Evaluated in float32.  The three tensors are stored under ``tensor`` (w)
    and the local names ``names`` gives for ``bias`` and ``alpha``."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.name = str(params.get("tensor", "weight"))
        names = dict(bias="bias", alpha="alpha")
        names.update(params.get("names") or {})
        self.names = names
        self.optional = bool(params.get("optional", False))
        self.weight = self.bias = self.alpha = None

    @property
    def present(self) -> bool:
        return self.weight is not None

    def tensor_specs(self):
        o, init = self.optional, ("absent" if self.optional else "")
        return [TensorSpec(self.name, (self.width,), "vector", optional=o, init=init),
                TensorSpec(self.names["bias"], (self.width,), "vector", optional=o, init=init or "around_zero"),
                TensorSpec(self.names["alpha"], (), "vector", optional=o, init=init or "unit_interval")]

    def load(self, fetch):
        w = fetch(self.name)
        if w is None and self.optional:
            self.weight = self.bias = self.alpha = None
            return
        hold = self.ctx.hold
        self.weight, self.bias = hold(w, "vector"), hold(fetch(self.names["bias"]), "vector")
        self.alpha = hold(fetch(self.names["alpha"]), "vector").reshape(1)

    def tensor(self, name):
        if name == self.name:
            return self.weight
        if name == self.names["bias"]:
            return self.bias
        return self.alpha.reshape(()) if name == self.names["alpha"] and self.alpha is not None else None

    def _norm(self):
        return ("tanh", self.alpha, self.weight, self.bias)

    def forward(self, x, out_dtype, rows=None):
        return ops.stream_update(x, None, norm=self._norm(), out_dtype=out_dtype, rows=rows)

    def add_forward(self, x, delta, out_dtype, rows=None, *, scale=None, rms=None):
        return ops.stream_update(x, delta, scale=scale, rms=rms, norm=self._norm(), out_dtype=out_dtype, rows=rows)

    def weight_bytes(self):
        return (2 * self.width + 1) * 4


# ---------------------------------------------------------------------------
class RotaryHalfSplit(Position):
    """Whole-head rotation of the pairs (i, i + head_dim/2) by the angle
    ``position * inv_freq[i]`` with ``inv_freq[i] = theta ** (-2i / head_dim)``,
    evaluated in float64 and rounded to float32 once."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        d = self.head_dim
        inv = [1.0 / (self.theta ** (2.0 * i / d)) for i in range(d // 2)]
        self.inv_freq = torch.tensor(inv, dtype=torch.float64).to(torch.float32).to(ctx.device)

    def rotary_inv_freq(self):
        return self.inv_freq

    def tables(self, batch):
        """cos/sin [tokens, head_dim/2] of this step, computed once and shared by
        every layer that uses an equal encoding."""
        key = ("rotary_half_split", self.head_dim, self.theta)
        t = batch.memo.get(key)
        if t is None:
            t = batch.memo[key] = ops.rope_table(batch.positions, self.inv_freq)
        return t


class NoPosition(Position):
    PROMPT_CAPTURABLE = True

    def rotary_inv_freq(self):
        return None

    def apply(self, q, k, positions):
        return None


# ---------------------------------------------------------------------------
class GQAttention(Mixer):
    """Causal attention with grouped key/value heads over a paged cache.

    q, k, v = x Wq^T, x Wk^T, x Wv^T (no bias); optional per-head norm of q and k
    (one weight vector shared by all heads) before the position encoding; k and v
    are appended to the cache; every new token attends to positions 0..its own;
    the result goes through Wo.  The three projections are held as one matrix.
    """

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.width, self.heads, self.kv_heads, self.head_dim = (int(p["width"]), int(p["heads"]),
                                                                int(p["kv_heads"]), int(p["head_dim"]))
        if self.heads % self.kv_heads != 0:
            raise ValueError("heads must be a multiple of kv_heads")
        if self.head_dim % 16 != 0 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"the attention kernels take a head_dim that is a multiple of 16 between 16 and 256, "
                             f"not {self.head_dim}")
        self.q_dim, self.kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = p.get("window")
        if self.window is not None:
            raise ValueError("windowed attention is not built")
        qk = p.get("qk_norm")
        self.q_norm = build_part("norm", qk, ctx) if qk is not None else None
        self.k_norm = build_part("norm", qk, ctx) if qk is not None else None
        if qk is not None and not isinstance(self.q_norm, RMSNorm):
            raise ValueError("the fused q/k norm kernel is an RMS norm; another norm needs its own kernel")
        self.position = build_part("position", p.get("position") or PartSpec("none"), ctx)
        self.PROMPT_CAPTURABLE = bool(self.position.PROMPT_CAPTURABLE)   # (its own kernels read the step from the device)
        self.qkv = Linear(self.q_dim + 2 * self.kv_dim, self.width, ctx)
        self.o = Linear(self.width, self.q_dim, ctx)

    def tensor_specs(self):
        specs = [TensorSpec("q_proj.weight", (self.q_dim, self.width)),
                 TensorSpec("k_proj.weight", (self.kv_dim, self.width)),
                 TensorSpec("v_proj.weight", (self.kv_dim, self.width)),
                 TensorSpec("o_proj.weight", (self.width, self.q_dim))]
        if self.q_norm is not None:
            specs += [TensorSpec("q_norm." + s.name, s.shape, s.role) for s in self.q_norm.tensor_specs()]
            specs += [TensorSpec("k_norm." + s.name, s.shape, s.role) for s in self.k_norm.tensor_specs()]
        return specs

    def load(self, fetch):
        self.qkv.load_rows([fetch("q_proj.weight"), fetch("k_proj.weight"), fetch("v_proj.weight")])
        self.o.load_rows([fetch("o_proj.weight")])
        if self.q_norm is not None:
            self.q_norm.load(lambda n: fetch("q_norm." + n))
            self.k_norm.load(lambda n: fetch("k_norm." + n))

    def tensor(self, name):
        q, kv = self.q_dim, self.kv_dim
        if name in ("q_proj.weight", "k_proj.weight", "v_proj.weight"):
            lo, hi = {"q": (0, q), "k": (q, q + kv), "v": (q + kv, q + 2 * kv)}[name[0]]
            return self.qkv.rows(lo, hi)
        if name == "o_proj.weight":
            return self.o.rows(0, self.width)
        for prefix, norm in (("q_norm.", self.q_norm), ("k_norm.", self.k_norm)):
            if name.startswith(prefix) and norm is not None:
                return norm.tensor(name[len(prefix):])
        return None

    def cache_need(self):
        return CacheNeed("paged_kv", kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def weight_bytes(self):
        return self.qkv.weight_bytes() + self.o.weight_bytes() + (2 * self.head_dim * 4 if self.q_norm else 0)

    ADDS_TO_RESIDUAL = True

    def forward(self, x, batch, cache, write_cache, residual=None):
        inv_freq = self.position.rotary_inv_freq()
        if inv_freq is None and not isinstance(self.position, NoPosition):
            q = self._encode_unfused(x, batch, cache, write_cache)
        else:
            qkv = self.qkv.forward_delta(x)              # float32 partial sums [splits, n, q_dim + 2 kv_dim]
            cos = sin = None
            if inv_freq is not None:
                cos, sin = self.position.tables(batch)
            if batch.is_decode and qkv.shape[0] <= 8 and not ops.plain_kernels() and ops.attention_decode_parts_supported(
                    batch.n_seqs, self.heads, self.kv_heads, self.head_dim, self.ctx.dtype):
                # the tensor-core decode attention: the projection's sums, the q/k norm, the rotation,
                # the cache append, the attention and the merge in one or two launches
                need = ops.attention_decode_parts_scratch(batch.n_seqs, self.heads, self.kv_heads, self.head_dim, batch.kv_bound)
                att = ops.attention_decode_parts_fused(
                    qkv, self.heads, self.kv_heads, self.head_dim, q_weight=self.q_norm.weight if self.q_norm else None,
                    k_weight=self.k_norm.weight if self.k_norm else None, eps=self.q_norm.eps if self.q_norm else 0.0,
                    cos=cos, sin=sin, kv=cache.kv, batch=batch, scale=self.scale,
                    scratch=batch.workspace.get("attention_decode_parts", need, torch.float32), write_kv=write_cache,
                    max_kv_len=batch.kv_bound)
                return self.o.forward_delta(att.view(batch.n_tokens, self.q_dim), residual)
            q = ops.qk_norm_rope_append(
                qkv, self.heads, self.kv_heads, self.head_dim,
                q_weight=self.q_norm.weight if self.q_norm else None,
                k_weight=self.k_norm.weight if self.k_norm else None,
                eps=self.q_norm.eps if self.q_norm else 0.0,
                cos=cos, sin=sin, kv=cache.kv, page_table=batch.page_table,
                seq_of_token=batch.seq_of_token, positions=batch.positions, write_kv=write_cache,
                dtype=self.ctx.dtype)
        if batch.is_decode:
            need = ops.attention_decode_scratch_floats(batch.n_seqs, self.heads, self.head_dim, batch.kv_bound,
                                                       self.ctx.dtype)
            att = ops.attention_decode(q, cache.kv, batch, self.scale,
                                       batch.workspace.get("attention_decode", need, torch.float32),
                                       max_kv_len=batch.kv_bound)
        else:
            att = ops.attention_prompt(q, cache.kv, batch, self.scale)
        return self.o.forward_delta(att.view(batch.n_tokens, self.q_dim), residual)


    def _encode_unfused(self, x, batch, cache, write_cache):
        """The way for a position encoding that the fused kernel does not know:
        project, norm q and k per head, let the encoding's own ``apply`` work on
        float32 q [n, heads, d] and k [n, kv_heads, d], then append k and v to the
        cache.  Slower than the fused kernel by a few copies."""
        n = x.shape[0]
        qkv = self.qkv.forward(x, torch.float32)
        q = qkv[:, :self.q_dim].reshape(n * self.heads, self.head_dim)
        k = qkv[:, self.q_dim:self.q_dim + self.kv_dim].reshape(n * self.kv_heads, self.head_dim)
        v = qkv[:, self.q_dim + self.kv_dim:]
        if self.q_norm is not None:
            q = self.q_norm.forward(q, torch.float32)
            k = self.k_norm.forward(k, torch.float32)
        q, k = q.view(n, self.heads, self.head_dim), k.view(n, self.kv_heads, self.head_dim)
        self.position.apply(q, k, batch.positions)
        encoded = torch.cat([q.view(n, -1), k.view(n, -1), v], dim=1).to(self.ctx.dtype)
        return ops.qk_norm_rope_append(
            encoded, self.heads, self.kv_heads, self.head_dim, q_weight=None, k_weight=None, eps=0.0, cos=None,
            sin=None, kv=cache.kv, page_table=batch.page_table, seq_of_token=batch.seq_of_token,
            positions=batch.positions, write_kv=write_cache)


# ---------------------------------------------------------------------------
class GatedMLP(FeedForward):
    """down( act(x gate^T) * (x up^T) ), no biases; gate and up are one matrix."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width, self.intermediate = int(params["width"]), int(params["intermediate"])
        act = params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"unsupported activation {act}")
        names = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        names.update(params.get("names") or {})
        self.names = names
        self.gate_up = Linear(2 * self.intermediate, self.width, ctx, gated=True)
        self.down = Linear(self.width, self.intermediate, ctx)

    def tensor_specs(self):
        nm = self.names
        return [TensorSpec(nm["gate"], (self.intermediate, self.width)),
                TensorSpec(nm["up"], (self.intermediate, self.width)),
                TensorSpec(nm["down"], (self.width, self.intermediate))]

    def load(self, fetch):
        nm = self.names
        self.gate_up.load_rows([fetch(nm["gate"]), fetch(nm["up"])])
        self.down.load_rows([fetch(nm["down"])])

    def tensor(self, name):
        i, nm = self.intermediate, self.names
        if name == nm["gate"]:
            return self.gate_up.rows(0, i)
        if name == nm["up"]:
            return self.gate_up.rows(i, 2 * i)
        return self.down.rows(0, self.width) if name == nm["down"] else None

    def weight_bytes(self):
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    ADDS_TO_RESIDUAL = True

    def forward(self, x, batch, residual=None):
        act = self.gate_up.forward(x, self.ctx.dtype)                   # [n, intermediate]
        return self.down.forward_delta(act, residual)


# ---------------------------------------------------------------------------
class PreNormResidual(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x)).  An addition is either left pending,
    so that the following norm's kernel performs it, or done by the part itself: a
    part whose class says ``ADDS_TO_RESIDUAL`` is handed the residual stream and
    returns None when it has added its result to it (its last kernel did).

    ``layer_scale`` (the local names of two float32 vectors of ``width`` numbers): the
    mixer's and the feed-forward's results are multiplied by them, element by element,
    before the sum; the factor travels with the pending sum, and the parts never add to
    the stream themselves.  ``post_norm`` (the local names of two float32 vectors under ``mixer``
    and ``ffn``, and ``eps``): a sublayer's result is divided by its root mean square and multiplied
    by the vector before the sum, x <- x + rms(sublayer(norm(x))) * w; it travels with the pending
    sum in the same way.  A layer whose feed-forward is of kind ``none`` ends after its
    mixer.  A ``side`` part, if the layer has one, runs last."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx, mixer, mixer_norm, ffn, ffn_norm):
        super().__init__(params, ctx, mixer, mixer_norm, ffn, ffn_norm)
        self.scale_names = dict(params.get("layer_scale") or {})
        post = dict(params.get("post_norm") or {})
        self.post_eps = float(post.pop("eps", 0.0))
        self.post_names = post
        self.width = int(params["width"]) if self.scale_names or self.post_names else 0
        self.scales = {}
        self.posts = {}

    def tensor_specs(self):
        no_ffn = getattr(self.ffn, "IS_NONE", False)
        specs = [TensorSpec(nm, (self.width,), "vector", optional=(k == "ffn" and no_ffn), init="absent" if k == "ffn" and no_ffn else "")
                 for k, nm in self.scale_names.items()]
        return specs + [TensorSpec(nm, (self.width,), "vector", optional=(k == "ffn" and no_ffn),
                                   init="absent" if k == "ffn" and no_ffn else "") for k, nm in self.post_names.items()]

    def load(self, fetch):
        for names, held in ((self.scale_names, self.scales), (self.post_names, self.posts)):
            for k, nm in names.items():
                t = fetch(nm)
                held[k] = None if t is None else self.ctx.hold(t, "vector")

    def tensor(self, name):
        for names, held in ((self.scale_names, self.scales), (self.post_names, self.posts)):
            for k, nm in names.items():
                if nm == name:
                    return held.get(k)
        return None

    def weight_bytes(self):
        return sum(4 * self.width for held in (self.scales, self.posts) for v in held.values() if v is not None)

    def _post(self, which):
        w = self.posts.get(which)
        return None if w is None else (w, self.post_eps)

    def forward(self, h, batch, cache, write_cache):
        dt = self.ctx.dtype
        h.act = None                     # (this block changes the stream without keeping a copy)
        scaled = bool(self.scale_names) or bool(self.post_names)
        if h.pending is not None and (h.scale is not None or h.rms is not None):
            xn = self.mixer_norm.add_forward(h.x, h.pending, dt, scale=h.scale, rms=h.rms)
        elif h.pending is not None:
            xn = self.mixer_norm.add_forward(h.x, h.pending, dt)
        else:
            xn = self.mixer_norm.forward(h.x, dt)
        h.defer(None)
        if getattr(self.mixer, "ADDS_TO_RESIDUAL", False) and not scaled:
            d = self.mixer.forward(xn, batch, cache, write_cache, residual=h.x)
        else:
            d = self.mixer.forward(xn, batch, cache, write_cache)
        if getattr(self.ffn, "IS_NONE", False):
            h.defer(None if d is None else as_splits(d), self.scales.get("mixer"), self._post("mixer"))
        else:
            if d is None:
                xn = self.ffn_norm.forward(h.x, dt)
            elif scaled:
                xn = self.ffn_norm.add_forward(h.x, as_splits(d), dt, scale=self.scales.get("mixer"), rms=self._post("mixer"))
            else:
                xn = self.ffn_norm.add_forward(h.x, as_splits(d), dt)
            if getattr(self.ffn, "ADDS_TO_RESIDUAL", False) and not scaled:
                d = self.ffn.forward(xn, batch, residual=h.x)
            else:
                d = self.ffn.forward(xn, batch)
            h.defer(None if d is None else as_splits(d), self.scales.get("ffn"), self._post("ffn"))
        if self.side is not None:
            self.side.forward(h, batch)
        return h


class PostNormResidual(Block):
    """x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ffn(x)): the sublayers read the
    stream itself and the norm follows the sum.  The stream stays float32; every norm also
    writes it in the compute dtype, which is what the next sublayer's matrix products read.
    A layer whose feed-forward is of kind ``none`` ends after its first half (if its second
    norm has a weight all the same, that norm is applied to alpha x)."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx, mixer, mixer_norm, ffn, ffn_norm):
        super().__init__(params, ctx, mixer, mixer_norm, ffn, ffn_norm)
        self.alpha = float(params.get("alpha", 1.0))

    def forward(self, h, batch, cache, write_cache):
        dt = self.ctx.dtype
        x = h.resolved()
        if h.act is None:
            h.act = ops.to_activation(x, dt)
        d = self.mixer.forward(h.act, batch, cache, write_cache)
        h.act = self.mixer_norm.scaled_add_forward(x, as_splits(d), self.alpha, dt)
        if getattr(self.ffn, "IS_NONE", False):
            if getattr(self.ffn_norm, "present", True):
                h.act = self.ffn_norm.scaled_add_forward(x, None, self.alpha, dt)
            return h
        d = self.ffn.forward(h.act, batch)
        h.act = self.ffn_norm.scaled_add_forward(x, as_splits(d), self.alpha, dt)
        return h


# ---------------------------------------------------------------------------
class TableEmbedding(Embedding):
    """x = table[token] * scale (+ the position's vector).  ``position`` of kind ``sinusoid``: element 2 i of position p's
    vector is sin(p base^(-2i/width)), element 2 i + 1 the cosine of the same angle; the frequencies are evaluated in
    float64 and rounded to float32 once, the angle is their float32 product with the position."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab, self.width = int(params["vocab"]), int(params["width"])
        self.name = str(params.get("tensor", "weight"))
        self.weight: Optional[torch.Tensor] = None
        self.scale = float(params.get("scale", 1.0))
        pos = params.get("position")
        self.freq: Optional[torch.Tensor] = None
        if pos is not None:
            if pos.get("kind") != "sinusoid":
                raise ValueError(f"an embedding's position vectors are of kind 'sinusoid', not {pos.get('kind')!r}")
            base, w = float(pos.get("base", 10000.0)), self.width
            f = [base ** (-2.0 * i / w) for i in range((w + 1) // 2)]
            self.freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(ctx.device)
        self.NEEDS_POSITIONS = self.freq is not None or self.scale != 1.0

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.width))]

    def load(self, fetch):
        self.weight = self.ctx.hold(fetch(self.name), "matrix")

    def tensor(self, name):
        return self.weight if name in (self.name, "weight") else None

    def forward(self, tokens, positions=None):
        if self.NEEDS_POSITIONS:
            return ops.embed_sinusoid(self.weight, tokens, positions, self.freq, self.scale)
        return ops.embed(self.weight, tokens)

    def weight_bytes(self):
        return 0            # a step reads one row per token, not the table


class LinearHead(Head):
    """logits = x W^T in float32.  ``tied``: W is the embedding table.  As in wick
    (model.rs:190) the head is also tied when its own tensor is absent.  ``soft_cap`` c:
    logits <- c tanh(logits / c)."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab, self.width = int(params["vocab"]), int(params["width"])
        self.tied = bool(params.get("tied", False))
        self.name = str(params.get("tensor", "weight"))
        cap = params.get("soft_cap")
        self.soft_cap = float(cap) if cap else None
        self.linear = Linear(self.vocab, self.width, ctx)
        self.is_tied = self.tied
        self.embedding: Optional[Embedding] = None

    PEERS = ("embedding",)

    def attach(self, peers):
        self.embedding = peers.get("embedding")

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.width), optional=True)]

    def load(self, fetch):
        w = None if self.tied else fetch(self.name)
        if w is None:
            table = self.embedding.tensor("weight") if self.embedding is not None else None
            if table is None:
                raise ValueError("a tied head needs the embedding table (loaded before it)")
            self.linear.use(table)
            self.is_tied = True
        else:
            self.linear.load_rows([w])
            self.is_tied = False

    def tensor(self, name):
        return self.linear.rows(0, self.vocab) if name == self.name and not self.is_tied else None

    def forward(self, x):
        z = self.linear.forward(x, torch.float32)
        return ops.soft_cap_(z, self.soft_cap) if self.soft_cap is not None else z

    def weight_bytes(self):
        return self.linear.weight_bytes()


register_part("norm", "rms", RMSNorm)
register_part("norm", "tanh", TanhNorm)
register_part("position", "rotary_half_split", RotaryHalfSplit)
register_part("position", "none", NoPosition)
register_part("mixer", "gqa_attention", GQAttention)
register_part("ffn", "gated_mlp", GatedMLP)
register_part("block", "prenorm_residual", PreNormResidual)
register_part("block", "postnorm_residual", PostNormResidual)
register_part("embedding", "table", TableEmbedding)
register_part("head", "linear", LinearHead)
