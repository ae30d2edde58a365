"""Gated linear attention as a mixer.

=============  ===========================  ==========================================
category       kind                         params
=============  ===========================  ==========================================
mixer          ``gated_linear_attention``   width, heads, head_dim (key channels of a
                                            head), v_dim, tau, eps, rank (of the decay's
                                            two-step projection; None: whatever the
                                            checkpoint's tensors have), q_scale (default
                                            head_dim^(-1/2)), names (q, k, v, gate, o,
                                            norm, decay_in, decay_out, decay_bias ->
                                            local names)
=============  ===========================  ==========================================

With h the mixer's input, H heads of dk key channels and dv value numbers:

* q = Wq h * q_scale, k = Wk h (H x dk each), v = Wv h (H x dv), g = Wg h (H x dv), low = W1 h (r numbers): one matrix
  product;
* z = W2 low + b (H x dk numbers); the decay of a key channel is a = sigmoid(z)^(1 / tau), evaluated as
  exp(-softplus(-z) / tau);
* per head S <- diag(a) S + k v^T (dk x dv; the decay acts on the rows that belong to key channels), o = S^T q;
* every head's o is divided by its root mean square over dv (eps inside the root) and multiplied by a weight of dv numbers
  that the heads share; the heads side by side are multiplied by silu(g) and go through Wo.

The state is one float32 record per sequence (kind ``state`` of the cache: zero when a sequence starts), read and brought
up to date by every step whatever its shape.  Everything between the two matrix products is float32, W2's product
included (W2 is held in float32; its rank is small).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, Mixer, TensorSpec, register_part
from .linear import Linear


class GatedLinearAttention(Mixer):
    PROMPT_CAPTURABLE = True
    RANDOM_RANK = 16                      # the rank random weights are drawn with where the parameters leave it open

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.width, self.heads = int(p["width"]), int(p["heads"])
        self.key_dim, self.v_dim = int(p["head_dim"]), int(p["v_dim"])
        self.tau, self.eps = float(p["tau"]), float(p["eps"])
        if self.heads <= 0 or self.key_dim <= 0 or self.v_dim <= 0 or self.tau <= 0:
            raise ValueError("heads, head_dim, v_dim and tau must be positive")
        self.rank = int(p["rank"]) if p.get("rank") else None
        self.q_scale = float(p["q_scale"]) if p.get("q_scale") is not None else self.key_dim ** -0.5
        self.hk, self.hv = self.heads * self.key_dim, self.heads * self.v_dim
        names = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", gate="g_proj.weight", o="o_proj.weight",
                     norm="norm.weight", decay_in="decay_in.weight", decay_out="decay_out.weight", decay_bias="decay_out.bias")
        names.update(p.get("names") or {})
        self.names = names
        self.input = None                 # Linear over [q | k | v | g | low]; made when the rank is known
        self.o = Linear(self.width, self.hv, ctx)
        self.w2 = self.b2 = self.norm_w = None

    def tensor_specs(self):
        nm, r = self.names, (self.rank if self.rank is not None else -1)
        return [TensorSpec(nm["q"], (self.hk, self.width)), TensorSpec(nm["k"], (self.hk, self.width)),
                TensorSpec(nm["v"], (self.hv, self.width)), TensorSpec(nm["gate"], (self.hv, self.width)),
                TensorSpec(nm["o"], (self.width, self.hv)), TensorSpec(nm["norm"], (self.v_dim,), "vector"),
                TensorSpec(nm["decay_in"], (r, self.width), init_arg=self.RANDOM_RANK),
                TensorSpec(nm["decay_out"], (self.hk, r), "vector", init="decay_out", init_arg=self.RANDOM_RANK),
                TensorSpec(nm["decay_bias"], (self.hk,), "vector", init="decay_bias")]

    def load(self, fetch):
        nm, hold = self.names, self.ctx.hold
        low, w2 = fetch(nm["decay_in"]), fetch(nm["decay_out"])
        rank = int(low.shape[0])
        if rank <= 0 or tuple(w2.shape) != (self.hk, rank) or (self.rank is not None and rank != self.rank):
            raise ValueError(f"the decay's projections have shapes {tuple(low.shape)} and {tuple(w2.shape)}; "
                             f"[r, {self.width}] and [{self.hk}, r] with one r are expected")
        self.loaded_rank = rank
        self.input = Linear(2 * self.hk + 2 * self.hv + rank, self.width, self.ctx)
        self.input.load_rows([fetch(nm["q"]), fetch(nm["k"]), fetch(nm["v"]), fetch(nm["gate"]), low])
        self.o.load_rows([fetch(nm["o"])])
        # (a matrix of the checkpoint's 16-bit numbers is the same numbers in float32)
        self.w2, self.b2 = hold(w2, "vector"), hold(fetch(nm["decay_bias"]), "vector")
        self.norm_w = hold(fetch(nm["norm"]), "vector")

    def tensor(self, name):
        nm, hk, hv = self.names, self.hk, self.hv
        spans = {nm["q"]: (0, hk), nm["k"]: (hk, 2 * hk), nm["v"]: (2 * hk, 2 * hk + hv), nm["gate"]: (2 * hk + hv, 2 * hk + 2 * hv)}
        if self.input is not None and name in spans:
            return self.input.rows(*spans[name])
        if self.input is not None and name == nm["decay_in"]:
            return self.input.rows(2 * hk + 2 * hv, 2 * hk + 2 * hv + self.loaded_rank)
        if name == nm["o"]:
            return self.o.rows(0, self.width)
        return {nm["decay_out"]: self.w2, nm["decay_bias"]: self.b2, nm["norm"]: self.norm_w}.get(name)

    def record_floats(self) -> int:
        return self.hv * self.key_dim

    def cache_need(self):
        return CacheNeed("state", shape=(self.record_floats(),), dtype=torch.float32)

    def weight_bytes(self):
        n = self.o.weight_bytes() + (self.input.weight_bytes() if self.input is not None else 0)
        return n + 4 * (self.hk * (1 + (self.loaded_rank if self.input is not None else 0)) + self.v_dim)

    def forward(self, x, batch, cache, write_cache):
        if not write_cache:
            raise RuntimeError("a linear-attention mixer keeps its own record; it cannot read another entry's")
        parts = self.input.forward_delta(x)                         # float32 [splits, n, cols]
        y = ops.gla_mix(parts, heads=self.heads, key_dim=self.key_dim, v_dim=self.v_dim, w2=self.w2, b2=self.b2, q_scale=self.q_scale,
                        tau=self.tau, records=cache.state, batch=batch)
        g = ops.gla_norm_gate(y, parts, 2 * self.hk + self.hv, self.heads, self.v_dim, self.norm_w, self.eps, self.ctx.dtype)
        return self.o.forward_delta(g)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
