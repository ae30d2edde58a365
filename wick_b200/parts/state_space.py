"""A selective state-space recurrence as a mixer.

=============  =========================  ==========================================
category       kind                       params
=============  =========================  ==========================================
mixer          ``selective_state_space``  width, heads, head_dim, state, groups,
                                          taps, norm_groups, eps, names (input,
                                          conv, conv_bias, dt_bias, a_log, d, norm,
                                          o -> local names)
=============  =========================  ==========================================

With h the mixer's input, Hs heads of P numbers (inner = Hs P), state size N, G groups of heads
that share B and C, K taps:

* W_in h = [z: inner | x: inner | B: G N | C: G N | dt: Hs], one matrix product;
* u = [x | B | C] passes a causal convolution per channel (weights [channels, K], the last
  column the token's own input, zeros before position 0, a bias) and silu;
* dt <- softplus(dt + dt_bias); per head, with a = exp(-exp(A_log) dt):
  S <- a S + dt B x^T (N x P), y = S^T C + D x;
* g = y * silu(z); each of ``norm_groups`` equal parts of g is divided by its own root mean
  square (eps inside the root) and multiplied by a weight; W_o on the result.

The state and the convolution's last K - 1 inputs are one float32 record per sequence (kind
``state`` of the cache: zero when a sequence starts), read and brought up to date by every step
whatever its shape.  Everything between the two matrix products is float32.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, Mixer, TensorSpec, register_part
from .linear import Linear


class SelectiveStateSpace(Mixer):
    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.width, self.heads, self.head_dim = int(p["width"]), int(p["heads"]), int(p["head_dim"])
        self.state, self.groups, self.taps = int(p["state"]), int(p["groups"]), int(p["taps"])
        self.norm_groups, self.eps = int(p.get("norm_groups", 1)), float(p["eps"])
        if self.heads <= 0 or self.groups <= 0 or self.heads % self.groups != 0:
            raise ValueError("heads must be a positive multiple of groups")
        self.inner = self.heads * self.head_dim
        if self.norm_groups <= 0 or self.inner % self.norm_groups != 0:
            raise ValueError(f"{self.inner} numbers cannot be normed in {self.norm_groups} equal parts")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"the convolution kernel takes 1 to 16 taps, not {self.taps}")
        self.channels = self.inner + 2 * self.groups * self.state
        self.cols = 2 * self.inner + 2 * self.groups * self.state + self.heads
        names = dict(input="in_proj.weight", conv="conv.weight", conv_bias="conv.bias", dt_bias="dt_bias", a_log="A_log",
                     d="D", norm="norm.weight", o="out_proj.weight")
        names.update(p.get("names") or {})
        self.names = names
        self.input = Linear(self.cols, self.width, ctx)
        self.o = Linear(self.width, self.inner, ctx)
        self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d = self.norm_w = None

    def tensor_specs(self):
        nm = self.names
        return [TensorSpec(nm["input"], (self.cols, self.width)),
                TensorSpec(nm["conv"], (self.channels, self.taps), "vector", init="conv_taps"),
                TensorSpec(nm["conv_bias"], (self.channels,), "vector", init="around_zero"),
                TensorSpec(nm["dt_bias"], (self.heads,), "vector", init="around_zero"),
                TensorSpec(nm["a_log"], (self.heads,), "vector", init="around_zero"),
                TensorSpec(nm["d"], (self.heads,), "vector"),
                TensorSpec(nm["norm"], (self.inner,), "vector"),
                TensorSpec(nm["o"], (self.width, self.inner))]

    def load(self, fetch):
        nm, hold = self.names, self.ctx.hold
        self.input.load_rows([fetch(nm["input"])])
        self.o.load_rows([fetch(nm["o"])])
        self.conv_w, self.conv_b = hold(fetch(nm["conv"]), "vector"), hold(fetch(nm["conv_bias"]), "vector")
        self.dt_bias, self.a_log, self.d = (hold(fetch(nm[k]), "vector") for k in ("dt_bias", "a_log", "d"))
        self.norm_w = hold(fetch(nm["norm"]), "vector")

    def tensor(self, name):
        nm = self.names
        if name == nm["input"]:
            return self.input.rows(0, self.cols)
        if name == nm["o"]:
            return self.o.rows(0, self.width)
        held = {nm["conv"]: self.conv_w, nm["conv_bias"]: self.conv_b, nm["dt_bias"]: self.dt_bias, nm["a_log"]: self.a_log,
                nm["d"]: self.d, nm["norm"]: self.norm_w}
        return held.get(name)

    def record_floats(self) -> int:
        return ops.ssm_record_floats(self.heads, self.head_dim, self.state, self.groups, self.taps)

    def cache_need(self):
        return CacheNeed("state", shape=(self.record_floats(),), dtype=torch.float32)

    def weight_bytes(self):
        return self.input.weight_bytes() + self.o.weight_bytes() + 4 * (self.channels * (self.taps + 1) + 3 * self.heads + self.inner)

    def forward(self, x, batch, cache, write_cache):
        if not write_cache:
            raise RuntimeError("a state-space mixer keeps its own record; it cannot read another entry's")
        parts = self.input.forward_delta(x)                         # float32 [splits, n, cols]
        y = ops.ssm_mix(parts, heads=self.heads, head_dim=self.head_dim, state=self.state, groups=self.groups, taps=self.taps,
                        conv_w=self.conv_w, conv_b=self.conv_b, dt_bias=self.dt_bias, a_log=self.a_log, d_skip=self.d,
                        records=cache.state, batch=batch)
        g = ops.ssm_gate_norm(y, parts, self.norm_w, self.eps, self.norm_groups, self.ctx.dtype)
        return self.o.forward_delta(g)


register_part("mixer", "selective_state_space", SelectiveStateSpace)
