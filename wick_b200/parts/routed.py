"""A mixture of gated experts chosen by a router.

=============  ======================  ==========================================
category       kind                    params
=============  ======================  ==========================================
ffn            ``routed_moe``          width, experts, identity (router outputs
                                       beyond the experts that stand for experts
                                       returning their input; default 0), top,
                                       intermediate, scores (``softmax``),
                                       correction (a vector added to the scores
                                       for the choice only), renormalize,
                                       names (expert: a pattern with ``{i}``,
                                       gate, up, down, router, correction)
=============  ======================  ==========================================

For a token with input h: z = W_router h over experts + identity outputs, in float32 (from the
product's float32 partial sums); s = softmax(z); the ``top`` outputs with the largest
s + correction are chosen (the lowest index among equals); the result is the sum over the chosen
outputs of s_i r_i (the chosen scores divided by their sum first, with ``renormalize``), where
r_i = down_i(silu(gate_i h) * (up_i h)) for an expert with matrices and r_i = h for one of the last
``identity`` outputs.

The experts' products reuse the kernels of the experts chosen by a table: the router's choice,
[tokens, top], is such a table with the token's number as its row.  From ``SORTED_FROM`` tokens on
(bfloat16) the (token, choice) pairs are sorted by expert and go through one tensor-core product over
tiles of 256 rows; the host does not know how many rows each expert gets, so the product runs over
the most tiles there can be (those beyond the last expert's return at once).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_part
from .linear import Linear


class RoutedMoE(FeedForward):
    PROMPT_CAPTURABLE = True
    SORTED_FROM = 16
    ROW_TILE = 256

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.width, self.experts, self.identity = int(p["width"]), int(p["experts"]), int(p.get("identity", 0))
        self.top, self.intermediate = int(p["top"]), int(p["intermediate"])
        self.outputs = self.experts + self.identity
        if self.experts <= 0 or self.identity < 0 or not 0 < self.top <= self.outputs:
            raise ValueError(f"{self.top} of {self.experts} + {self.identity} router outputs per token")
        if str(p.get("scores", "softmax")) != "softmax":
            raise ValueError(f"router scores {p.get('scores')!r} are not built (softmax)")
        self.has_correction = bool(p.get("correction", False))
        self.renormalize = bool(p.get("renormalize", False))
        names = dict(expert="experts.{i}.", gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight",
                     router="router.weight", correction="router.correction")
        names.update(p.get("names") or {})
        self.names = names
        self.router = Linear(self.outputs, self.width, ctx)
        self.correction: Optional[torch.Tensor] = None
        self.gate_up: Optional[torch.Tensor] = None      # [experts, 2, intermediate, width]
        self.down: Optional[torch.Tensor] = None         # [experts, width, intermediate]
        self.up_tiles: Optional[torch.Tensor] = None     # the same matrices as tiles of the tensor-core product (bfloat16)
        self.down_tiles: Optional[torch.Tensor] = None

    def _expert(self, i: int, which: str) -> str:
        return self.names["expert"].format(i=i) + self.names[which]

    def tensor_specs(self):
        f, w = self.intermediate, self.width
        specs = []
        for i in range(self.experts):
            specs += [TensorSpec(self._expert(i, "gate"), (f, w)), TensorSpec(self._expert(i, "up"), (f, w)),
                      TensorSpec(self._expert(i, "down"), (w, f))]
        specs.append(TensorSpec(self.names["router"], (self.outputs, w), init="router"))
        if self.has_correction:
            specs.append(TensorSpec(self.names["correction"], (self.outputs,), "vector", init="around_zero"))
        return specs

    def load(self, fetch):
        hold = self.ctx.hold
        self.gate_up = torch.stack([torch.stack([hold(fetch(self._expert(i, "gate")), "matrix"),
                                                 hold(fetch(self._expert(i, "up")), "matrix")]) for i in range(self.experts)])
        self.down = torch.stack([hold(fetch(self._expert(i, "down")), "matrix") for i in range(self.experts)])
        self.router.load_rows([fetch(self.names["router"])])
        self.correction = hold(fetch(self.names["correction"]), "vector") if self.has_correction else None
        self.up_tiles = self.down_tiles = None
        if (self.ctx.dtype == torch.bfloat16 and self.gate_up.is_cuda and not ops.plain_kernels()
                and self.width % 8 == 0 and self.intermediate % 8 == 0):
            from ..ops import gemm_tc
            self.up_tiles = torch.cat([gemm_tc.pack(self.gate_up[i].reshape(2 * self.intermediate, self.width), gated=True)
                                       for i in range(self.experts)], 0)
            self.down_tiles = torch.cat([gemm_tc.pack(self.down[i]) for i in range(self.experts)], 0)

    def tensor(self, name):
        for i in range(self.experts):
            pre = self.names["expert"].format(i=i)
            if name.startswith(pre):
                which = name[len(pre):]
                if which == self.names["gate"]:
                    return self.gate_up[i, 0]
                if which == self.names["up"]:
                    return self.gate_up[i, 1]
                if which == self.names["down"]:
                    return self.down[i]
        if name == self.names["router"]:
            return self.router.rows(0, self.outputs)
        if self.has_correction and name == self.names["correction"]:
            return self.correction
        return None

    def weight_bytes(self):
        """What a step of one token reads: the router and (at most) ``top`` experts."""
        el = 2 if self.ctx.dtype == torch.bfloat16 else 4
        return self.router.weight_bytes() + min(self.top, self.experts) * 3 * self.intermediate * self.width * el

    def forward(self, x, batch):
        n = x.shape[0]
        logits = self.router.forward_delta(x)                        # float32 [splits, n, outputs]
        choice, weight, ident = ops.moe_router(logits, self.correction, self.top, renormalize=self.renormalize)
        own = x if self.identity else None
        if self.up_tiles is not None and n >= self.SORTED_FROM:
            return self._forward_sorted(x, choice, weight, ident, own)
        hidden = ops.moe_table_up(x, ident, choice, self.gate_up)   # [n, top, ff]; pairs of outputs without matrices are passed over
        y = ops.moe_expert_down(hidden, ident, choice, self.down)
        return ops.moe_combine_weighted(y, None, choice, weight, own, self.experts).unsqueeze(0)

    def _forward_sorted(self, x, choice, weight, ident, own):
        from ..ops import gemm_tc
        n, dt, pad = x.shape[0], self.ctx.dtype, self.ROW_TILE
        counts, row_of, tiles = ops.moe_route(ident, choice, self.experts, pad=pad)
        rows = min(self.experts, n * self.top) * pad + (n * self.top) // pad * pad
        f, w = self.intermediate, self.width
        f_pad, w_pad = (f + 127) // 128 * 128, (w + 127) // 128 * 128
        xs = ops.moe_gather(x, row_of, rows)
        hidden = torch.empty((rows, f), dtype=dt, device=x.device)
        y = torch.empty((rows, w), dtype=torch.float32, device=x.device)
        gemm_tc.gemm_tc_pair(xs, self.up_tiles, f, out=hidden, ldo=f, gated=True, pair_offset=f_pad, b_packed=True,
                             groups=tiles, group_rows=2 * f_pad)
        gemm_tc.gemm_tc_pair(hidden, self.down_tiles, w, out=y, ldo=w, b_packed=True, groups=tiles, group_rows=w_pad)
        return ops.moe_combine_weighted(y, row_of, choice, weight, own, self.experts).unsqueeze(0)


register_part("ffn", "routed_moe", RoutedMoE)
