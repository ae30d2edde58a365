"""A mixture of experts chosen by a router.

=============  ======================  ==========================================
category       kind                    params
=============  ======================  ==========================================
ffn            ``routed_moe``          width, experts, identity (router outputs
                                       beyond the experts that stand for experts
                                       returning their input; default 0), top,
                                       intermediate, scores (``softmax`` or
                                       ``sigmoid``), correction (a vector added to
                                       the scores for the choice only),
                                       renormalize, norm_eps (added to the chosen
                                       scores' sum), route_scale (a factor of the
                                       weights), groups (None or {"count", "keep"}),
                                       expert (``gated``: down(silu(gate h) * up h);
                                       ``relu2``: down(max(up h, 0)^2)), shared
                                       (PartSpec of a feed-forward every token
                                       uses, or None), shared_gate (True: its
                                       result times the sigmoid of a number per
                                       token), names (expert: a pattern with
                                       ``{i}``, gate, up, down, router, correction,
                                       shared: a prefix, shared_gate)
=============  ======================  ==========================================

For a token with input h: z = W_router h over experts + identity outputs, in float32 (from the
product's float32 partial sums); s = softmax(z), or sigmoid(z) of each output; the ``top`` outputs with
the largest s + correction are chosen (the lowest index among equals); the result is the sum over the chosen
outputs of s_i r_i (the chosen scores divided by their sum + ``norm_eps`` first, with ``renormalize``; times
``route_scale``), where r_i = down_i(silu(gate_i h) * (up_i h)) (or down_i(max(up_i h, 0)^2) for experts of one
matrix) for an expert with matrices and r_i = h for one of the last ``identity`` outputs.  ``groups``: the
experts form ``count`` equal groups of neighbours; a group's score is the sum of its two largest s + correction,
and only experts of the ``keep`` best groups can be chosen.  ``shared``: a feed-forward that runs for every
token; its result is added, with ``shared_gate`` times sigmoid(w_sg . h), one number per token (float32).

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
from .base import FeedForward, TensorSpec, as_splits, build_part, register_part
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
        self.scores = str(p.get("scores", "softmax"))
        if self.scores not in ops.ROUTER_SCORES:
            raise ValueError(f"router scores {p.get('scores')!r} are not built ({', '.join(ops.ROUTER_SCORES)})")
        self.has_correction = bool(p.get("correction", False))
        self.renormalize = bool(p.get("renormalize", False))
        self.norm_eps, self.route_scale = float(p.get("norm_eps", 0.0)), float(p.get("route_scale", 1.0))
        groups = p.get("groups")
        self.group_count, self.group_keep = (int(groups["count"]), int(groups["keep"])) if groups else (0, 0)
        if self.group_count and (self.identity or self.experts % self.group_count or not 0 < self.group_keep <= self.group_count
                                 or self.group_keep * (self.experts // self.group_count) < self.top):
            raise ValueError(f"{self.experts} experts do not form {self.group_count} equal groups of which {self.group_keep} hold {self.top} choices")
        self.expert_kind = str(p.get("expert", "gated"))
        if self.expert_kind not in ("gated", "relu2"):
            raise ValueError(f"experts are 'gated' or 'relu2', not {self.expert_kind!r}")
        self.gated = self.expert_kind == "gated"
        names = dict(expert="experts.{i}.", gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight",
                     router="router.weight", correction="router.correction", shared="shared.", shared_gate="shared_gate.weight")
        names.update(p.get("names") or {})
        self.names = names
        shared = p.get("shared")
        self.shared = build_part("ffn", shared, ctx) if shared is not None else None
        self.has_shared_gate = self.shared is not None and bool(p.get("shared_gate", False))
        self.PROMPT_CAPTURABLE = self.shared is None or bool(self.shared.PROMPT_CAPTURABLE)
        # (the shared expert's gate is one more row of the router's matrix: one product gives the logits and the gate's number)
        self.router = Linear(self.outputs + (1 if self.has_shared_gate else 0), self.width, ctx)
        self.correction: Optional[torch.Tensor] = None
        self.gate_up: Optional[torch.Tensor] = None      # [experts, 2, intermediate, width] (gate, up); [experts, 1, ...] for experts of one matrix
        self.down: Optional[torch.Tensor] = None         # [experts, width, intermediate]
        self.up_tiles: Optional[torch.Tensor] = None     # the same matrices as tiles of the tensor-core product (bfloat16)
        self.down_tiles: Optional[torch.Tensor] = None

    def _expert(self, i: int, which: str) -> str:
        return self.names["expert"].format(i=i) + self.names[which]

    def tensor_specs(self):
        f, w = self.intermediate, self.width
        specs = []
        for i in range(self.experts):
            if self.gated:
                specs.append(TensorSpec(self._expert(i, "gate"), (f, w)))
            specs += [TensorSpec(self._expert(i, "up"), (f, w)), TensorSpec(self._expert(i, "down"), (w, f))]
        specs.append(TensorSpec(self.names["router"], (self.outputs, w), init="router"))
        if self.has_correction:
            specs.append(TensorSpec(self.names["correction"], (self.outputs,), "vector", init="around_zero"))
        if self.shared is not None:
            specs += [TensorSpec(self.names["shared"] + s.name, s.shape, s.role, s.optional, s.init, s.init_arg)
                      for s in self.shared.tensor_specs()]
        if self.has_shared_gate:
            specs.append(TensorSpec(self.names["shared_gate"], (1, w), init="router"))
        return specs

    def load(self, fetch):
        hold = self.ctx.hold
        which = ("gate", "up") if self.gated else ("up",)
        self.gate_up = torch.stack([torch.stack([hold(fetch(self._expert(i, k)), "matrix") for k in which]) for i in range(self.experts)])
        self.down = torch.stack([hold(fetch(self._expert(i, "down")), "matrix") for i in range(self.experts)])
        self.router.load_rows([fetch(self.names["router"])] + ([fetch(self.names["shared_gate"])] if self.has_shared_gate else []))
        self.correction = hold(fetch(self.names["correction"]), "vector") if self.has_correction else None
        if self.shared is not None:
            self.shared.load(lambda n: fetch(self.names["shared"] + n))
        self.up_tiles = self.down_tiles = None
        if (self.ctx.dtype == torch.bfloat16 and self.gate_up.is_cuda and not ops.plain_kernels()
                and self.width % 8 == 0 and self.intermediate % 8 == 0):
            from ..ops import gemm_tc
            self.up_tiles = torch.cat([gemm_tc.pack(self.gate_up[i].reshape(len(which) * self.intermediate, self.width), gated=self.gated)
                                       for i in range(self.experts)], 0)
            self.down_tiles = torch.cat([gemm_tc.pack(self.down[i]) for i in range(self.experts)], 0)

    def tensor(self, name):
        for i in range(self.experts):
            pre = self.names["expert"].format(i=i)
            if name.startswith(pre):
                which = name[len(pre):]
                if self.gated and which == self.names["gate"]:
                    return self.gate_up[i, 0]
                if which == self.names["up"]:
                    return self.gate_up[i, 1 if self.gated else 0]
                if which == self.names["down"]:
                    return self.down[i]
        if name == self.names["router"]:
            return self.router.rows(0, self.outputs)
        if self.has_correction and name == self.names["correction"]:
            return self.correction
        if self.has_shared_gate and name == self.names["shared_gate"]:
            return self.router.rows(self.outputs, self.outputs + 1)
        if self.shared is not None and name.startswith(self.names["shared"]):
            return self.shared.tensor(name[len(self.names["shared"]):])
        return None

    def weight_bytes(self):
        """What a step of one token reads: the router and (at most) ``top`` experts."""
        el = 2 if self.ctx.dtype == torch.bfloat16 else 4
        n = self.router.weight_bytes() + min(self.top, self.experts) * (3 if self.gated else 2) * self.intermediate * self.width * el
        if self.shared is not None:
            n += self.shared.weight_bytes()
        return n

    def forward(self, x, batch):
        n = x.shape[0]
        logits = self.router.forward_delta(x)                        # float32 [splits, n, outputs (+ 1: the shared expert's gate)]
        choice, weight, ident = ops.moe_router(logits, self.correction, self.top, renormalize=self.renormalize, scores=self.scores,
                                               groups=self.group_count, keep=self.group_keep, scale=self.route_scale,
                                               norm_eps=self.norm_eps, outputs=self.outputs)
        own = x if self.identity else None
        base = base_gate = None
        if self.shared is not None:
            base = as_splits(self.shared.forward(x, batch))
            if self.has_shared_gate:
                base_gate = logits                                  # (its last column)
        if self.up_tiles is not None and n >= self.SORTED_FROM:
            return self._forward_sorted(x, choice, weight, ident, own, base, base_gate)
        hidden = ops.moe_table_up(x, ident, choice, self.gate_up)   # [n, top, ff]; pairs of outputs without matrices are passed over
        y = ops.moe_expert_down(hidden, ident, choice, self.down)
        return ops.moe_combine_weighted(y, None, choice, weight, own, self.experts, base, base_gate, self.outputs).unsqueeze(0)

    def _forward_sorted(self, x, choice, weight, ident, own, base=None, base_gate=None):
        from ..ops import gemm_tc
        n, dt, pad = x.shape[0], self.ctx.dtype, self.ROW_TILE
        counts, row_of, tiles = ops.moe_route(ident, choice, self.experts, pad=pad)
        rows = min(self.experts, n * self.top) * pad + (n * self.top) // pad * pad
        f, w = self.intermediate, self.width
        f_pad, w_pad = (f + 127) // 128 * 128, (w + 127) // 128 * 128
        xs = ops.moe_gather(x, row_of, rows)
        hidden = torch.empty((rows, f), dtype=dt, device=x.device)
        y = torch.empty((rows, w), dtype=torch.float32, device=x.device)
        if self.gated:
            gemm_tc.gemm_tc_pair(xs, self.up_tiles, f, out=hidden, ldo=f, gated=True, pair_offset=f_pad, b_packed=True,
                                 groups=tiles, group_rows=2 * f_pad)
        else:
            gemm_tc.gemm_tc_pair(xs, self.up_tiles, f, out=hidden, ldo=f, b_packed=True, groups=tiles, group_rows=f_pad)
            ops.relu_squared_(hidden)
        gemm_tc.gemm_tc_pair(hidden, self.down_tiles, w, out=y, ldo=w, b_packed=True, groups=tiles, group_rows=w_pad)
        return ops.moe_combine_weighted(y, row_of, choice, weight, own, self.experts, base, base_gate, self.outputs).unsqueeze(0)


register_part("ffn", "routed_moe", RoutedMoE)
