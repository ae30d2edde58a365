"""What changes the stream from something else than the stream alone.

=============  ======================  ==========================================
category       kind                    params
=============  ======================  ==========================================
side           ``gated_token_rows``    width, dim, offset, eps, table (the place
                                       of the model's shared table part), names
                                       (gate, proj, norm -> local names)
side           ``mix_with_embedding``  width, tensor (local name of the matrix)
side           ``pass_offset``         width, passes, add_embedding, tensor (local
                                       name of the [passes, width] vectors)
=============  ======================  ==========================================

``pass_offset`` (a shared part that a schedule entry names in ``before``, with the number t of the pass as its index):
x <- x + x0 + s_t, where x0, the embedding's output for the same token, is added before every pass but the first (with
``add_embedding``) and s_t is row t of the part's tensor.  float32, one kernel.

``mix_with_embedding`` (a shared part that a schedule entry names in ``before``): with x the stream
and x0 the embedding's output for the same token, x <- W [x; x0], W of shape [width, 2 width] with the
stream's columns first.  The stream is replaced, not added to.

With x the stream after the layer's feed-forward and e the ``dim`` numbers from ``offset``
on of the token's row in the shared table:  g = gelu(Wgate x) * e  (gelu in its tanh
form), y = Wproj g, and x <- x + y / sqrt(mean(y^2) + eps) * w.  The gate reads the stream
itself, so the layer's pending sum is resolved first; the part's own sum stays pending,
with the norm, for whoever reads the stream next.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import SideInput, TensorSpec, register_part
from .linear import Linear


class GatedTokenRows(SideInput):
    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width, self.dim, self.offset = int(params["width"]), int(params["dim"]), int(params["offset"])
        self.eps = float(params["eps"])
        self.table_place = str(params["table"])
        self.PEERS = (self.table_place,)
        names = dict(gate="gate.weight", proj="proj.weight", norm="norm.weight")
        names.update(params.get("names") or {})
        self.names = names
        self.gate = Linear(self.dim, self.width, ctx)
        self.proj = Linear(self.width, self.dim, ctx)
        self.norm_weight = None
        self.table = None

    def attach(self, peers):
        self.table = peers[self.table_place]

    def tensor_specs(self):
        nm = self.names
        return [TensorSpec(nm["gate"], (self.dim, self.width)), TensorSpec(nm["proj"], (self.width, self.dim)),
                TensorSpec(nm["norm"], (self.width,), "vector")]

    def load(self, fetch):
        nm = self.names
        self.gate.load_rows([fetch(nm["gate"])])
        self.proj.load_rows([fetch(nm["proj"])])
        self.norm_weight = self.ctx.hold(fetch(nm["norm"]), "vector")
        rows = self.table.tensor("weight")
        if rows is None or rows.shape[1] < self.offset + self.dim:
            raise ValueError(f"the shared table has no columns {self.offset} .. {self.offset + self.dim}")

    def tensor(self, name):
        nm = self.names
        if name == nm["gate"]:
            return self.gate.rows(0, self.dim)
        if name == nm["proj"]:
            return self.proj.rows(0, self.width)
        return self.norm_weight if name == nm["norm"] else None

    def weight_bytes(self):
        return self.gate.weight_bytes() + self.proj.weight_bytes() + 4 * self.width

    def forward(self, h, batch, index=0):
        dt = self.ctx.dtype
        h.resolved(dt)                                               # x with the layer's sums, and its copy in h.act
        z = self.gate.forward(h.act, torch.float32)                  # [n, dim]
        g = ops.gelu_gate_rows(z, self.table.tensor("weight"), batch.tokens, self.offset, dt)
        h.defer(self.proj.forward_delta(g), rms=(self.norm_weight, self.eps))


class MixWithEmbedding(SideInput):
    PROMPT_CAPTURABLE = True
    NEEDS_EMBEDDING_OUTPUT = True          # the model leaves the embedding's output in the step's memo

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.name = str(params.get("tensor", "weight"))
        self.mix = Linear(self.width, 2 * self.width, ctx)

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width, 2 * self.width), init="mix_pair")]

    def load(self, fetch):
        self.mix.load_rows([fetch(self.name)])

    def tensor(self, name):
        return self.mix.rows(0, self.width) if name == self.name else None

    def weight_bytes(self):
        return self.mix.weight_bytes()

    def forward(self, h, batch, index=0):
        x0 = batch.memo.get("embedding_output")
        if x0 is None:
            raise RuntimeError("the step's memo holds no embedding output")
        x = h.resolved()
        both = ops.concat_activation(x, x0, self.ctx.dtype)           # [n, 2 width]: the stream, then the embedding's output
        h.x = self.mix.forward(both, torch.float32)
        h.act = None
        h.defer(None)


class PassOffset(SideInput):
    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width, self.passes = int(params["width"]), int(params["passes"])
        self.add_embedding = bool(params.get("add_embedding", True))
        self.NEEDS_EMBEDDING_OUTPUT = self.add_embedding   # the model leaves the embedding's output in the step's memo
        self.name = str(params.get("tensor", "weight"))
        self.steps = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.passes, self.width), "vector", init="around_zero")]

    def load(self, fetch):
        self.steps = self.ctx.hold(fetch(self.name), "vector")

    def tensor(self, name):
        return self.steps if name == self.name else None

    def weight_bytes(self):
        return 4 * self.width

    def forward(self, h, batch, index=0):
        if not 0 <= index < self.passes:
            raise ValueError(f"pass {index} of {self.passes}")
        x0 = None
        if self.add_embedding and index > 0:
            x0 = batch.memo.get("embedding_output")
            if x0 is None:
                raise RuntimeError("the step's memo holds no embedding output")
        ops.stream_offset_(h.resolved(), x0, self.steps[index])
        h.act = None


register_part("side", "pass_offset", PassOffset)
register_part("side", "gated_token_rows", GatedTokenRows)
register_part("side", "mix_with_embedding", MixWithEmbedding)
