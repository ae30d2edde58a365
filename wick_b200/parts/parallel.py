"""Mixers side by side.

=============  ======================  ==========================================
category       kind                    params
=============  ======================  ==========================================
mixer          ``parallel``            width, branches: a sequence of {"part":
                                       PartSpec of a mixer, "scale": a number,
                                       "prefix": what its tensors' local names
                                       begin with}
=============  ======================  ==========================================

Every branch reads the same input; the result is the sum of the branches' results, each times its
``scale``: sum_i scale_i * branch_i(h).  Each branch keeps what it asks of the cache for itself (the
need of kind ``several``: a view per branch).  The branches' partial sums are added up in index order
and the terms in the order of the branches, by one kernel.
"""
from __future__ import annotations

from .. import ops
from .base import CacheNeed, Mixer, TensorSpec, as_splits, build_part, register_part


class Parallel(Mixer):
    MAX_BRANCHES = 4

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        branches = list(params["branches"])
        if not 1 <= len(branches) <= self.MAX_BRANCHES:
            raise ValueError(f"1 to {self.MAX_BRANCHES} mixers stand side by side, not {len(branches)}")
        self.branches = [build_part("mixer", b["part"], ctx) for b in branches]
        self.scales = [float(b.get("scale", 1.0)) for b in branches]
        self.prefixes = [str(b.get("prefix", "")) for b in branches]
        if len(set(self.prefixes)) != len(self.prefixes):
            raise ValueError("the branches' tensors need prefixes of their own")
        self.PROMPT_CAPTURABLE = all(bool(m.PROMPT_CAPTURABLE) for m in self.branches)
        self.PEERS = tuple(sorted({p for m in self.branches for p in m.PEERS}))

    def attach(self, peers):
        for m in self.branches:
            if m.PEERS:
                m.attach({k: peers[k] for k in m.PEERS})

    def tensor_specs(self):
        return [TensorSpec(pre + s.name, s.shape, s.role, s.optional, s.init, s.init_arg)
                for pre, m in zip(self.prefixes, self.branches) for s in m.tensor_specs()]

    def load(self, fetch):
        for pre, m in zip(self.prefixes, self.branches):
            m.load((lambda p: (lambda local: fetch(p + local)))(pre))

    def tensor(self, name):
        for pre, m in zip(self.prefixes, self.branches):
            if name.startswith(pre):
                t = m.tensor(name[len(pre):])
                if t is not None:
                    return t
        return None

    def cache_need(self):
        needs = tuple(m.cache_need() for m in self.branches)
        return CacheNeed("several", parts=needs) if any(n is not None for n in needs) else None

    def weight_bytes(self):
        return sum(m.weight_bytes() for m in self.branches)

    def forward(self, x, batch, cache, write_cache):
        views = cache.parts if cache is not None else [None] * len(self.branches)
        terms = [(as_splits(m.forward(x, batch, v, write_cache)), f) for m, v, f in zip(self.branches, views, self.scales)]
        return ops.weighted_sum(terms)


register_part("mixer", "parallel", Parallel)
