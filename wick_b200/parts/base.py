"""The interfaces of the parts a layer is put together from, and their registry.

Categories: ``mixer`` (token mixing over the sequence: attention here),
``ffn`` (feed-forward), ``norm``, ``position`` (position encoding), ``block``
(the arrangement of the former in one layer), ``side`` (what a layer adds to the
stream after its feed-forward from something else than the stream alone),
``embedding`` and ``head``.

A part is built from a :class:`~wick_b200.models.spec.PartSpec` — its registered
kind plus its sizes and constants — and a :class:`BuildContext` (compute dtype
and device).  It declares the tensors it needs by local name, receives them
through :meth:`Part.load`, and computes with the kernels of ``wick_b200.ops``.
No part knows which model it is in, which layer it is, or what its neighbours
are: everything it needs is in its parameters and in the arguments of
``forward``.

Adding a part: subclass the category's base class, implement its methods,
and call :func:`register_part` with a new kind name; a model spec can then
name that kind.  Nothing else in the package has to change.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..models.spec import PartSpec

CATEGORIES = ("mixer", "ffn", "norm", "position", "block", "side", "embedding", "head")


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    """A tensor a part needs.  ``role`` decides how it is held:
    ``matrix``: in the compute dtype (bfloat16 or float32);
    ``vector``: always float32 (norm weights and the like: tensors that a
    checkpoint stores in 32-bit stay 32-bit, and 16-bit vectors are widened
    exactly, as wick does for every 1-D tensor, model.rs:136-142);
    ``table``: integers, as int32.

    ``init`` tells the random-weights writer what a sensible value looks like where the
    role's default (matrices N(0, std), vectors 1 + N(0, vector_std)) is none:
    ``around_zero`` (a vector that is added, or a norm weight stored as its distance from
    one), ``unit_interval`` (a blend factor), ``distinct_below`` (integer rows of different
    values below ``init_arg``), ``absent`` (an optional tensor that random models leave out),
    ``conv_taps`` (a short filter's taps, N(0, 1 / taps)), ``router`` (rows whose scores differ
    from token to token), ``mix_pair`` (a matrix [w, 2 w] near the sum of its two halves' inputs), ``decay_out`` and
    ``decay_bias`` (the second step and the bias of a decay's logits).

    A size of -1 in ``shape`` is whatever the checkpoint has there (the part checks it against its other tensors when it
    loads); random weights take ``init_arg`` for it."""

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False
    init: str = ""
    init_arg: int = 0


@dataclasses.dataclass(frozen=True)
class BuildContext:
    dtype: torch.dtype            # torch.bfloat16 or torch.float32
    device: torch.device

    def hold(self, t: torch.Tensor, role: str) -> torch.Tensor:
        """Move a loaded tensor to the device in the dtype its role asks for."""
        if role == "matrix":
            dt = self.dtype
        elif role == "vector":
            dt = torch.float32
        elif role == "table":
            dt = torch.int32
        else:
            raise ValueError(f"unknown tensor role {role}")
        if t.dtype == torch.float16 and dt == torch.bfloat16:
            t = t.to(torch.float32)          # f16 -> f32 -> bf16, round to nearest even (model.rs:67-71)
        return t.to(device=self.device, dtype=dt).contiguous()


Fetch = Callable[[str], Optional[torch.Tensor]]


@dataclasses.dataclass(frozen=True)
class CacheNeed:
    """What a mixer asks of the cache for one schedule entry.

    kind ``paged_kv``: keys and values of every position, ``kv_heads`` x
    ``head_dim`` each, in pages (values ``v_head_dim`` each, if that is given and
    differs); ``window`` (tokens) if only the last ones are ever read.  kind ``paged_rows``:
    one row of ``shape`` per position, in the same pages.  kind ``state``: one record of fixed
    ``shape`` and ``dtype`` per sequence, zeroed when the sequence starts.  kind ``several``:
    a mixer made of several keeps what each of ``parts`` asks for; its cache view's ``parts``
    are the views of those, in order."""

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    shape: Tuple[int, ...] = ()
    dtype: Optional[torch.dtype] = None   # None: the compute dtype
    v_head_dim: Optional[int] = None      # None: as head_dim
    parts: Tuple["CacheNeed", ...] = ()


class Part:
    category = ""
    # Other places of the model whose part this one needs to see ("embedding", "final_norm",
    # "head"): the model hands them over through :meth:`attach` before any weight is loaded.
    # (An output head that shares the embedding table names "embedding".)
    PEERS: Tuple[str, ...] = ()
    # True if a prompt step of this part reads the step's shape (which token belongs to which
    # sequence, lengths, positions, pages) from the batch's DEVICE arrays only and sizes its
    # launches by ``batch.n_tokens``, ``batch.n_seqs`` and ``batch.q_tiles`` alone.  The engine
    # captures prompt steps of padded sizes and replays them for other prompts only if every
    # part of the model says so; the host lists of such a captured batch (``q_lens``,
    # ``starts``) describe no real prompt.
    PROMPT_CAPTURABLE = False

    def __init__(self, params: Mapping[str, Any], ctx: BuildContext):
        self.params = dict(params)
        self.ctx = ctx

    def attach(self, peers: Mapping[str, "Part"]) -> None:
        """Receive the parts named in ``PEERS`` (place -> part)."""

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, fetch: Fetch) -> None:
        """Take the tensors named by :meth:`tensor_specs` (``fetch(local_name)``
        returns a tensor of the declared shape, or None for an absent optional
        one) and keep them on the device."""

    def tensor(self, name: str) -> Optional[torch.Tensor]:
        """The tensor held under the local ``name``, in the shape and layout a checkpoint
        stores it in (on the device, in the dtype it is held in), however the part keeps
        it for its kernels; None if the part holds none of that name.  For handing a
        model's weights to another implementation."""
        return None

    def weight_bytes(self) -> int:
        """Bytes of weights one forward pass of this part reads."""
        return 0


class Norm(Part):
    category = "norm"

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Normalise the float32 rows of ``x`` [n, width] (only ``rows`` of
        them, if given) into a new [n or len(rows), width] tensor."""
        raise NotImplementedError

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None, *, scale: Optional[torch.Tensor] = None,
                    rms: Optional[Tuple[torch.Tensor, float]] = None) -> torch.Tensor:
        """``x += sum(delta)`` in float32 and in place (``delta`` is
        [splits, n, width], summed in index order), then normalise.  With
        ``rows`` only those rows are normalised and ``x`` need not be brought up
        to date (nobody reads it afterwards).  ``scale`` (float32 [width]): the
        sum is multiplied by it element by element before it is added; ``rms``
        (weight, eps): the sum is divided by its root mean square and multiplied
        by the weight first.  A norm without a kernel for these resolves the sum
        into ``x`` with the stream kernel and normalises then."""
        from .. import ops
        ops.stream_update(x, delta, scale=scale, rms=rms)
        return self.forward(x, out_dtype, rows)

    def scaled_add_forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], alpha: float,
                           out_dtype: torch.dtype) -> torch.Tensor:
        """The norm AFTER the sum: ``x <- norm(alpha * x + sum(delta))`` in float32 and in
        place (``delta`` [splits, n, width] or None); returns the new rows in ``out_dtype``
        (for float32, ``x`` itself)."""
        x.mul_(alpha)
        if delta is not None:
            x.add_(delta.sum(0) if delta.shape[0] > 1 else delta[0])
        x.copy_(self.forward(x, torch.float32))
        return x if out_dtype == torch.float32 else x.to(out_dtype)


class Position(Part):
    category = "position"

    def rotary_inv_freq(self) -> Optional[torch.Tensor]:
        """If this encoding is a half-split rotation of whole heads by
        ``position * inv_freq[i]``, the float32 table [head_dim/2] (kernels then
        fuse it); otherwise None and :meth:`apply` is called."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Encode positions into q [n, heads, d] and k [n, kv_heads, d] in place."""
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, x: torch.Tensor, batch: "Any", cache: "Any", write_cache: bool) -> torch.Tensor:
        """x: [tokens, width] in the compute dtype (already normalised).
        batch: the step's :class:`~wick_b200.engine.batch.StepBatch`.
        cache: the view of this schedule entry's cache storage for this batch
        (None if :meth:`cache_need` is None).  write_cache is False when the
        entry reads an earlier entry's cache.
        Returns float32 [splits, tokens, width], to be summed into the residual.

        A mixer (or feed-forward) whose class sets ``ADDS_TO_RESIDUAL = True`` is
        also given ``residual=`` (the float32 residual stream [tokens, width]); it
        may add its result to it itself (each element once, in a fixed order) and
        return None."""
        raise NotImplementedError


class FeedForward(Part):
    category = "ffn"

    def forward(self, x: torch.Tensor, batch: "Any") -> torch.Tensor:
        """x: [tokens, width], compute dtype.  Returns float32 [splits, tokens, width]."""
        raise NotImplementedError


class Hidden:
    """The residual stream between blocks: float32 ``x`` [tokens, width] and a
    float32 ``pending`` [splits, tokens, width] that has still to be added to it
    (kept apart so that the next norm's kernel can do the addition).  ``scale``
    (float32 [width]) is a factor, element by element, of the pending sum; ``rms``
    (weight, eps) says that the pending sum is divided by its root mean square and
    multiplied by the weight before it is added; both are None for a plain sum.  ``act``
    is ``x`` in the compute dtype where a block has made that copy (blocks whose
    sublayers read the stream itself), else None."""

    __slots__ = ("x", "pending", "act", "scale", "rms")

    def __init__(self, x: torch.Tensor, pending: Optional[torch.Tensor] = None):
        self.x, self.pending, self.act = x, pending, None
        self.scale: Optional[torch.Tensor] = None
        self.rms: Optional[Tuple[torch.Tensor, float]] = None

    def defer(self, delta: Optional[torch.Tensor], scale: Optional[torch.Tensor] = None,
              rms: Optional[Tuple[torch.Tensor, float]] = None) -> None:
        """Leave ``delta`` (None: nothing) to be added by whoever reads the stream next."""
        self.pending, self.scale, self.rms = delta, (scale if delta is not None else None), (rms if delta is not None else None)

    def resolved(self, act_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """The stream with everything added; with ``act_dtype`` its copy in that type is
        made on the way and left in ``act``."""
        from .. import ops
        if self.pending is not None and (self.scale is not None or self.rms is not None or act_dtype is not None):
            self.act = ops.stream_update(self.x, self.pending, scale=self.scale, rms=self.rms, out_dtype=act_dtype)
            self.defer(None)
        elif self.pending is not None:
            p = self.pending
            self.x.add_(p.sum(0) if p.shape[0] > 1 else p[0])
            self.pending = None
        elif act_dtype is not None and self.act is None:
            self.act = ops.to_activation(self.x, act_dtype)
        return self.x


class Block(Part):
    category = "block"

    def __init__(self, params, ctx, mixer: Mixer, mixer_norm: Norm, ffn: FeedForward, ffn_norm: Norm):
        super().__init__(params, ctx)
        self.mixer, self.mixer_norm, self.ffn, self.ffn_norm = mixer, mixer_norm, ffn, ffn_norm
        self.side: Optional["SideInput"] = None        # set by the model where the layer's spec names one

    def forward(self, h: Hidden, batch: "Any", cache: "Any", write_cache: bool) -> Hidden:
        raise NotImplementedError


class SideInput(Part):
    """What a layer adds to the stream after its feed-forward from something else than
    the stream alone."""
    category = "side"

    def forward(self, h: Hidden, batch: "Any", index: int = 0) -> None:
        """``h`` comes with everything of the layer added or pending; the part leaves
        its own addition in ``h`` (added, or pending through :meth:`Hidden.defer`).  ``index``:
        the number a schedule entry gives a shared part that runs before it (which pass begins)."""
        raise NotImplementedError


class Embedding(Part):
    category = "embedding"

    NEEDS_POSITIONS = False      # True: forward is also given the tokens' positions (int32 [n])

    def forward(self, tokens: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        """int32 [n] -> float32 [n, width]."""
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """[n, width] in the compute dtype -> float32 logits [n, vocab]."""
        raise NotImplementedError


_PARTS: Dict[str, Dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: type) -> type:
    if category not in _PARTS:
        raise ValueError(f"unknown part category {category}")
    _PARTS[category][kind] = cls
    return cls


def part_class(category: str, kind: str) -> type:
    try:
        return _PARTS[category][kind]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(category, {})))
        raise KeyError(f"no {category} part of kind {kind!r} is registered (known: {known})") from None


def build_part(category: str, spec: PartSpec, ctx: BuildContext, *args) -> Part:
    return part_class(category, spec.kind)(spec.params, ctx, *args)


def as_splits(delta: torch.Tensor) -> torch.Tensor:
    """A part may return [tokens, width]; the residual path wants [splits, tokens, width]."""
    return delta if delta.dim() == 3 else delta.unsqueeze(0)
