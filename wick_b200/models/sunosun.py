"""The Sunosun decoder as a model spec.

The embedding's rows are multiplied by a factor and a sinusoid vector of the position is added.  Every layer is
a pre-norm residual block, x <- x + mixer(norm1(x)), then x <- x + ff(norm2(x)), RMS norms with plain weights.
Mixers: ``gla`` (a gated linear attention: a matrix state per head with a decay per key channel, a per-head norm
of the result and an output gate) or ``parallel`` (a causal softmax attention with biased projections, no
positions and a sink of score 0, beside a gated linear attention; the two results are added with a factor each).
The feed-forward is a gated one or a mixture of one-matrix experts (squared ReLU) chosen by sigmoid scores
within the best groups of experts, plus an expert every token uses whose result is gated by one number per
token.  A range of layers may run several times in a row with the same weights and a state of its own each time;
every pass begins with x <- x + (the embedding's output, but for the first pass) + a vector of the pass.  The
logits come from the embedding table itself and are soft-capped.
Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.base import Architecture, register_architecture
from ..config.sunosun import SunosunAttention, SunosunConfig, SunosunLinearAttention, SunosunMLP
from ..parts import linear_attention as _linear_attention, parallel as _parallel, routed as _routed, side_input as _side   # register the kinds  # noqa: F401
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, SharedPart

_ATT_NAMES = dict(q="q", k="k", v="v", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b")
_GLA_NAMES = dict(q="q", k="k", v="v", gate="g", o="o", norm="norm", decay_in="a1", decay_out="a2", decay_bias="a2.b")
_DENSE_NAMES = dict(gate="gate", up="up", down="down")
_EXPERT_NAMES = dict(up="up", down="down", expert="e{i}.", router="router", correction="correction", shared="shared.",
                     shared_gate="shared.sg")

SINUSOID_BASE = 10000.0            # the position vectors' base
NORM_EPS = 1e-20                   # added to the chosen experts' scores' sum
GROUP_TOP = 2                      # a group's score adds up this many of its members' scores (fixed in the router's kernel)


def _attention(cfg: SunosunConfig, m: SunosunAttention) -> PartSpec:
    return PartSpec("attention", {
        "width": cfg.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim, "scale": m.scale,
        "bias": True, "qk_norm": None, "position": None, "mask": None, "sink_value": 0.0, "names": _ATT_NAMES})


def _linear_attention_spec(cfg: SunosunConfig, m: SunosunLinearAttention) -> PartSpec:
    return PartSpec("gated_linear_attention", {
        "width": cfg.width, "heads": m.heads, "head_dim": m.dim, "v_dim": m.vdim, "tau": m.tau, "eps": cfg.norm_eps,
        "rank": m.rank, "names": _GLA_NAMES})


def _feed_forward(cfg: SunosunConfig, m: SunosunMLP) -> PartSpec:
    if m.kind == "dense":
        return PartSpec("gated_mlp", {"width": cfg.width, "intermediate": m.ff, "activation": "silu", "names": _DENSE_NAMES})
    shared = PartSpec("mlp", {"width": cfg.width, "intermediate": m.shared_ff, "activation": "relu2",
                              "names": {"up": "up", "down": "down"}}) if m.shared_ff else None
    return PartSpec("routed_moe", {
        "width": cfg.width, "experts": m.experts, "top": m.top, "intermediate": m.ff, "scores": "sigmoid", "correction": True,
        "renormalize": True, "norm_eps": NORM_EPS, "route_scale": m.scale, "expert": "relu2",
        "groups": {"count": m.group_count, "keep": m.group_keep} if m.group_count else None,
        "shared": shared, "shared_gate": shared is not None, "names": _EXPERT_NAMES})


def build_spec(cfg: SunosunConfig) -> ModelSpec:
    def norm(optional=False):
        return PartSpec("rms", {"width": cfg.width, "eps": cfg.norm_eps, "tensor": "", "optional": optional})

    layers = []
    for i, L in enumerate(cfg.layers):
        if L.type == "gla":
            mixer = _linear_attention_spec(cfg, L.mixer)
        else:
            mixer = PartSpec("parallel", {"width": cfg.width, "branches": (
                {"part": _attention(cfg, L.mixer.left), "scale": L.mixer.left_scale, "prefix": "left."},
                {"part": _linear_attention_spec(cfg, L.mixer.right), "scale": L.mixer.right_scale, "prefix": "right."})})
        ffn = PartSpec("none") if L.mlp is None else _feed_forward(cfg, L.mlp)
        layers.append(LayerSpec(block=PartSpec("prenorm_residual", {"width": cfg.width}), mixer=mixer, mixer_norm=norm(), ffn=ffn,
                                ffn_norm=norm(optional=L.mlp is None), prefix=f"l{i}.",
                                names={"mixer": "mix.", "mixer_norm": "norm1", "ffn": "mlp.", "ffn_norm": "norm2"}))
    shared = ()
    if cfg.loop is not None:
        shared = (SharedPart("pass_offset", "side", PartSpec("pass_offset", {"width": cfg.width, "passes": cfg.loop.times,
                                                                             "add_embedding": True, "tensor": ""}), "loop.step"),)
    spec = ModelSpec(
        architecture=cfg.architecture, vocab=cfg.vocab_size, width=cfg.width, max_position=cfg.max_position,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "width": cfg.width, "tensor": "", "scale": cfg.embedding_scale,
                                     "position": {"kind": "sinusoid", "base": SINUSOID_BASE}}),
        embedding_prefix="embed", layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, before="pass_offset" if t is not None else None, before_index=t or 0)
                       for i, t in cfg.run_order()),
        final_norm=norm(), final_norm_prefix="final.norm",
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "width": cfg.width, "tied": True, "tensor": "",
                                 "soft_cap": cfg.logit_softcap}),
        head_prefix="head", shared=shared)
    spec.validate()
    return spec


SUNOSUN = register_architecture(Architecture(names=("Sunosun", "sunosun"), config_cls=SunosunConfig, build_spec=build_spec))
