"""The Fasunex decoder as a model spec.

Every layer is a pre-norm residual block whose sublayers' results are normed once more before they
join the stream: x <- x + norm1b(mixer(norm1(x))), then x <- x + norm2b(ff(norm2(x))), RMS norms with
plain weights.  Mixers: ``attention`` (no value matrix: the keys as projected are the values; q and k
normed per head; no positions; a sink; an output gate) or ``parallel`` (a chunked attention with a
rotation, a weightless norm of q and k after it, a sink and an output gate, beside a state-space
recurrence with a short convolution; the two results are added with a factor each).  The feed-forward
is a mixture of gated experts chosen by a router, some of whose outputs stand for experts that return
their input.  A range of layers may run several times in a row with the same weights and a cache of
its own each time; every pass begins with a product that mixes the stream with the embedding output.
Tensor names: ``embed``, ``loop.in``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import Architecture, register_architecture
from ..config.fasunex import FasunexAttention, FasunexConfig, FasunexStateSpace
from ..parts import parallel as _parallel, routed as _routed, side_input as _side, state_space as _state_space   # register the kinds  # noqa: F401
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, SharedPart

_MIX_NAMES = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", sink="sink", gate="g")
_SSM_NAMES = dict(input="in", conv="conv", conv_bias="conv.b", dt_bias="dt_bias", a_log="A_log", d="D", norm="norm", o="o")
_EXPERT_NAMES = dict(gate="gate", up="up", down="down", expert="e{i}.", router="router", correction="correction")


def _attention(cfg: FasunexConfig, m: FasunexAttention, keys_are_values: bool) -> PartSpec:
    position = PartSpec("rotary_pairs", {"head_dim": m.dim, "dims": m.rot_dims, "theta": m.rot_base,
                                         "pairing": "halves"}) if m.rot_dims else None
    return PartSpec("attention", {
        "width": cfg.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim, "scale": m.scale,
        "qk_norm": "head", "qk_norm_weight": keys_are_values, "qk_norm_after_rotation": not keys_are_values,
        "eps": cfg.norm_eps, "position": position, "values": "keys" if keys_are_values else "own",
        "mask": {"kind": "block", "size": m.mask_size} if m.mask_size is not None else None, "sink": True,
        "gate": True, "names": _MIX_NAMES})


def _state_space(cfg: FasunexConfig, s: FasunexStateSpace) -> PartSpec:
    return PartSpec("selective_state_space", {
        "width": cfg.width, "heads": s.heads, "head_dim": s.vdim, "state": s.state, "groups": s.groups, "taps": s.conv,
        "norm_groups": s.norm_groups, "eps": cfg.norm_eps, "names": _SSM_NAMES})


def build_spec(cfg: FasunexConfig) -> ModelSpec:
    def norm(optional=False):
        return PartSpec("rms", {"width": cfg.width, "eps": cfg.norm_eps, "tensor": "", "optional": optional})

    layers = []
    for i, L in enumerate(cfg.layers):
        if L.type == "attention":
            mixer = _attention(cfg, L.mixer, True)
        else:
            mixer = PartSpec("parallel", {"width": cfg.width, "branches": (
                {"part": _attention(cfg, L.mixer.left, False), "scale": L.mixer.left_scale, "prefix": "left."},
                {"part": _state_space(cfg, L.mixer.right), "scale": L.mixer.right_scale, "prefix": "right."})})
        if L.mlp is None:
            ffn = PartSpec("none")
        else:
            ffn = PartSpec("routed_moe", {"width": cfg.width, "experts": L.mlp.experts, "identity": L.mlp.identity,
                                          "top": L.mlp.top, "intermediate": L.mlp.ff, "scores": "softmax",
                                          "correction": True, "renormalize": False, "names": _EXPERT_NAMES})
        block = PartSpec("prenorm_residual", {"width": cfg.width,
                                              "post_norm": {"mixer": "norm1b", "ffn": "norm2b", "eps": cfg.norm_eps}})
        layers.append(LayerSpec(block=block, mixer=mixer, mixer_norm=norm(), ffn=ffn, ffn_norm=norm(optional=L.mlp is None),
                                prefix=f"l{i}.", names={"mixer": "mix.", "mixer_norm": "norm1", "ffn": "mlp.", "ffn_norm": "norm2"}))
    shared = ()
    if cfg.loop is not None:
        shared = (SharedPart("pass_input", "side", PartSpec("mix_with_embedding", {"width": cfg.width, "tensor": ""}), "loop.in"),)
    spec = ModelSpec(
        architecture=cfg.architecture, vocab=cfg.vocab_size, width=cfg.width, max_position=cfg.max_position,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "width": cfg.width, "tensor": ""}), embedding_prefix="embed",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, before="pass_input" if enter else None) for i, enter in cfg.run_order()),
        final_norm=norm(), final_norm_prefix="final.norm",
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "width": cfg.width, "tied": False, "tensor": ""}),
        head_prefix="head", shared=shared)
    spec.validate()
    return spec


FASUNEX = register_architecture(Architecture(names=("Fasunex", "fasunex"), config_cls=FasunexConfig, build_spec=build_spec))
