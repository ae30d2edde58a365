"""The Sunosun decoder and its mechanisms against the plain implementation in ``tests/plain/sunosun_plain.py``: every
mechanism alone through its part or kernel, then whole models through the engine (prompts, decoding, portions, batches,
reused pages, slots and records, far tokens, generation).  The configurations differ from each other in every size and
option and include the values that make mechanisms vanish or coincide (no loop, a loop over one layer, no soft cap, an
embedding factor of one, one key/value head, as many as query heads, groups of one expert, one group, no groups, no
shared expert, one choice, tau = 1, no feed-forward, widths and head sizes that are no multiples of four)."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import wick_b200 as wick  # noqa: E402
from wick_b200 import ops  # noqa: E402
from wick_b200.engine.batch import BatchLayout, StepBatch, fill_host  # noqa: E402
from wick_b200.models.spec import PartSpec  # noqa: E402
from wick_b200.parts.base import BuildContext, Hidden, build_part  # noqa: E402
from wick_b200.parts import attention as _att, linear_attention as _gla, parallel as _par, routed as _routed, side_input as _side  # noqa: E402,F401
from wick_b200.weights.safetensors_io import SafeTensorsDir  # noqa: E402
from helpers import random_tokens, tmp_root  # noqa: E402
from plain import sunosun_plain as P  # noqa: E402

PAGE = 64
DEV = "cuda"


def gla(heads, dim, vdim, tau, rank=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, tau=tau)
    if rank is not None:
        m["rank"] = rank
    return m


def left(heads, kv, dim, vdim, scale):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)


def par(l, r, ls, rs):
    return dict(type="parallel", mixer=dict(left=l, right=r, left_scale=ls, right_scale=rs))


def lin(m):
    return dict(type="gla", mixer=m)


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, scale, groups=None, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


# SA: a loop of two passes over the two middle layers; groups of two experts; a layer without feed-forward; a rank of 5
CONFIG_SA = dict(architecture="Sunosun", vocab=211, width=64, norm={"eps": 1e-5}, embedding={"scale": 2.0}, logit_softcap=9.0,
                 loop={"start": 1, "stop": 3, "times": 2}, layers=[
    layer(lin(gla(3, 8, 4, 4.0, 5)), dense(80)),
    layer(par(left(4, 2, 16, 24, 0.3), gla(2, 4, 12, 1.0), 0.7, 1.3), None),
    layer(lin(gla(1, 16, 16, 16.0)), moe(24, 3, 1, 1.0)),
    layer(lin(gla(3, 8, 4, 4.0, 5)), moe(40, 6, 3, 2.5, groups=(3, 2), shared=20)),
])
# SB: no loop, no soft cap, an embedding factor of one; as many key/value heads as query heads; groups of one expert of which
# all are kept; one group; a shared expert without groups
CONFIG_SB = dict(architecture="Sunosun", vocab=130, width=72, norm={"eps": 1e-6}, layers=[
    layer(par(left(3, 3, 8, 8, 0.35), gla(6, 4, 8, 2.0, 2), 1.0, 1.0), moe(52, 5, 2, 1.0, groups=(5, 5))),
    layer(lin(gla(2, 24, 20, 8.0)), moe(44, 4, 4, 0.5, groups=(1, 1), shared=12)),
    layer(par(left(6, 1, 10, 16, 0.3), gla(2, 20, 40, 32.0, 7), 0.5, -2.0), moe(16, 9, 2, 3.0, shared=40)),
])
# SC: heads of 64 and 128 numbers (the tensor-core attention), states of 128 x 128 and 64 x 96, a loop of three passes over the
# first layer alone
CONFIG_SC = dict(architecture="Sunosun", vocab=300, width=128, norm={"eps": 1e-5}, embedding={"scale": 0.5}, logit_softcap=30.0,
                 loop={"start": 0, "stop": 1, "times": 3}, layers=[
    layer(par(left(2, 1, 64, 64, 0.125), gla(2, 64, 96, 16.0), 1.1, 1.2), moe(64, 8, 2, 1.5, groups=(4, 2), shared=96)),
    layer(lin(gla(1, 128, 128, 8.0)), dense(256)),
    layer(par(left(4, 2, 128, 128, 0.09), gla(2, 32, 32, 4.0), 0.8, 0.6), None),
])
# SD: a width that is no multiple of eight, heads of 40, 24, 6, 10 and 9 numbers, a rank of 3, seven groups, a loop of three
# passes over the last layer
CONFIG_SD = dict(architecture="Sunosun", vocab=77, width=100, norm={"eps": 1e-6}, embedding={"scale": 1.5}, logit_softcap=5.0,
                 loop={"start": 2, "stop": 3, "times": 3}, layers=[
    layer(lin(gla(5, 6, 10, 3.0, 3)), moe(36, 14, 3, 1.0, groups=(7, 3), shared=28)),
    layer(par(left(5, 1, 40, 24, 0.2), gla(1, 9, 36, 16.0), 0.7, 1.3), dense(50)),
    layer(par(left(2, 2, 6, 6, 0.4), gla(3, 10, 6, 64.0, 1), 1.0, 1.0), moe(50, 7, 3, 2.0)),
])
CONFIGS = {"SA": CONFIG_SA, "SB": CONFIG_SB, "SC": CONFIG_SC, "SD": CONFIG_SD}
_models = {}
STD = 0.15
# float32 is compared on weights large enough for every part to weigh in the logits; bfloat16 on smaller ones, where an
# expert chosen differently after a router's close call (rounding decides it) moves the later rows less
STD_OF = {"float32": STD, "bfloat16": 0.08}


def write_model(cfg, d, seed=5, std=STD):
    wick.write_random_model(wick.config_from_json(cfg), seed, d, std=std)
    st = SafeTensorsDir(d)
    return {n: st.get(n).tensor() for n in st.names()}


def model(name, seed=5, std=STD):
    key = (name, seed, std)
    if key not in _models:
        d = os.path.join(tmp_root(), f"suno-{name}-{seed}-{std}")
        _models[key] = (d, write_model(CONFIGS[name], d, seed, std))
    return _models[key]


def engine(name, dtype, max_tokens=1024, **kw):
    return wick.Engine.from_dir(model(name, std=STD_OF[dtype])[0], dtype=dtype, max_tokens=max_tokens, **kw)


_plain = {}


def plain(name, tokens, dtype="float32"):
    key = (name, tuple(tokens), STD_OF[dtype])
    if key not in _plain:
        _plain[key] = P.forward(CONFIGS[name], model(name, std=STD_OF[dtype])[1], list(tokens)).float()
    return _plain[key]


def close(got, ref, dtype, what="", tol=None):
    """float32: every row within ``tol`` of the scale.  bfloat16: with random weights a router's close call may choose another
    expert than the plain model's, which replaces a whole expert's output at that row (and, through the states, moves later
    rows a little), so the median row must be within ``tol``, nine rows in ten within three times that, and at most one row in
    twenty further than a third of the scale away; float32 is the sharp comparison."""
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = max(1.0, ref.abs().max().item())
    rows = (got - ref).abs().reshape(got.shape[0], -1).max(-1).values / scale
    f32 = dtype in ("float32", torch.float32)
    tol = tol or (2e-4 if f32 else 2e-2)
    if f32:
        if rows.max().item() > tol:
            raise AssertionError(f"{what}: differs by {rows.max().item():.3e} of the scale {scale:.3g}, worst row {int(rows.argmax())}")
        return
    med, q90, worst = rows.median().item(), rows.quantile(0.9).item(), rows.max().item()
    far = int((rows > 0.34).sum())
    if med > tol or q90 > 3 * tol or far > max(1, rows.numel() // 20):
        raise AssertionError(f"{what}: median {med:.3e}, nine in ten within {q90:.3e}, worst {worst:.3e} (row {int(rows.argmax())}) "
                             f"of the scale {scale:.3g}")


def tight(got, ref, dtype, what="", tol=None):
    """For one mechanism alone, with the same choices on both sides: every row within the dtype's rounding."""
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = max(1e-6, ref.abs().max().item())
    worst = (got - ref).abs().max().item() / scale
    tol = tol or (3e-5 if dtype in ("float32", torch.float32) else 2.5e-2)
    assert worst <= tol, f"{what}: differs by {worst:.3e} of the scale {scale:.3g}"


DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def seq_batch(n_new, start=0, pages=None, slot=1):
    """A step of one sequence: ``n_new`` tokens after ``start`` cached ones."""
    n_pages = (start + n_new + PAGE - 1) // PAGE
    pages = pages if pages is not None else list(range(1, n_pages + 1))
    lay = BatchLayout(1, n_new, len(pages), 0)
    host = np.zeros(lay.size, dtype=np.int32)
    fill_host(lay, host, tokens=[[0] * n_new], starts=[start], slots=[slot], pages=[pages], want=[[]])
    return StepBatch(lay, torch.from_numpy(host).to(DEV), q_lens=[n_new], starts=[start])


def make_part(category, kind, params, dtype, tensors):
    """The part with the given tensors (local name -> float tensor), and the tensors as the part holds them (rounded to
    bfloat16 where it keeps them so), as float64 for the plain functions."""
    ctx = BuildContext(dtype=TORCH[dtype], device=torch.device(DEV))
    part = build_part(category, PartSpec(kind, params), ctx)
    specs = {s.name: s for s in part.tensor_specs()}
    assert set(specs) == set(tensors), (sorted(specs), sorted(tensors))
    for n, s in specs.items():
        assert all(a == b or b == -1 for a, b in zip(tensors[n].shape, s.shape)), (n, tuple(tensors[n].shape), s.shape)
    held = {n: (t.to(TORCH[dtype]) if specs[n].role == "matrix" else t.float()) for n, t in tensors.items()}
    part.load(lambda n: held[n])
    return part, {n: t.double() for n, t in held.items()}


def rnd(g, *shape, std=1.0):
    return torch.randn(*shape, generator=g) * std


ATT_NAMES = dict(q="q", k="k", v="v", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b")
GLA_NAMES = dict(q="q", k="k", v="v", gate="g", o="o", norm="norm", decay_in="a1", decay_out="a2", decay_bias="a2.b")
MOE_NAMES = dict(up="up", down="down", expert="e{i}.", router="router", correction="correction", shared="shared.", shared_gate="shared.sg")


def attention_params(width, m):
    return {"width": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"], "scale": m["scale"],
            "bias": True, "qk_norm": None, "position": None, "mask": None, "sink_value": 0.0, "names": ATT_NAMES}


def attention_part(dtype, width, m, g, std=0.3):
    """The attention part as the design uses it (biased projections, no positions, a sink of score 0) and random tensors."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = {"q": rnd(g, H * d, width, std=std), "k": rnd(g, G * d, width, std=std), "v": rnd(g, G * e, width, std=std),
         "o": rnd(g, width, H * e, std=std), "q.b": rnd(g, H * d, std=0.5), "k.b": rnd(g, G * d, std=0.5), "v.b": rnd(g, G * e, std=0.5)}
    return make_part("mixer", "attention", attention_params(width, m), dtype, t)


def gla_params(width, m, eps):
    return {"width": width, "heads": m["heads"], "head_dim": m["dim"], "v_dim": m["vdim"], "tau": m["tau"], "eps": eps,
            "rank": m.get("rank"), "names": GLA_NAMES}


def gla_part(dtype, width, m, eps, g, std=0.3, rank=None, decay_logit=None):
    """The linear-attention part and random tensors; ``decay_logit``: every channel's decay is sigmoid(that)^(1 / tau)."""
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    r = rank or m.get("rank") or 6
    t = {"q": rnd(g, H * dk, width, std=std), "k": rnd(g, H * dk, width, std=std), "v": rnd(g, H * dv, width, std=std),
         "g": rnd(g, H * dv, width, std=std), "o": rnd(g, width, H * dv, std=std), "norm": 1 + 0.3 * rnd(g, dv),
         "a1": rnd(g, r, width, std=std), "a2": rnd(g, H * dk, r, std=1.5), "a2.b": 1 + rnd(g, H * dk)}
    if decay_logit is not None:
        t["a2"], t["a2.b"] = torch.zeros(H * dk, r), torch.full((H * dk,), float(decay_logit))
    return make_part("mixer", "gated_linear_attention", gla_params(width, m, eps), dtype, t)


def kv_cache(part, n_pages, dtype):
    need = part.cache_need()
    e = need.head_dim if need.v_head_dim is None else need.v_head_dim
    if e != need.head_dim:
        return torch.zeros((n_pages, need.kv_heads * PAGE * (need.head_dim + e)), dtype=TORCH[dtype], device=DEV)
    return torch.zeros((n_pages, 2, need.kv_heads, PAGE, need.head_dim), dtype=TORCH[dtype], device=DEV)


class View:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def gla_view(part, slots=3):
    """Records as the cache hands them out: NaN everywhere but in slot 1, which a sequence has just opened."""
    rec = torch.full((slots, part.record_floats()), float("nan"), device=DEV)
    rec[1].zero_()
    return View(state=rec, slots=None)


def run_mixer(part, h, dtype, cuts, view):
    """The part's result for the rows of ``h`` fed in portions of the sizes ``cuts``: float32 [n, width]."""
    out, at = [], 0
    for n in cuts:
        x = h[at:at + n].to(DEV, TORCH[dtype]).contiguous()
        d = part.forward(x, seq_batch(n, at), view, True)
        out.append(d.sum(0) if d.dim() == 3 else d)
        at += n
    assert at == h.shape[0]
    return torch.cat(out)


def as_held(h, dtype):
    return h.to(TORCH[dtype]).double()


# ---------------------------------------------------------------------------
# mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,scale", [(64, 2.0), (101, 1.0), (6, 0.25), (258, 3.5)])
def test_embedding_rows_times_a_factor_plus_the_positions_vectors(dtype, width, scale):
    g = torch.Generator().manual_seed(width)
    vocab = 50
    part, t = make_part("embedding", "table", {"vocab": vocab, "width": width, "tensor": "", "scale": scale,
                                               "position": {"kind": "sinusoid", "base": 10000.0}}, dtype, {"": rnd(g, vocab, width)})
    pos = torch.tensor([0, 1, 2, 3, 63, 64, 65, 1000, 4097, 30000], dtype=torch.int32)
    toks = torch.randint(0, vocab, (len(pos),), generator=g, dtype=torch.int32)
    got = part.forward(toks.to(DEV), pos.to(DEV))
    assert got.dtype == torch.float32
    rows = t[""][toks.long()] * scale
    # the angle is the float32 product of the position and a frequency that was rounded to float32 once
    pv32 = torch.cat([P.position_vectors(1, width, torch.float32, first=int(p)) for p in pos])
    assert (got.cpu().double() - (rows + pv32.double())).abs().max().item() <= 2e-6 * max(1.0, scale * 4)
    # against the exact angle: a float32 angle of 30000 is off by up to 30000 * 2^-24
    pv = torch.cat([P.position_vectors(1, width, torch.float64, first=int(p)) for p in pos])
    assert (got.cpu().double() - (rows + pv)).abs().max().item() <= 3e-3
    assert (got.cpu().double()[:7] - (rows + pv)[:7]).abs().max().item() <= 1e-5
    # position 0: sines 0 and cosines 1, so the vector shows which elements are which
    zero = part.forward(toks[:1].to(DEV), pos[:1].to(DEV)).cpu().double()[0] - rows[0]
    assert zero[0::2].abs().max() < 1e-6 and (zero[1::2] - 1).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,e,scale", [(4, 1, 16, 32, 0.3), (2, 2, 12, 20, 0.3), (3, 3, 8, 8, 0.4), (2, 1, 64, 64, 0.125),
                                            (4, 2, 128, 128, 0.09), (6, 3, 48, 40, 0.15), (5, 1, 40, 24, 0.2), (2, 2, 6, 6, 0.5)])
def test_attention_with_biases_without_positions_and_one_added_to_the_denominator(dtype, H, G, d, e, scale):
    g = torch.Generator().manual_seed(H * 100 + d + e)
    width, n = 48, 200
    m = left(H, G, d, e, scale)
    part, t = attention_part(dtype, width, m, g)
    h = rnd(g, n, width)
    ref = P.softmax_attention(as_held(h, dtype), t, "", m)
    for cuts in ([n], [1] * 4 + [2, 60, 5, 64, 65], [199, 1]):
        got = run_mixer(part, h, dtype, cuts, View(kv=kv_cache(part, 5, dtype)))
        tight(got, ref, dtype, f"cuts {cuts[:3]}")


def test_the_first_token_shares_its_weight_with_the_sink():
    """One token alone: its weight is exp(s) / (1 + exp(s)), not 1; with a zero query the score is 0 and the weight one half."""
    g = torch.Generator().manual_seed(5)
    width, m = 24, left(2, 1, 8, 12, 0.5)
    part, t = attention_part("float32", width, m, g)
    held = {k: v.float() for k, v in t.items()}
    held["q"], held["q.b"] = torch.zeros_like(held["q"]), torch.zeros_like(held["q.b"])
    part, t = make_part("mixer", "attention", attention_params(width, m), "float32", held)
    h = rnd(g, 1, width)
    v = h.double() @ t["v"].T + t["v.b"]                               # [1, e]; both query heads read the one key/value head
    want = 0.5 * torch.cat([v, v], -1) @ t["o"].T
    got = run_mixer(part, h, "float32", [1], View(kv=kv_cache(part, 2, "float32")))
    tight(got, want, "float32", "half the value")
    # three tokens with zero queries: weights 1/2; 1/3, 1/3; 1/4, 1/4, 1/4
    h = rnd(g, 3, width)
    v = h.double() @ t["v"].T + t["v.b"]
    mean = torch.stack([v[:i + 1].sum(0) / (i + 2) for i in range(3)])
    want = torch.cat([mean, mean], -1) @ t["o"].T
    for cuts in ([3], [1, 1, 1], [2, 1]):
        tight(run_mixer(part, h, "float32", cuts, View(kv=kv_cache(part, 2, "float32"))), want, "float32", f"cuts {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_that_stands_out_far_back_and_at_page_borders(dtype):
    """With Wk = Wq, equal biases, and inputs at two positions i > j that differ only by a vector that Wq maps to zero, the
    score of (i, j) equals that of (i, i), the squared length of a query of 64 numbers, which stands out among hundreds of
    products of unrelated vectors: the result at i is close to the mean of v_i and v_j.  A twin at a later position is not seen.  The rows
    are checked against the plain function in a prompt, in portions and decoded alone."""
    g = torch.Generator().manual_seed(77)
    width, H, d, n = 160, 2, 64, 640
    m = left(H, H, d, d, 0.0117)                          # (the pair's score is around 30, the others' around 0 +- 4)
    part, t = attention_part(dtype, width, m, g, std=0.5)
    held = {k: v.float() for k, v in t.items()}
    held["k"], held["k.b"] = held["q"].clone(), held["q.b"].clone()
    part, t = make_part("mixer", "attention", attention_params(width, m), dtype, held)
    h = rnd(g, n, width)
    pairs = [(599, 3), (598, 0), (450, 63), (639, 64), (601, 597), (127, 1), (128, 65), (511, 448), (512, 447), (383, 320), (384, 191),
             (192, 193), (255, 256)]                                  # (the last two: the twin comes later)
    null = torch.linalg.svd(t["q"])[2][H * d:].T.float()       # [width, width - H d]: what the q (and k) matrix maps to zero
    for i, j in pairs:
        h[j] = h[i] + null @ rnd(g, null.shape[1], std=3.0)
    hd = as_held(h, dtype)
    ref = P.softmax_attention(hd, t, "", m)
    q = (hd @ t["q"].T + t["q.b"]).view(n, H, d)
    for i, j in pairs:
        others = torch.einsum("hd,jhd->hj", q[i], q[:i]) * m["scale"]
        own = (q[i] * q[i]).sum(-1) * m["scale"]
        others[:, j if j < i else 0] = -1e9
        assert (own - others.max(-1).values).min() > 6, "the pair's score does not stand out"
    for cuts in ([n], [300, 340], [64, 64, 2, 190, 320]):
        got = run_mixer(part, h, dtype, cuts, View(kv=kv_cache(part, 11, dtype)))
        tight(got, ref, dtype, f"cuts {cuts[:3]}")
    for i, j in pairs[:8]:                                    # decoded: i alone after a prompt that ends right before it
        got = run_mixer(part, h[:i + 1], dtype, [i, 1], View(kv=kv_cache(part, 11, dtype)))
        tight(got[i:], ref[i:i + 1], dtype, f"position {i} decoded, its twin at {j}")
    # a twin that is seen matters (without it the row is another one); one that comes later does not
    h2 = h.clone()
    for i, j in pairs:
        h2[j] = rnd(g, width)
    ref2 = P.softmax_attention(as_held(h2, dtype), t, "", m)
    for i, j in pairs:
        moved = (ref2[i] - ref[i]).abs().max() > 1e-2 * ref.abs().max()
        assert moved == (j < i), (i, j)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dk,dv,rank,tau", [(3, 8, 4, 5, 4.0), (2, 16, 16, 4, 16.0), (1, 6, 10, 3, 1.0), (2, 128, 128, 16, 8.0),
                                               (4, 20, 36, 2, 2.0), (1, 300, 8, 7, 16.0), (2, 64, 96, 16, 16.0), (5, 9, 7, 1, 64.0),
                                               (2, 16, 8, 40, 4.0), (1, 12, 20, 64, 2.0), (3, 100, 12, 33, 8.0)])
def test_gated_linear_attention_in_any_portions(dtype, H, dk, dv, rank, tau):
    g = torch.Generator().manual_seed(H * 1000 + dk)
    width, n = 40, 350                                       # (a step of 192 tokens or more is scanned in chunks of 64)
    m = gla(H, dk, dv, tau, rank)
    part, t = gla_part(dtype, width, m, 1e-5, g)
    h = rnd(g, n, width)
    ref = P.gated_linear_attention(as_held(h, dtype), t, "", m, 1e-5)
    a = P.decays(as_held(h, dtype), t, "", m)
    assert a.min() > 0 and a.max() <= 1 and (a.max() - a.min()) > 0.05, "decays that differ from channel to channel"
    for cuts in ([n], [1] * 6 + [2, 3, 2, 59, 64, 1, 1, 12, 200], [349, 1], [75, 75, 8, 192], [192, 158]):
        got = run_mixer(part, h, dtype, cuts, gla_view(part))
        tight(got, ref, dtype, f"cuts {cuts[:3]}")


def test_the_recurrence_and_the_per_head_norm_on_their_own():
    """ops.gla_mix and ops.gla_norm_gate from given q, k, v, g and decay logits (W2 the identity): the state after the
    step, [H][dv][dk] in the record, is the plain recurrence's last state, and the decay acts on key channels."""
    g = torch.Generator().manual_seed(8)
    H, dk, dv, n, tau = 2, 5, 3, 70, 2.0
    q, k, v, gate, z = rnd(g, n, H * dk), rnd(g, n, H * dk), rnd(g, n, H * dv), rnd(g, n, H * dv), 2 * rnd(g, n, H * dk)
    parts = torch.cat([q, k, v, gate, z], -1)[None].contiguous().to(DEV)
    rec = torch.full((3, H * dv * dk), float("nan"), device=DEV)
    rec[1].zero_()
    w2 = torch.eye(H * dk).to(DEV)
    for cuts in ([n], [1] * 5 + [65]):
        rec[1].zero_()
        outs, at = [], 0
        for c in cuts:
            outs.append(ops.gla_mix(parts[:, at:at + c].contiguous(), heads=H, key_dim=dk, v_dim=dv, w2=w2, b2=None, q_scale=0.5, tau=tau,
                                    records=rec, batch=seq_batch(c, at)))
            at += c
        a = torch.exp(torch.nn.functional.logsigmoid(z.double()) / tau).view(n, H, dk)
        o, S = P.decayed_outer_products(0.5 * q.double().view(n, H, dk), k.double().view(n, H, dk), v.double().view(n, H, dv), a)
        tight(torch.cat(outs), o.reshape(n, H * dv), "float32", f"o, cuts {cuts[:2]}")
        tight(rec[1].view(H, dv, dk), S.transpose(1, 2), "float32", f"the record, cuts {cuts[:2]}")
        assert torch.isnan(rec[0]).all() and torch.isnan(rec[2]).all()
    w = 1 + 0.3 * rnd(g, dv)
    got = ops.gla_norm_gate(torch.cat(outs), parts, 2 * H * dk + H * dv, H, dv, w.to(DEV), 1e-3, torch.float32)
    want = P.norm(o, w.double(), 1e-3).reshape(n, H * dv) * P.silu(gate.double())
    tight(got, want, "float32", "norm and gate")


def test_the_state_remembers_a_token_hundreds_of_positions_back():
    """With decays near one (a logit of 9 under tau = 16) the state keeps what one early token wrote: the result 500
    positions later moves when that token changes, in a prompt, in portions and token by token, as the plain one does."""
    g = torch.Generator().manual_seed(3)
    width, n = 24, 520
    m = gla(2, 6, 10, 16.0, 3)
    part, t = gla_part("float32", width, m, 1e-5, g, decay_logit=9.0)
    h = rnd(g, n, width, std=0.3)
    h2 = h.clone()
    h2[7] = 4 * rnd(g, width)
    ref, ref2 = (P.gated_linear_attention(x.double(), t, "", m, 1e-5) for x in (h, h2))
    assert (ref[515:] - ref2[515:]).abs().max() > 1e-2 * ref.abs().max(), "the early token must show late"
    for cuts in ([n], [8, 400, 112], [500] + [1] * 20):
        tight(run_mixer(part, h, "float32", cuts, gla_view(part)), ref, "float32", f"cuts {cuts[:3]}", tol=1e-4)
        tight(run_mixer(part, h2, "float32", cuts, gla_view(part)), ref2, "float32", f"changed, cuts {cuts[:3]}", tol=1e-4)
    # with strong decays (a logit of -9 under tau = 1) nothing of it is left a few tokens later
    part3, t3 = gla_part("float32", width, gla(2, 6, 10, 1.0, 3), 1e-5, g, decay_logit=-9.0)
    r3, r32 = (P.gated_linear_attention(x.double(), t3, "", gla(2, 6, 10, 1.0, 3), 1e-5) for x in (h[:40], h2[:40]))
    assert (r3[12:] - r32[12:]).abs().max() < 1e-9 * r3.abs().max() and (r3[7] - r32[7]).abs().max() > 1e-3
    tight(run_mixer(part3, h2[:40], "float32", [5, 1, 1, 1, 32], gla_view(part3)), r32, "float32", "strong decays")


def test_the_first_tokens_start_from_zeros_not_from_the_record_of_the_slots_last_user():
    g = torch.Generator().manual_seed(4)
    width = 24
    m = gla(2, 6, 10, 4.0, 3)
    part, t = gla_part("float32", width, m, 1e-5, g)
    h = rnd(g, 9, width)
    ref = P.gated_linear_attention(h.double(), t, "", m, 1e-5)
    view = gla_view(part)
    run_mixer(part, rnd(g, 30, width), "float32", [30], view)          # another sequence leaves its record in slot 1
    assert view.state[1].abs().max() > 0
    for cuts in ([9], [1, 1, 1, 2, 4]):
        view.state[1].zero_()                                 # (what the cache does when a sequence opens in the slot)
        tight(run_mixer(part, h, "float32", cuts, view), ref, "float32", f"cuts {cuts}")
    assert torch.isnan(view.state[2]).all() and torch.isnan(view.state[0]).all(), "another slot's record was written"


@pytest.mark.parametrize("E,top,count,keep", [(6, 3, 3, 2), (8, 2, 4, 1), (16, 4, 4, 2), (9, 1, 9, 9), (10, 2, 1, 1), (6, 2, 0, 0), (64, 6, 8, 3),
                                              (14, 3, 7, 3), (5, 5, 5, 5)])
def test_the_router_chooses_within_the_best_groups_by_corrected_sigmoid_scores(E, top, count, keep):
    g = torch.Generator().manual_seed(E * 7 + top)
    n = 90
    parts = (1.5 * rnd(g, 3, n, E)).to(DEV)
    z = parts.double().sum(0).cpu()
    r = {"experts": E, "top": top, "scale": 2.5}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    # corrections around zero, and strongly negative ones: every choice score is below zero, and a group that is not kept
    # must still lose against them
    for corr in (rnd(g, E, std=0.3), rnd(g, E, std=0.3) - 3.0):
        choice, weight, ident = ops.moe_router(parts, corr.to(DEV), top, renormalize=True, scores="sigmoid", groups=count, keep=keep,
                                               scale=2.5, norm_eps=1e-20)
        want, w = P.choose_experts(z, corr.double(), r)
        order = choice.cpu().long().argsort(-1)
        order_w = want.argsort(-1)
        assert torch.equal(choice.cpu().long().gather(1, order), want.gather(1, order_w)), "the chosen experts"
        assert torch.allclose(weight.cpu().double().gather(1, order), w.gather(1, order_w), rtol=3e-5, atol=1e-7)
        assert torch.allclose(weight.cpu().double().sum(-1), torch.full((n,), 2.5).double(), rtol=1e-5)
        assert torch.equal(ident.cpu(), torch.arange(n, dtype=torch.int32))
    if count and keep < count:
        # the best single expert sits in a group whose two largest add up to less than another group's: it is not chosen
        per = E // count
        s = torch.full((1, E), 0.1)
        s[0, 0] = 0.95
        s[0, per:per + min(2, per)] = 0.7 if per > 1 else 0.97
        parts1 = torch.logit(s)[None].to(DEV)
        choice, _, _ = ops.moe_router(parts1, None, 1, renormalize=True, scores="sigmoid", groups=count, keep=1, scale=1.0, norm_eps=1e-20)
        assert choice.item() == per, choice


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,ff,width,groups,shared", [(6, 3, 40, 64, (3, 2), 20), (3, 1, 52, 72, None, None), (4, 4, 44, 72, (1, 1), 12),
                                                          (9, 2, 16, 48, None, 40), (16, 4, 96, 128, (4, 2), 64), (14, 3, 36, 100, (7, 3), 28)])
def test_one_matrix_experts_with_a_gated_shared_expert(dtype, E, top, ff, width, groups, shared):
    g = torch.Generator().manual_seed(E * 10 + top)
    mlp = moe(ff, E, top, 1.7, groups, shared)
    sh = PartSpec("mlp", {"width": width, "intermediate": shared, "activation": "relu2", "names": {"up": "up", "down": "down"}}) if shared else None
    params = {"width": width, "experts": E, "top": top, "intermediate": ff, "scores": "sigmoid", "correction": True, "renormalize": True,
              "norm_eps": 1e-20, "route_scale": 1.7, "expert": "relu2", "groups": {"count": groups[0], "keep": groups[1]} if groups else None,
              "shared": sh, "shared_gate": sh is not None, "names": MOE_NAMES}
    t = {"router": rnd(g, E, width, std=0.5), "correction": rnd(g, E, std=0.1)}
    for i in range(E):
        t[f"e{i}.up"], t[f"e{i}.down"] = rnd(g, ff, width, std=0.2), rnd(g, width, ff, std=0.2)
    if shared:
        t["shared.up"], t["shared.down"], t["shared.sg"] = rnd(g, shared, width, std=0.2), rnd(g, width, shared, std=0.2), rnd(g, 1, width, std=0.5)
    part, td = make_part("ffn", "routed_moe", params, dtype, t)
    for n in (1, 5, 15, 16, 40, 300):                         # few tokens walk the matrices by expert; from 16 on the rows are sorted
        h = rnd(g, n, width)
        ref = P.expert_ff(as_held(h, dtype), td, "", mlp)
        got = part.forward(h.to(DEV, TORCH[dtype]).contiguous(), seq_batch(n))
        tight(got.sum(0), ref, dtype, f"{n} tokens")
    if shared:
        # a gate far below zero switches the shared expert off; far above, it is added whole
        for sg, f in ((-40.0, 0.0), (40.0, 1.0)):
            h = rnd(g, 20, width).abs()
            t2 = dict(t)
            t2["shared.sg"] = torch.full((1, width), sg)
            part2, td2 = make_part("ffn", "routed_moe", params, dtype, t2)
            hd = as_held(h, dtype)
            ref = P.expert_ff(hd, dict(td2, **{"shared.sg": torch.zeros(1, width).double()}), "", dict(mlp, shared=None)) + f * P.small_ff(hd, td2, "shared.")
            tight(part2.forward(h.to(DEV, TORCH[dtype]).contiguous(), seq_batch(20)).sum(0), ref, dtype, f"gate {sg}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_gated_feed_forward(dtype):
    g = torch.Generator().manual_seed(21)
    for width, ff in ((40, 72), (100, 50), (128, 256)):
        t = {"gate": rnd(g, ff, width, std=0.2), "up": rnd(g, ff, width, std=0.2), "down": rnd(g, width, ff, std=0.2)}
        part, td = make_part("ffn", "gated_mlp", {"width": width, "intermediate": ff, "activation": "silu",
                                                  "names": dict(gate="gate", up="up", down="down")}, dtype, t)
        for n in (1, 7, 130):
            h = rnd(g, n, width)
            got = part.forward(h.to(DEV, TORCH[dtype]).contiguous(), seq_batch(n))
            tight(got.sum(0) if got.dim() == 3 else got, P.dense_ff(as_held(h, dtype), td, ""), dtype, f"width {width}, {n} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_and_linear_attention_side_by_side_add_up_with_their_factors(dtype):
    g = torch.Generator().manual_seed(9)
    width, n = 40, 230
    ml, mr = left(4, 2, 16, 24, 0.3), gla(3, 12, 8, 4.0, 4)
    pl, tl = attention_part(dtype, width, ml, g)
    pr, tr = gla_part(dtype, width, mr, 1e-5, g)
    params = {"width": width, "branches": ({"part": PartSpec("attention", pl.params), "scale": 1.2, "prefix": "left."},
                                           {"part": PartSpec("gated_linear_attention", pr.params), "scale": -0.7, "prefix": "right."})}
    tensors = {**{"left." + k: v.float() for k, v in tl.items()}, **{"right." + k: v.float() for k, v in tr.items()}}
    part, t = make_part("mixer", "parallel", params, dtype, tensors)
    need = part.cache_need()
    assert need.kind == "several" and [p.kind for p in need.parts] == ["paged_kv", "state"]
    h = rnd(g, n, width)
    ref = P.parallel_mixer(as_held(h, dtype), t, "", dict(left=ml, right=mr, left_scale=1.2, right_scale=-0.7), 1e-5)
    for cuts in ([n], [1, 1, 2, 62, 64, 100]):
        view = View(parts=[View(kv=kv_cache(pl, 5, dtype)), gla_view(pr)])
        got = run_mixer(part, h, dtype, cuts, view)
        assert got.shape == (n, width)
        tight(got, ref, dtype, f"cuts {cuts[:3]}")


def test_a_pass_begins_with_the_embedding_output_and_the_vector_of_the_pass():
    g = torch.Generator().manual_seed(10)
    width, n = 36, 11
    steps = rnd(g, 3, width)
    part, _ = make_part("side", "pass_offset", {"width": width, "passes": 3, "add_embedding": True, "tensor": ""}, "float32", {"": steps})
    x, x0 = rnd(g, n, width), rnd(g, n, width)
    for t in range(3):
        h = Hidden(x.clone().to(DEV))
        b = seq_batch(n)
        b.memo["embedding_output"] = x0.to(DEV)
        part.forward(h, b, t)
        want = x + (x0 if t > 0 else 0) + steps[t]
        assert (h.resolved().cpu() - want).abs().max().item() <= 1e-6, t
    with pytest.raises(ValueError):
        part.forward(Hidden(x.clone().to(DEV)), seq_batch(n), 3)


def test_soft_capped_logits():
    z = torch.tensor([[-1000.0, -9.0, -0.5, 0.0, 0.25, 3.0, 50.0, 1e6]])
    for cap in (5.0, 30.0):
        got = ops.soft_cap_(z.clone().to(DEV), cap).cpu()
        assert torch.allclose(got.double(), cap * torch.tanh(z.double() / cap), rtol=1e-5, atol=1e-6) and got.abs().max() <= cap


# ---------------------------------------------------------------------------
# whole models through the engine
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["SA", "SB", "SC", "SD"])
def test_prompt_decoding_and_portions_agree_with_the_plain_model(name, dtype):
    cfg = CONFIGS[name]
    toks = random_tokens(cfg["vocab"], 230, seed=11)
    ref = plain(name, toks, dtype)
    eng = engine(name, dtype)
    s = eng.open_seq()
    close(eng.step([s], [toks], [list(range(len(toks)))]), ref, dtype, "whole prompt")
    eng.close_seq(s)
    # the first tokens one by one, then portions of 2, 3, 61, 64 and 70 tokens, then one by one again
    s = eng.open_seq()
    at, rows = 0, []
    for n in [1] * 7 + [2, 3, 61, 2, 64, 70] + [1] * 13:
        rows.append(eng.step([s], [toks[at:at + n]], [list(range(n))]).clone())
        at += n
    close(torch.cat(rows), ref[:at], dtype, "portions")
    eng.close_seq(s)
    # a prompt long enough for the chunked scan in one step, then its last tokens one by one
    s = eng.open_seq()
    rows = [eng.step([s], [toks[:198]], [list(range(198))]).clone()]
    rows += [eng.step([s], [[t]]).clone() for t in toks[198:]]
    close(torch.cat(rows), ref, dtype, "a long portion, then decoded")
    eng.close_seq(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["SA", "SC", "SD"])
def test_the_stream_after_every_layer_run(name, dtype):
    """The residual stream after each layer run (a looped layer counts each time) against the plain model's."""
    toks = random_tokens(CONFIGS[name]["vocab"], 90, seed=13)
    taps = []
    P.forward(CONFIGS[name], model(name, std=STD_OF[dtype])[1], toks, taps=taps)
    eng = engine(name, dtype, use_graphs=False)
    seen, fwd = [], eng.model.forward
    eng.model.forward = lambda batch, cache: fwd(batch, cache, tap=lambda i, x: seen.append(x.clone().cpu()))
    s = eng.open_seq()
    eng.step([s], [toks])
    assert len(seen) == len(taps) == len(eng.spec.schedule)
    for i, (got, ref) in enumerate(zip(seen, taps)):
        close(got, ref.float(), dtype, f"after layer run {i}", 1e-4 if dtype == "float32" else 4e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_passes_page_borders(dtype):
    name = "SA"
    toks = random_tokens(CONFIGS[name]["vocab"], 200, seed=12)
    ref = plain(name, toks, dtype)
    eng = engine(name, dtype)
    s = eng.open_seq()
    rows = [eng.step([s], [toks[:3]], [[2]]).clone()]
    for p in range(3, len(toks)):
        rows.append(eng.step([s], [[toks[p]]]).clone())
    close(torch.cat(rows), ref[2:], dtype, "decoded")


def test_an_early_token_shows_in_the_logits_hundreds_of_positions_later():
    """Every recurrence's decay is set near one (a2 = 0, a bias of 9), so the states keep the first tokens: changing token 2
    moves the logits at position 600, in the plain model and, by the same amount, in the engine, for a prompt in one step,
    in portions, and decoded."""
    cfg = CONFIGS["SA"]
    d0, w = model("SA")
    w = {k: v.clone() for k, v in w.items()}
    for k in list(w):
        if k.endswith(".a2"):
            w[k] = torch.zeros_like(w[k])
        if k.endswith(".a2.b"):
            w[k] = torch.full_like(w[k], 9.0)
    d = os.path.join(tmp_root(), "suno-SA-remembers")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    from wick_b200.weights.safetensors_io import write_safetensors
    write_safetensors(os.path.join(d, "model.safetensors"), w)
    a = random_tokens(cfg["vocab"], 604, seed=14)
    b = list(a)
    b[2] = (a[2] + 17) % cfg["vocab"]
    ra, rb = P.forward(cfg, w, a).float(), P.forward(cfg, w, b).float()
    assert (ra[600:] - rb[600:]).abs().max() > 3e-2 * ra.abs().max(), "the early token must show late"
    eng = wick.Engine.from_dir(d, dtype="float32", max_tokens=2048)
    for toks, ref in ((a, ra), (b, rb)):
        for cuts in ([604], [3, 2, 395, 200] + [1] * 4, [590] + [1] * 14):
            s = eng.open_seq()
            at, rows = 0, []
            for n in cuts:
                rows.append(eng.step([s], [toks[at:at + n]], [list(range(n))]).clone())
                at += n
            eng.close_seq(s)
            close(torch.cat(rows), ref, "float32", f"cuts {cuts[:3]}", 3e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["SA", "SB", "SD"])
def test_a_batch_of_unequal_requests_equals_each_alone(name, dtype):
    cfg = CONFIGS[name]
    lens = [1, 65, 130, 9, 64]
    prompts = [random_tokens(cfg["vocab"], n + 12, seed=20 + i) for i, n in enumerate(lens)]
    eng = engine(name, dtype, max_tokens=2048)
    alone = []
    for p, n in zip(prompts, lens):
        s = eng.open_seq()
        rows = [eng.step([s], [p[:n]], [list(range(n))]).clone()]
        for t in p[n:]:
            rows.append(eng.step([s], [[t]]).clone())
        alone.append(torch.cat(rows))
        eng.close_seq(s)
        close(alone[-1], plain(name, p, dtype), dtype, f"alone, {n} tokens")
    slots = [eng.open_seq() for _ in prompts]
    got = [[] for _ in prompts]
    first = eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [list(range(n)) for n in lens])
    at = 0
    for i, n in enumerate(lens):
        got[i].append(first[at:at + n].clone())
        at += n
    live = list(range(len(prompts)))
    for step in range(12):
        if step == 5:                                      # two requests end early; the others go on
            for i in (1, 3):
                eng.close_seq(slots[i])
                live.remove(i)
        out = eng.step([slots[i] for i in live], [[prompts[i][lens[i] + step]] for i in live])
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1].clone())
    for i in range(len(prompts)):
        g = torch.cat(got[i])
        close(g, plain(name, prompts[i], dtype)[:g.shape[0]], dtype, f"request {i} in a batch")
        if dtype == "float32":
            assert (g - alone[i][:g.shape[0]]).abs().max().item() <= 3e-5, f"request {i} differs in a batch"


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_of_long_prompts_is_scanned_in_chunks_like_each_alone(dtype):
    name = "SB"
    cfg = CONFIGS[name]
    lens = [250, 64, 193, 3]
    prompts = [random_tokens(cfg["vocab"], n, seed=40 + i) for i, n in enumerate(lens)]
    eng = engine(name, dtype, max_tokens=2048)
    slots = [eng.open_seq() for _ in prompts]
    first = eng.step(slots, prompts, [list(range(n)) for n in lens])
    at = 0
    for i, n in enumerate(lens):
        close(first[at:at + n], plain(name, prompts[i], dtype), dtype, f"request {i}")
        at += n


def poison_free(eng):
    """NaN in every page that no sequence holds and in every record of a slot that no sequence has."""
    held = eng.cache.pages.held()
    free = [p for p in range(1, eng.cache.n_pages) if p not in held]
    live = set(eng.cache.seqs)
    idle = [s for s in range(1, eng.cache.max_seqs + 1) if s not in live]
    for g in eng.cache.groups:
        if g.need.kind in ("paged_kv", "paged_rows") and free:
            g.storage[:, torch.tensor(free, device=g.storage.device)] = float("nan")
        if g.need.kind == "state" and idle:
            g.storage[:, torch.tensor(idle, device=g.storage.device)] = float("nan")


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_slots_and_records_that_were_given_back_are_used_again(dtype):
    name = "SB"
    cfg = CONFIGS[name]
    eng = engine(name, dtype, max_tokens=320)
    a, b = random_tokens(cfg["vocab"], 150, seed=31), random_tokens(cfg["vocab"], 140, seed=32)
    s1 = eng.open_seq()
    eng.step([s1], [a])
    s2 = eng.open_seq()
    eng.step([s2], [b[:70]])
    eng.close_seq(s1)                                      # its three pages, its slot and its records come back
    poison_free(eng)
    s3 = eng.open_seq()
    assert s3 == s1
    out = eng.step([s3], [a[:100]], [list(range(100))])
    assert set(eng.cache.pages_of(s3)) & {1, 2, 3}
    close(out, plain(name, a[:100], dtype), dtype, "in reused pages")
    rows = [eng.step([s2, s3], [[b[70 + i]], [a[100 + i]]]).clone() for i in range(30)]
    close(torch.stack([r[0] for r in rows]), plain(name, b[:100], dtype)[70:], dtype, "the request that stayed")
    close(torch.stack([r[1] for r in rows]), plain(name, a[:130], dtype)[100:], dtype, "the request in reused pages")
    eng.cache.check()


def test_a_request_cannot_go_back_to_an_earlier_position_but_can_start_over():
    eng = engine("SA", "float32")
    toks = random_tokens(CONFIGS["SA"]["vocab"], 40, seed=33)
    s = eng.open_seq()
    first = eng.step([s], [toks]).clone()
    with pytest.raises(ValueError):
        eng.truncate_seq(s, 20)                              # (the recurrences' records hold all 40 tokens)
    eng.truncate_seq(s, 0)
    again = eng.step([s], [toks[:17]], [[]])
    again = eng.step([s], [toks[17:]])
    assert (again - first).abs().max().item() <= 3e-5


@pytest.mark.parametrize("name", ["SA", "SC"])
def test_greedy_generation_through_the_library_entry(name):
    cfg = CONFIGS[name]
    prompts = [random_tokens(cfg["vocab"], n, seed=50 + n) for n in (3, 40, 71)]
    eng = engine(name, "float32")
    out = wick.generate(eng, prompts, wick.GenOptions(max_tokens=24, sampler=wick.SamplerConfig.greedy()))
    for p, r in zip(prompts, out):
        assert len(r.tokens) == 24
        ref = plain(name, list(p) + r.tokens)               # (causal: row i is the prefix's last row)
        for i, t in enumerate(r.tokens):                    # every token is the plain model's best (or ties with it)
            row = ref[len(p) - 1 + i]
            assert row[t] >= row.max() - 1e-3, (name, len(p), i)
    eng_b = engine(name, "bfloat16")
    out_b = wick.generate(eng_b, prompts, wick.GenOptions(max_tokens=8, sampler=wick.SamplerConfig.greedy()))
    for p, r in zip(prompts, out_b):
        assert len(r.tokens) == 8 and all(0 <= t < cfg["vocab"] for t in r.tokens)


def test_the_command_line_writes_runs_and_times_the_design(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root)
    cmd = [sys.executable, os.path.join(root, "bin", "wick")]
    cfg_path, d = str(tmp_path / "cfg.json"), str(tmp_path / "m")
    with open(cfg_path, "w") as f:
        json.dump(CONFIG_SA, f)
    r = subprocess.run(cmd + ["random", d, "--config", cfg_path, "--seed", "4"], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    st = SafeTensorsDir(d)
    w = {n: st.get(n).tensor() for n in st.names()}
    prompts = [[5, 17, 3], [9, 9, 200, 1, 77, 3, 3, 14]]
    r = subprocess.run(cmd + ["run", d, "--ids", "5,17,3", "--ids", "9,9,200,1,77,3,3,14", "-n", "6", "-t", "0", "-q", "f32"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    assert "Sunosun" in r.stderr
    lines = [json.loads(l) for l in r.stdout.strip().splitlines()]
    for p, toks in zip(prompts, lines):
        assert len(toks) == 6
        ref = P.forward(CONFIG_SA, w, p + toks).float()
        for i, t in enumerate(toks):
            row = ref[len(p) - 1 + i]
            assert row[t] >= row.max() - 1e-3, (p, i)
    args = ["run", d, "--ids", "5,17,3", "-n", "12", "-t", "0.9", "--top-k", "20", "--seed", "7", "-q", "bf16"]
    a = subprocess.run(cmd + args, capture_output=True, text=True, env=env, timeout=600)
    b = subprocess.run(cmd + args, capture_output=True, text=True, env=env, timeout=600)
    assert a.returncode == 0 and a.stdout == b.stdout, a.stderr
    assert all(0 <= t < CONFIG_SA["vocab"] for t in json.loads(a.stdout.strip().splitlines()[0]))
    r = subprocess.run(cmd + ["bench", d, "--prompt-len", "16", "-n", "4", "--batch", "2", "-q", "bf16"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "tok/s" in r.stdout, r.stderr


def test_the_trace_runner_serves_the_design():
    name = "SD"
    d = model(name)[0]
    cfg = CONFIGS[name]
    a, b = random_tokens(cfg["vocab"], 70, seed=61), random_tokens(cfg["vocab"], 9, seed=62)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:66], "want": [0, 65]}, {"id": "y", "tokens": b[:5], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[66:67], "want": [0]}, {"id": "y", "tokens": b[5:6], "want": [0]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": a[67:68], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "x", "tokens": a[68:69], "want": [0]}], "end": ["x"]}]
    out = os.path.join(tmp_root(), "suno-trace-out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out,
                        "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    V = cfg["vocab"]
    ra, rb = plain(name, a), plain(name, b)
    read = lambda i: torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, V))
    close(read(0), ra[[0, 65]], "float32", "step 0")
    close(read(1), torch.stack([ra[66], rb[5]]), "float32", "step 1")
    assert not os.path.exists(os.path.join(out, "2.f32"))
    close(read(3), ra[68:69], "float32", "step 3")
