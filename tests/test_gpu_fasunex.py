"""The Fasunex decoder and its mechanisms against the plain implementation in ``tests/plain/fasunex_plain.py``: every
mechanism alone through its part or kernel, then whole models through the engine (prompts, decoding, portions, batches,
reused pages and slots, chunk edges, generation).  The configurations differ from each other in every size and option and
include the values that make mechanisms vanish or coincide (no loop, a loop over one layer, no mask, no rotation, one
key/value head, as many as query heads, one group, no identity outputs, one choice, every output chosen, one tap, no
feed-forward)."""
import copy
import json
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
from wick_b200.parts.base import BuildContext, build_part  # noqa: E402
from wick_b200.parts import attention as _att, parallel as _par, routed as _routed, state_space as _ssm  # noqa: E402,F401
from wick_b200.weights.safetensors_io import SafeTensorsDir  # noqa: E402
from helpers import random_tokens, tmp_root  # noqa: E402
from plain import fasunex_plain as P  # noqa: E402

PAGE = 64
DEV = "cuda"


def att(heads, kv, dim, scale):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale))


def left(heads, kv, dim, vdim, scale, mask=None, rot=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if mask is not None:
        m["mask"] = {"size": mask}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def right(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def par(l, r, ls, rs):
    return dict(type="parallel", mixer=dict(left=l, right=r, left_scale=ls, right_scale=rs))


def moe(ff, experts, identity, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


# FA: a loop over the two middle layers; chunks of 50 and 21 positions; identity outputs; a layer without feed-forward
CONFIG_FA = dict(architecture="Fasunex", vocab=211, width=64, norm={"eps": 1e-5}, loop={"start": 1, "stop": 3, "times": 2}, layers=[
    layer(att(4, 2, 16, 0.3), moe(40, 6, 2, 3)),
    layer(par(left(4, 1, 16, 32, 0.25, mask=50, rot=(8, 1e4)), right(4, 8, 16, 2, 4, 2), 1.2, 0.9), None),
    layer(att(2, 2, 32, 0.2), moe(24, 5, 1, 2)),
    layer(par(left(2, 2, 12, 20, 0.3, mask=21, rot=(12, 5e4)), right(3, 5, 7, 3, 3, 1), 0.8, -1.1), moe(40, 6, 2, 3)),
])
# FB: no loop; a left branch without mask and without rotation; one tap; one choice; every output chosen
CONFIG_FB = dict(architecture="Fasunex", vocab=130, width=72, norm={"eps": 1e-6}, layers=[
    layer(par(left(3, 3, 8, 8, 0.35), right(6, 4, 24, 1, 1, 3), 1.0, 1.0), moe(52, 3, 0, 1)),
    layer(att(6, 1, 10, 0.33), moe(44, 2, 2, 4)),
    layer(par(left(6, 2, 10, 16, 0.3, mask=64, rot=(4, 1e3)), right(2, 20, 40, 2, 2, 1), 0.5, 2.0), moe(16, 9, 3, 2)),
])
# FC: heads of 64 and 128 numbers (the tensor-core attention), a state of 128, a loop over the first layer alone
CONFIG_FC = dict(architecture="Fasunex", vocab=300, width=128, norm={"eps": 1e-5}, loop={"start": 0, "stop": 1, "times": 3}, layers=[
    layer(par(left(2, 1, 64, 64, 0.125, mask=70, rot=(32, 1e4)), right(2, 64, 128, 1, 4, 2), 1.1, 1.2), moe(64, 8, 2, 2)),
    layer(att(2, 1, 128, 0.09), moe(128, 4, 0, 2)),
    layer(att(4, 2, 64, 0.125), None),
])
# FD: a width that is no multiple of eight, heads of 40, 24, 8 and 6 numbers, five groups, seven taps, a chunk longer than the
# prompts, a loop of three passes over one layer
CONFIG_FD = dict(architecture="Fasunex", vocab=77, width=100, norm={"eps": 1e-6}, loop={"start": 1, "stop": 2, "times": 3}, layers=[
    layer(att(3, 1, 40, 0.2), moe(36, 4, 1, 2)),
    layer(par(left(5, 1, 24, 8, 0.2, mask=33, rot=(6, 1e4)), right(5, 12, 20, 5, 2, 1), 0.7, 1.3), moe(50, 7, 0, 3)),
    layer(par(left(2, 2, 6, 6, 0.4, mask=300), right(1, 36, 9, 1, 7, 4), 1.0, 1.0), None),
])
CONFIGS = {"FA": CONFIG_FA, "FB": CONFIG_FB, "FC": CONFIG_FC, "FD": CONFIG_FD}
_models = {}
STD = 0.15


def write_model(cfg, d, seed=5, std=STD):
    wick.write_random_model(wick.config_from_json(cfg), seed, d, std=std)
    st = SafeTensorsDir(d)
    return {n: st.get(n).tensor() for n in st.names()}


def model(name, seed=5, std=STD):
    key = (name, seed, std)
    if key not in _models:
        d = os.path.join(tmp_root(), f"fas-{name}-{seed}-{std}")
        _models[key] = (d, write_model(CONFIGS[name], d, seed, std))
    return _models[key]


def engine(name, dtype, max_tokens=1024, **kw):
    return wick.Engine.from_dir(model(name)[0], dtype=dtype, max_tokens=max_tokens, **kw)


_plain = {}


def plain(name, tokens):
    key = (name, tuple(tokens))
    if key not in _plain:
        _plain[key] = P.forward(CONFIGS[name], model(name)[1], list(tokens)).float()
    return _plain[key]


def close(got, ref, dtype, what="", tol=None):
    """float32: every row within ``tol`` of the scale.  bfloat16: with random weights a router's close call may choose another
    expert than the plain model's, which replaces a whole expert's output at that row (and, through the caches, moves later
    rows a little), so the median row must be within ``tol``, nine rows in ten within twice that, and at most one row in
    twenty further than a third of the scale away; float32 is the sharp comparison."""
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = max(1.0, ref.abs().max().item())
    rows = (got - ref).abs().reshape(got.shape[0], -1).max(-1).values / scale
    f32 = dtype in ("float32", torch.float32)
    tol = tol or (2e-4 if f32 else 5e-2)
    if f32:
        if rows.max().item() > tol:
            raise AssertionError(f"{what}: differs by {rows.max().item():.3e} of the scale {scale:.3g}, worst row {int(rows.argmax())}")
        return
    med, q90, worst = rows.median().item(), rows.quantile(0.9).item(), rows.max().item()
    far = int((rows > 0.34).sum())
    if med > tol or q90 > 2 * tol or far > max(1, rows.numel() // 20):
        raise AssertionError(f"{what}: median {med:.3e}, nine in ten within {q90:.3e}, worst {worst:.3e} (row {int(rows.argmax())}) "
                             f"of the scale {scale:.3g}")


def tight(got, ref, dtype, what=""):
    """For one mechanism alone, with the same choices on both sides: every row within the dtype's rounding."""
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = max(1e-6, ref.abs().max().item())
    worst = (got - ref).abs().max().item() / scale
    tol = 3e-5 if dtype in ("float32", torch.float32) else 2.5e-2
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
        assert tuple(tensors[n].shape) == tuple(s.shape), (n, tuple(tensors[n].shape), s.shape)
    held = {n: (t.to(TORCH[dtype]) if specs[n].role == "matrix" else t.float()) for n, t in tensors.items()}
    part.load(lambda n: held[n])
    return part, {n: t.double() for n, t in held.items()}


def rnd(g, *shape, std=1.0):
    return torch.randn(*shape, generator=g) * std


MIX_NAMES = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", sink="sink", gate="g")
SSM_NAMES = dict(input="in", conv="conv", conv_bias="conv.b", dt_bias="dt_bias", a_log="A_log", d="D", norm="norm", o="o")
MOE_NAMES = dict(gate="gate", up="up", down="down", expert="e{i}.", router="router", correction="correction")


def attention_part(dtype, width, m, eps, keys_are_values, g, std=0.3):
    """The attention part as the design uses it and random tensors for it."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    params = {"width": width, "heads": H, "kv_heads": G, "head_dim": d, "v_dim": e, "scale": m["scale"], "qk_norm": "head",
              "qk_norm_weight": keys_are_values, "qk_norm_after_rotation": not keys_are_values, "eps": eps,
              "position": PartSpec("rotary_pairs", {"head_dim": d, "dims": rot["dims"], "theta": rot["base"], "pairing": "halves"}) if rot else None,
              "values": "keys" if keys_are_values else "own",
              "mask": {"kind": "block", "size": m["mask"]["size"]} if m.get("mask") else None, "sink": True, "gate": True, "names": MIX_NAMES}
    t = {"q": rnd(g, H * d, width, std=std), "k": rnd(g, G * d, width, std=std), "g": rnd(g, H * e, width, std=std),
         "o": rnd(g, width, H * e, std=std), "sink": rnd(g, H)}
    if keys_are_values:
        t["q.norm"], t["k.norm"] = 1 + 0.3 * rnd(g, d), 1 + 0.3 * rnd(g, d)
    else:
        t["v"] = rnd(g, G * e, width, std=std)
    return make_part("mixer", "attention", params, dtype, t)


def kv_cache(part, n_pages, dtype):
    need = part.cache_need()
    e = need.head_dim if need.v_head_dim is None else need.v_head_dim
    if e != need.head_dim:
        return torch.zeros((n_pages, need.kv_heads * PAGE * (need.head_dim + e)), dtype=TORCH[dtype], device=DEV)
    return torch.zeros((n_pages, 2, need.kv_heads, PAGE, need.head_dim), dtype=TORCH[dtype], device=DEV)


class View:
    def __init__(self, **kw):
        self.__dict__.update(kw)


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
def test_a_normed_sublayer_result_joins_the_stream_and_the_sum_is_normed_in_one_kernel():
    """x <- x + rms(sum of the partial sums) * wb, then rms(x) * w in the activation type: widths that are and are not
    multiples of four, every row or selected rows (one named twice), the sum's norm and the stream's norm with eps of
    their own."""
    g = torch.Generator().manual_seed(4)

    def rms(v, eps):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)

    for width, rows in ((40, 7), (101, 9), (258, 5), (2052, 33)):
        x, d = 2 * torch.randn(rows, width, generator=g), torch.randn(3, rows, width, generator=g)
        wb, w = 1 + 0.2 * torch.randn(width, generator=g), 1 + 0.3 * torch.randn(width, generator=g)
        X = x.double() + rms(d.double().sum(0), 1e-5) * wb.double()
        ref = rms(X, 3e-4) * w.double()
        for dtype in DTYPES:
            xd = x.to(DEV)
            out = ops.stream_update(xd, d.to(DEV), rms=(wb.to(DEV), 1e-5), norm=("rms", w.to(DEV), 3e-4), out_dtype=TORCH[dtype])
            tight(xd, X, "float32", f"the stream, width {width}")
            tight(out, ref, dtype, f"its norm, width {width}")
            xd = x.to(DEV)
            idx = torch.tensor([rows - 1, 0, rows - 1], dtype=torch.int32)
            out = ops.stream_update(xd, d.to(DEV), rms=(wb.to(DEV), 1e-5), norm=("rms", w.to(DEV), 3e-4), out_dtype=TORCH[dtype],
                                    rows=idx.to(DEV))
            tight(out, ref[idx.long()], dtype, f"selected rows, width {width}")
            assert torch.equal(xd.cpu(), x)
        # the norm alone, nothing added
        xd = x.to(DEV)
        out = ops.stream_update(xd, None, norm=("rms", w.to(DEV), 3e-4), out_dtype=torch.float32)
        tight(out, rms(x.double(), 3e-4) * w.double(), "float32", f"the norm alone, width {width}")
        assert torch.equal(xd.cpu(), x)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,scale", [(4, 2, 16, 0.3), (6, 1, 10, 0.33), (2, 2, 64, 0.125), (3, 3, 48, 0.2), (2, 1, 128, 0.09)])
def test_attention_whose_keys_are_its_values(dtype, H, G, d, scale):
    g = torch.Generator().manual_seed(H * 100 + d)
    width, n = 40, 150
    m = dict(heads=H, kv_heads=G, dim=d, vdim=d, scale=scale)
    part, t = attention_part(dtype, width, m, 1e-5, True, g)
    h = rnd(g, n, width)
    ref = P.attention_keys_as_values(as_held(h, dtype), t, "", m, 1e-5)
    for cuts in ([n], [1] * 5 + [2, 3, 59, 64, 17]):
        got = run_mixer(part, h, dtype, cuts, View(kv=kv_cache(part, 4, dtype)))
        tight(got, ref, dtype, f"cuts {cuts[:3]}")
    # the values are the keys BEFORE the norm: with norm weights far from one the two differ
    assert (t["k.norm"] - 1).abs().max() > 0.1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,e,mask,rot", [(4, 1, 16, 32, 50, (8, 1e4)), (2, 2, 12, 20, 21, (12, 5e4)), (3, 3, 8, 8, None, None),
                                              (2, 1, 64, 64, 70, (32, 1e4)), (4, 2, 128, 128, 64, (128, 1e6)), (2, 2, 32, 16, 1, (2, 10.0))])
def test_chunked_attention_with_a_rotation_before_the_norm(dtype, H, G, d, e, mask, rot):
    g = torch.Generator().manual_seed(H * 100 + d + e)
    width, n = 48, 200
    m = left(H, G, d, e, 0.3 if d < 64 else 0.1, mask, rot)
    part, t = attention_part(dtype, width, m, 1e-6, False, g)
    h = rnd(g, n, width)
    ref = P.attention_chunked(as_held(h, dtype), t, "", m, 1e-6)
    for cuts in ([n], [1] * 4 + [2, 60, 5, 64, 65]):
        got = run_mixer(part, h, dtype, cuts, View(kv=kv_cache(part, 5, dtype)))
        tight(got, ref, dtype, f"cuts {cuts[:3]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_that_stands_out_far_back_at_page_borders_and_at_the_chunks_edges(dtype):
    """With Wk = Wq and inputs at two positions i and j that differ only by a vector that Wq maps to zero, the score of (i, j)
    is the largest there can be (d * scale after the weightless norm), as is that of (i, i): the result at i is the mean of v_i
    and v_j if j is visible and v_i if not.  The rows in question are checked against the plain function in a prompt and
    when decoded alone."""
    g = torch.Generator().manual_seed(77)
    width, H, d, chunk, n = 48, 2, 16, 200, 640
    m = left(H, H, d, d, 1.5, chunk, None)
    part, t = attention_part(dtype, width, m, 1e-6, False, g, std=0.5)
    wq = t["q"].clone()
    part2, t = make_part("mixer", "attention", part.params, dtype, {**{k: v.float() for k, v in t.items()}, "k": wq.float()})
    h = rnd(g, n, width)
    pairs = [(599, 400), (598, 399), (450, 401), (639, 600), (601, 597), (199, 0), (200, 198), (511, 448), (512, 447), (383, 320), (384, 201)]
    null = torch.linalg.svd(t["q"])[2][H * d:].T.float()       # [width, width - H d]: what the q (and k) matrix maps to zero
    for i, j in pairs:
        h[i] = rnd(g, width)
        h[j] = h[i] + null @ rnd(g, null.shape[1], std=3.0)
    ref = P.attention_chunked(as_held(h, dtype), t, "", m, 1e-6)
    for i, j in pairs:                                        # the pair's score: d * scale = 24, against scores around zero
        q = P.rms((as_held(h, dtype)[i] @ t["q"].T).view(H, d), 1e-6)
        assert (q * q).sum(-1).min() * 1.5 > 20, "the pair's score does not stand out"
    got = run_mixer(part2, h, dtype, [n], View(kv=kv_cache(part2, 11, dtype)))
    tight(got, ref, dtype, "whole prompt")
    # decoded: every i of the pairs alone, after a prompt that ends right before it
    for i, j in pairs[:7]:
        view = View(kv=kv_cache(part2, 11, dtype))
        got = run_mixer(part2, h[:i + 1], dtype, [i, 1], view)
        tight(got[i:], ref[i:i + 1], dtype, f"position {i} decoded, its twin at {j}")
    # the visible twin matters (without it the row is another one), the hidden one does not
    h2 = h.clone()
    for i, j in pairs:
        h2[j] = rnd(g, width)
    ref2 = P.attention_chunked(as_held(h2, dtype), t, "", m, 1e-6)
    for i, j in pairs:
        moved = (ref2[i] - ref[i]).abs().max() > 1e-2 * ref.abs().max()
        if i // chunk == j // chunk:
            assert moved, (i, j)
    assert not (ref2[200] - ref[200]).abs().max() > 1e-2 * ref.abs().max()      # (200, 198): its twin lies in the chunk before
    got2 = run_mixer(part2, h2, dtype, [300, 340], View(kv=kv_cache(part2, 11, dtype)))
    tight(got2, ref2, dtype, "without the twins")


def ssm_part(dtype, width, m, eps, g, std=0.3, a_log=None, dt_bias=None):
    Hs, Pn, N, Gs, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner, ch = Hs * Pn, Hs * Pn + 2 * Gs * N
    params = {"width": width, "heads": Hs, "head_dim": Pn, "state": N, "groups": Gs, "taps": K, "norm_groups": m["norm_groups"],
              "eps": eps, "names": SSM_NAMES}
    t = {"in": rnd(g, 2 * inner + 2 * Gs * N + Hs, width, std=std), "conv": rnd(g, ch, K, std=0.5), "conv.b": rnd(g, ch, std=0.2),
         "dt_bias": rnd(g, Hs, std=0.5) if dt_bias is None else torch.full((Hs,), float(dt_bias)),
         "A_log": rnd(g, Hs, std=0.5) if a_log is None else torch.full((Hs,), float(a_log)), "D": rnd(g, Hs),
         "norm": 1 + 0.3 * rnd(g, inner), "o": rnd(g, width, inner, std=std)}
    return make_part("mixer", "selective_state_space", params, dtype, t)


def records(part, slots=3):
    return torch.full((slots, part.record_floats()), float("nan"), device=DEV)


def ssm_view(part):
    rec = records(part)
    rec[1].zero_()                                            # (what the cache does when a sequence opens in slot 1)
    return View(state=rec, slots=None)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hs,Pn,N,Gs,K,ng", [(4, 8, 16, 2, 4, 2), (3, 5, 7, 3, 3, 1), (6, 4, 24, 1, 1, 3), (2, 64, 128, 1, 4, 2),
                                             (2, 20, 40, 2, 2, 1), (1, 32, 300, 1, 5, 4)])
def test_the_state_space_recurrence_in_any_portions(dtype, Hs, Pn, N, Gs, K, ng):
    g = torch.Generator().manual_seed(Hs * 1000 + N)
    width, n = 40, 350                                       # (a step of 192 tokens or more is scanned in chunks of 64)
    m = right(Hs, Pn, N, Gs, K, ng)
    part, t = ssm_part(dtype, width, m, 1e-5, g)
    h = rnd(g, n, width)
    ref = P.state_space(as_held(h, dtype), t, "", m, 1e-5)
    for cuts in ([n], [1] * 6 + [2, 3, 2, 59, 64, 1, 1, 12, 200], [349, 1], [75, 75, 8, 192], [192, 158]):
        got = run_mixer(part, h, dtype, cuts, ssm_view(part))
        tight(got, ref, dtype, f"cuts {cuts[:3]}")


def test_the_state_remembers_a_token_hundreds_of_positions_back():
    """With a decay near one (A = -exp(-9), dt around 0.7) the state keeps what one early token wrote: the result 500
    positions later moves when that token changes, in a prompt, in portions and token by token, as the plain one does."""
    g = torch.Generator().manual_seed(3)
    width, n = 24, 520
    m = right(2, 6, 10, 1, 3, 1)
    part, t = ssm_part("float32", width, m, 1e-5, g, a_log=-9.0, dt_bias=0.0)
    h = rnd(g, n, width, std=0.3)
    h2 = h.clone()
    h2[7] = 4 * rnd(g, width)
    ref, ref2 = (P.state_space(x.double(), t, "", m, 1e-5) for x in (h, h2))
    assert (ref[515:] - ref2[515:]).abs().max() > 1e-2 * ref.abs().max(), "the early token must show late"
    for cuts in ([n], [8, 400, 112], [500] + [1] * 20):
        tight(run_mixer(part, h, "float32", cuts, ssm_view(part)), ref, "float32", f"cuts {cuts[:3]}")
        tight(run_mixer(part, h2, "float32", cuts, ssm_view(part)), ref2, "float32", f"changed, cuts {cuts[:3]}")


def test_the_first_tokens_see_zeros_before_the_start_not_the_record_of_the_slots_last_user():
    g = torch.Generator().manual_seed(4)
    width = 24
    m = right(2, 6, 10, 2, 4, 2)
    part, t = ssm_part("float32", width, m, 1e-5, g)
    h = rnd(g, 9, width)
    ref = P.state_space(h.double(), t, "", m, 1e-5)
    view = ssm_view(part)
    run_mixer(part, rnd(g, 30, width), "float32", [30], view)          # another sequence leaves its record in slot 1
    view.state[1].zero_()                                     # the slot is opened again
    for cuts in ([9], [1, 1, 1, 2, 4]):
        view.state[1].zero_()
        tight(run_mixer(part, h, "float32", cuts, view), ref, "float32", f"cuts {cuts}")
    assert torch.isnan(view.state[2]).all(), "another slot's record was written"


@pytest.mark.parametrize("n_out,top,identity", [(7, 3, 2), (3, 1, 0), (4, 4, 2), (20, 4, 4), (130, 6, 10), (2, 2, 1)])
def test_the_router_chooses_by_corrected_scores_and_weighs_by_plain_ones(n_out, top, identity):
    g = torch.Generator().manual_seed(n_out)
    n = 70
    parts = rnd(g, 3, n, n_out).to(DEV)
    corr = rnd(g, n_out, std=0.2).to(DEV)
    z = parts.double().sum(0).cpu()
    s = torch.softmax(z, -1)
    for c, renorm in ((corr, False), (None, False), (corr, True)):
        choice, weight, ident = ops.moe_router(parts, c, top, renormalize=renorm)
        pick = s + (c.double().cpu() if c is not None else 0)
        want = torch.topk(pick, top, dim=-1).indices
        assert torch.equal(choice.cpu().long(), want), "choices (in the order of their corrected scores)"
        w = torch.gather(s, 1, want)
        if renorm:
            w = w / w.sum(-1, keepdim=True)
        assert torch.allclose(weight.cpu().double(), w, rtol=2e-5, atol=1e-7)
        assert torch.equal(ident.cpu(), torch.arange(n, dtype=torch.int32))
    # equal scores: the lowest index first
    same = torch.zeros(1, 5, n_out, device=DEV)
    choice, weight, _ = ops.moe_router(same, None, top)
    assert choice.cpu().tolist() == [list(range(top))] * 5 and torch.allclose(weight.cpu(), torch.full((5, top), 1.0 / n_out))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,I,top,ff,width", [(6, 2, 3, 40, 64), (3, 0, 1, 52, 72), (2, 2, 4, 44, 72), (9, 3, 2, 16, 48), (16, 4, 4, 96, 128)])
def test_routed_experts_with_identity_outputs(dtype, E, I, top, ff, width):
    g = torch.Generator().manual_seed(E * 10 + top)
    params = {"width": width, "experts": E, "identity": I, "top": top, "intermediate": ff, "scores": "softmax", "correction": True,
              "renormalize": False, "names": MOE_NAMES}
    t = {"router": rnd(g, E + I, width, std=0.5), "correction": rnd(g, E + I, std=0.1)}
    for i in range(E):
        t[f"e{i}.gate"], t[f"e{i}.up"], t[f"e{i}.down"] = rnd(g, ff, width, std=0.2), rnd(g, ff, width, std=0.2), rnd(g, width, ff, std=0.2)
    part, td = make_part("ffn", "routed_moe", params, dtype, t)
    m = {"router": {"experts": E, "identity": I, "top": top}}
    for n in (1, 5, 15, 16, 40, 300):                         # few tokens walk the matrices by expert; from 16 on the rows are sorted
        h = rnd(g, n, width)
        ref = P.routed_experts(as_held(h, dtype), td, "", m)
        got = part.forward(h.to(DEV, TORCH[dtype]).contiguous(), seq_batch(n))
        tight(got.sum(0), ref, dtype, f"{n} tokens")
    if I:
        # a router that always prefers the identity outputs: the result is the input times their scores
        t2 = dict(t, correction=torch.cat([torch.full((E,), -5.0), torch.full((I,), 5.0)]))
        part2, td2 = make_part("ffn", "routed_moe", dict(params, top=I), dtype, t2)
        h = rnd(g, 20, width)
        hd = as_held(h, dtype)
        s = torch.softmax(hd @ td2["router"].T, -1)[:, E:].sum(-1, keepdim=True)
        got = part2.forward(h.to(DEV, TORCH[dtype]).contiguous(), seq_batch(20))
        tight(got.sum(0), s * hd, dtype, "identity outputs alone")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixers_side_by_side_add_up_with_their_factors(dtype):
    g = torch.Generator().manual_seed(9)
    width, n = 40, 130
    ml, mr = left(4, 2, 16, 16, 0.3, 50, (8, 1e4)), right(3, 8, 12, 3, 4, 1)
    pl, tl = attention_part(dtype, width, ml, 1e-5, False, g)
    pr, tr = ssm_part(dtype, width, mr, 1e-5, g)
    params = {"width": width, "branches": ({"part": PartSpec("attention", pl.params), "scale": 1.2, "prefix": "left."},
                                           {"part": PartSpec("selective_state_space", pr.params), "scale": -0.7, "prefix": "right."})}
    tensors = {**{"left." + k: v.float() for k, v in tl.items()}, **{"right." + k: v.float() for k, v in tr.items()}}
    part, t = make_part("mixer", "parallel", params, dtype, tensors)
    need = part.cache_need()
    assert need.kind == "several" and [p.kind for p in need.parts] == ["paged_kv", "state"]
    h = rnd(g, n, width)
    ref = P.parallel_mixer(as_held(h, dtype), t, "", dict(left=ml, right=mr, left_scale=1.2, right_scale=-0.7), 1e-5)
    for cuts in ([n], [1, 1, 2, 62, 64]):
        view = View(parts=[View(kv=kv_cache(pl, 4, dtype)), ssm_view(pr)])
        got = run_mixer(part, h, dtype, cuts, view)
        assert got.shape == (n, width)
        tight(got, ref, dtype, f"cuts {cuts[:3]}")


# ---------------------------------------------------------------------------
# whole models through the engine
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["FA", "FB", "FC", "FD"])
def test_prompt_decoding_and_portions_agree_with_the_plain_model(name, dtype):
    cfg = CONFIGS[name]
    toks = random_tokens(cfg["vocab"], 230, seed=11)
    ref = plain(name, toks)
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
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["FA", "FC"])
def test_the_stream_after_every_layer_run(name, dtype):
    """The residual stream after each layer run (a looped layer counts each time) against the plain model's."""
    toks = random_tokens(CONFIGS[name]["vocab"], 90, seed=13)
    taps = []
    P.forward(CONFIGS[name], model(name)[1], toks, taps=taps)
    eng = engine(name, dtype, use_graphs=False)
    seen, fwd = [], eng.model.forward
    eng.model.forward = lambda batch, cache: fwd(batch, cache, tap=lambda i, x: seen.append(x.clone().cpu()))
    s = eng.open_seq()
    eng.step([s], [toks])
    assert len(seen) == len(taps) == len(eng.spec.schedule)
    for i, (got, ref) in enumerate(zip(seen, taps)):
        close(got, ref.float(), dtype, f"after layer run {i}", 1e-4 if dtype == "float32" else 4e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_passes_chunk_edges_and_page_borders(dtype):
    name = "FA"                                              # chunks of 50 and 21 positions, pages of 64
    toks = random_tokens(CONFIGS[name]["vocab"], 200, seed=12)
    ref = plain(name, toks)
    eng = engine(name, dtype)
    s = eng.open_seq()
    rows = [eng.step([s], [toks[:3]], [[2]]).clone()]
    for p in range(3, len(toks)):
        rows.append(eng.step([s], [[toks[p]]]).clone())
    close(torch.cat(rows), ref[2:], dtype, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["FA", "FB", "FD"])
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
        close(alone[-1], plain(name, p), dtype, f"alone, {n} tokens")
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
        close(g, plain(name, prompts[i])[:g.shape[0]], dtype, f"request {i} in a batch")
        if dtype == "float32":
            assert (g - alone[i][:g.shape[0]]).abs().max().item() <= 3e-5, f"request {i} differs in a batch"


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
    name = "FB"
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
    close(out, plain(name, a[:100]), dtype, "in reused pages")
    rows = [eng.step([s2, s3], [[b[70 + i]], [a[100 + i]]]).clone() for i in range(30)]
    close(torch.stack([r[0] for r in rows]), plain(name, b[:100])[70:], dtype, "the request that stayed")
    close(torch.stack([r[1] for r in rows]), plain(name, a[:130])[100:], dtype, "the request in reused pages")
    eng.cache.check()


def test_a_request_cannot_go_back_to_an_earlier_position_but_can_start_over():
    eng = engine("FA", "float32")
    toks = random_tokens(CONFIGS["FA"]["vocab"], 40, seed=33)
    s = eng.open_seq()
    first = eng.step([s], [toks]).clone()
    with pytest.raises(ValueError):
        eng.truncate_seq(s, 20)                              # (the recurrence's record holds all 40 tokens)
    eng.truncate_seq(s, 0)
    again = eng.step([s], [toks[:17]], [[]])
    again = eng.step([s], [toks[17:]])
    assert (again - first).abs().max().item() <= 3e-5


@pytest.mark.parametrize("name", ["FA", "FC"])
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
        json.dump(CONFIG_FA, f)
    r = subprocess.run(cmd + ["random", d, "--config", cfg_path, "--seed", "4"], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    st = SafeTensorsDir(d)
    w = {n: st.get(n).tensor() for n in st.names()}
    prompts = [[5, 17, 3], [9, 9, 200, 1, 77, 3, 3, 14]]
    r = subprocess.run(cmd + ["run", d, "--ids", "5,17,3", "--ids", "9,9,200,1,77,3,3,14", "-n", "6", "-t", "0", "-q", "f32"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    assert "Fasunex" in r.stderr
    lines = [json.loads(l) for l in r.stdout.strip().splitlines()]
    for p, toks in zip(prompts, lines):
        assert len(toks) == 6
        ref = P.forward(CONFIG_FA, w, p + toks).float()
        for i, t in enumerate(toks):
            row = ref[len(p) - 1 + i]
            assert row[t] >= row.max() - 1e-3, (p, i)
    args = ["run", d, "--ids", "5,17,3", "-n", "12", "-t", "0.9", "--top-k", "20", "--seed", "7", "-q", "bf16"]
    a = subprocess.run(cmd + args, capture_output=True, text=True, env=env, timeout=600)
    b = subprocess.run(cmd + args, capture_output=True, text=True, env=env, timeout=600)
    assert a.returncode == 0 and a.stdout == b.stdout, a.stderr
    assert all(0 <= t < CONFIG_FA["vocab"] for t in json.loads(a.stdout.strip().splitlines()[0]))
    r = subprocess.run(cmd + ["bench", d, "--prompt-len", "16", "-n", "4", "--batch", "2", "-q", "bf16"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "tok/s" in r.stdout, r.stderr


def test_the_trace_runner_serves_the_design():
    name = "FA"
    d = model(name)[0]
    cfg = CONFIGS[name]
    a, b = random_tokens(cfg["vocab"], 70, seed=61), random_tokens(cfg["vocab"], 9, seed=62)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:66], "want": [0, 65]}, {"id": "y", "tokens": b[:5], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[66:67], "want": [0]}, {"id": "y", "tokens": b[5:6], "want": [0]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": a[67:68], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "x", "tokens": a[68:69], "want": [0]}], "end": ["x"]}]
    out = os.path.join(tmp_root(), "fas-trace-out")
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
