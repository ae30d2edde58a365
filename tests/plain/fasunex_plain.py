"""A plain, slow implementation of the Fasunex decoder, one function per mechanism.

Written from the design's equations in torch on the CPU (float64 by default), it shares
no code with the package: it takes the ``config.json`` dictionary and a dictionary of
tensors by checkpoint name, and runs one whole sequence at once (recurrences token by
token).

Notation: n tokens, width D, positions p from 0; attention: H query heads, G key/value
heads, head size d (queries, keys) and e (values); state-space branch: Hs heads of P
numbers, state size N, Gs groups, K taps.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [n, heads, d]: element i of the first ``dims`` turns with element i + dims/2 by the
    angle p * base^(-2i/dims); the elements from ``dims`` on pass."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a = positions.to(x.dtype) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def visible(n: int, chunk: Optional[int]) -> torch.Tensor:
    """[n, n] bool: query i sees key j iff j <= i and (with ``chunk``) both lie in the same run
    of ``chunk`` positions counted from position 0."""
    p = torch.arange(n)
    vis = p[None, :] <= p[:, None]
    if chunk is not None:
        vis &= (p[None, :] // chunk) == (p[:, None] // chunk)
    return vis


def sink_softmax(scores: torch.Tensor, vis: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """scores [H, n, n], sink [H]: exp(s_j) / (sum over visible j of exp(s_j) + exp(sink))."""
    s = scores.masked_fill(~vis[None], -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def attend(q, k, v, scale, vis, sink):
    """q [n, H, d], k [n, G, d], v [n, G, e] -> [n, H * e]; query head h reads key/value head h // (H / G)."""
    n, H, _ = q.shape
    G = k.shape[1]
    kk = k.repeat_interleave(H // G, dim=1)
    vv = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * scale
    w = sink_softmax(scores, vis, sink)
    return torch.einsum("hij,jhe->ihe", w, vv).reshape(n, -1)


def attention_keys_as_values(h, t: Dict[str, torch.Tensor], pre: str, m: dict, eps: float):
    """The mixer whose values are its keys as projected: no value matrix, no positions in the scores,
    q and k normed per head with a weight, every earlier key visible, a sink, an output gate."""
    n = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ t[pre + "q"].T).view(n, H, d)
    k = (h @ t[pre + "k"].T).view(n, G, d)
    v = k
    q, k = norm(q, t[pre + "q.norm"], eps), norm(k, t[pre + "k.norm"], eps)
    y = attend(q, k, v, m["scale"], visible(n, None), t[pre + "sink"])
    return (y * torch.sigmoid(h @ t[pre + "g"].T)) @ t[pre + "o"].T


def attention_chunked(h, t, pre: str, m: dict, eps: float):
    """The left branch: own values, a rotation of half-split pairs, then a weightless norm of q and k,
    keys of the query's own chunk, a sink, an output gate."""
    n = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(n)
    q = (h @ t[pre + "q"].T).view(n, H, d)
    k = (h @ t[pre + "k"].T).view(n, G, d)
    v = (h @ t[pre + "v"].T).view(n, G, e)
    rot = m.get("rot")
    if rot:
        q, k = rotate_halves(q, pos, rot["dims"], rot["base"]), rotate_halves(k, pos, rot["dims"], rot["base"])
    q, k = rms(q, eps), rms(k, eps)
    chunk = m["mask"]["size"] if m.get("mask") else None
    y = attend(q, k, v, m["scale"], visible(n, chunk), t[pre + "sink"])
    return (y * torch.sigmoid(h @ t[pre + "g"].T)) @ t[pre + "o"].T


def causal_conv(u, w, b):
    """u [n, C], w [C, K] (the last column is the current token's), zeros before the start."""
    n, C = u.shape
    K = w.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], 0)
    out = torch.zeros_like(u)
    for j in range(K):
        out = out + pad[j:j + n] * w[:, j]
    return out + b


def state_space(h, t, pre: str, m: dict, eps: float):
    """The right branch: a selective state-space recurrence per head, gated and normed in groups."""
    n = h.shape[0]
    Hs, P, N, Gs = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hs * P
    proj = h @ t[pre + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * Gs * N], proj[:, 2 * inner + 2 * Gs * N:]
    xbc = silu(causal_conv(xbc, t[pre + "conv"], t[pre + "conv.b"]))
    x = xbc[:, :inner].view(n, Hs, P)
    B = xbc[:, inner:inner + Gs * N].view(n, Gs, N)
    C = xbc[:, inner + Gs * N:].view(n, Gs, N)
    dt = softplus(dt + t[pre + "dt_bias"])
    decay = torch.exp(-torch.exp(t[pre + "A_log"]) * dt)                  # [n, Hs]
    S = torch.zeros(Hs, N, P, dtype=h.dtype)
    y = torch.zeros(n, Hs, P, dtype=h.dtype)
    for i in range(n):
        for hd in range(Hs):
            g = hd // (Hs // Gs)
            S[hd] = decay[i, hd] * S[hd] + dt[i, hd] * torch.outer(B[i, g], x[i, hd])
            y[i, hd] = S[hd].T @ C[i, g] + t[pre + "D"][hd] * x[i, hd]
    y = y.reshape(n, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(n, parts, inner // parts), eps).reshape(n, inner) * t[pre + "norm"]
    return y @ t[pre + "o"].T


def parallel_mixer(h, t, pre: str, m: dict, eps: float):
    return (m["left_scale"] * attention_chunked(h, t, pre + "left.", m["left"], eps)
            + m["right_scale"] * state_space(h, t, pre + "right.", m["right"], eps))


def routed_experts(h, t, pre: str, m: dict):
    """Experts chosen by a router: scores softmax(W h) over experts + identity outputs; the ``top`` largest of
    score + correction are chosen; each weighs its score; the last ``identity`` outputs return h itself."""
    r = m["router"]
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    s = torch.softmax(h @ t[pre + "router"].T, -1)
    choice = s + t[pre + "correction"] if pre + "correction" in t else s
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for ex in torch.topk(choice[i], top).indices.tolist():
            if ex >= E:
                y = h[i]
            else:
                p = f"{pre}e{ex}."
                y = t[p + "down"] @ (silu(t[p + "gate"] @ h[i]) * (t[p + "up"] @ h[i]))
            out[i] = out[i] + s[i, ex] * y
    return out


def layer(x, t, i: int, L: dict, eps: float):
    pre = f"l{i}."
    h = norm(x, t[pre + "norm1"], eps)
    if L["type"] == "attention":
        y = attention_keys_as_values(h, t, pre + "mix.", L["mixer"], eps)
    elif L["type"] == "parallel":
        y = parallel_mixer(h, t, pre + "mix.", L["mixer"], eps)
    else:
        raise ValueError(L["type"])
    x = x + norm(y, t[pre + "norm1b"], eps)
    if L.get("mlp") is not None:
        h = norm(x, t[pre + "norm2"], eps)
        x = x + norm(routed_experts(h, t, pre + "mlp.", L["mlp"]), t[pre + "norm2b"], eps)
    return x


def run_order(cfg: dict) -> List[dict]:
    """The layer runs in order: {"layer": i, "enter": whether the pass input comes before it}."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [{"layer": i, "enter": False} for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [{"layer": i, "enter": False} for i in range(a)]
    for _ in range(times):
        order += [{"layer": i, "enter": i == a} for i in range(a, b)]
    return order + [{"layer": i, "enter": False} for i in range(b, n)]


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, taps: Optional[list] = None):
    """Logits [n, vocab] of one whole sequence; ``taps`` collects the stream after every layer run."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x0 = t["embed"][torch.tensor(tokens)]
    x = x0
    for e in run_order(cfg):
        if e["enter"]:
            x = torch.cat([x, x0], -1) @ t["loop.in"].T
        x = layer(x, t, e["layer"], cfg["layers"][e["layer"]], eps)
        if taps is not None:
            taps.append(x.clone())
    return norm(x, t["final.norm"], eps) @ t["head"].T
