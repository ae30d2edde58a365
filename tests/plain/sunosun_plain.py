"""A plain, slow implementation of the Sunosun decoder, one function per mechanism.

Written from the design's equations in torch on the CPU (float64 by default), it shares
no code with the package: it takes the ``config.json`` dictionary and a dictionary of
tensors by checkpoint name, and runs one whole sequence at once (the recurrence token by
token).

Notation: n tokens, width D, positions p from 0; attention: H query heads, G key/value
heads, head size d (queries, keys) and e (values); linear attention: Hr heads with keys of
dk and values of dv numbers, a decay per key channel; experts: E experts in groups of
neighbours, ``top`` chosen.
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


def relu2(z):
    return torch.relu(z) ** 2


def position_vectors(n: int, width: int, dtype, first: int = 0, base: float = 10000.0) -> torch.Tensor:
    """[n, width]: entry 2i of position p is sin(p base^(-2i/width)), entry 2i+1 the cosine of the same angle."""
    out = torch.zeros((n, width), dtype=dtype)
    p = torch.arange(first, first + n, dtype=dtype)
    for i in range((width + 1) // 2):
        a = p * (base ** (-2.0 * i / width))
        out[:, 2 * i] = torch.sin(a)
        if 2 * i + 1 < width:
            out[:, 2 * i + 1] = torch.cos(a)
    return out


def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    """Rows of the table times ``scale`` plus the positions' vectors."""
    x = table[tokens] * scale
    return x + position_vectors(len(tokens), table.shape[1], x.dtype)


def one_more_softmax(scores: torch.Tensor, vis: torch.Tensor) -> torch.Tensor:
    """scores [H, n, n]: exp(s_j) / (1 + sum over visible j of exp(s_j)): a further key of score 0 without a value."""
    s = scores.masked_fill(~vis[None], -math.inf)
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(-m))


def softmax_attention(h, t: Dict[str, torch.Tensor], pre: str, m: dict) -> torch.Tensor:
    """Causal attention with biased projections, no positions, grouped key/value heads and the further key of score 0."""
    n = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[pre + "q"].T + t[pre + "q.b"]).reshape(n, H, d)
    k = (h @ t[pre + "k"].T + t[pre + "k.b"]).reshape(n, G, d)
    v = (h @ t[pre + "v"].T + t[pre + "v.b"]).reshape(n, G, e)
    kk = k.repeat_interleave(H // G, dim=1)
    vv = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    p = torch.arange(n)
    w = one_more_softmax(scores, p[None, :] <= p[:, None])
    return torch.einsum("hij,jhe->ihe", w, vv).reshape(n, H * e) @ t[pre + "o"].T


def decays(h, t, pre: str, m: dict) -> torch.Tensor:
    """[n, Hr, dk]: sigmoid(W2 (W1 h) + b) ^ (1 / tau), a number in (0, 1) per key channel."""
    z = (h @ t[pre + "a1"].T) @ t[pre + "a2"].T + t[pre + "a2.b"]
    return torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).reshape(h.shape[0], m["heads"], m["dim"])


def decayed_outer_products(q, k, v, a, state: Optional[torch.Tensor] = None):
    """q, k, a [n, Hr, dk], v [n, Hr, dv]; token by token S <- a_t (rows) * S + k_t v_t^T and o_t = S^T q_t.
    Returns (o [n, Hr, dv], the last S [Hr, dk, dv])."""
    n, Hr, dk = q.shape
    S = torch.zeros((Hr, dk, v.shape[2]), dtype=q.dtype) if state is None else state.clone()
    out = []
    for i in range(n):
        S = a[i][:, :, None] * S + k[i][:, :, None] * v[i][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[i]))
    return torch.stack(out), S


def gated_linear_attention(h, t, pre: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    Hr, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ t[pre + "q"].T).reshape(n, Hr, dk) * dk ** -0.5
    k = (h @ t[pre + "k"].T).reshape(n, Hr, dk)
    v = (h @ t[pre + "v"].T).reshape(n, Hr, dv)
    o, _ = decayed_outer_products(q, k, v, decays(h, t, pre, m))
    o = norm(o, t[pre + "norm"], eps).reshape(n, Hr * dv)
    return (o * silu(h @ t[pre + "g"].T)) @ t[pre + "o"].T


def parallel_mixer(h, t, pre: str, m: dict, eps: float) -> torch.Tensor:
    left = softmax_attention(h, t, pre + "left.", m["left"])
    right = gated_linear_attention(h, t, pre + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def dense_ff(h, t, pre: str) -> torch.Tensor:
    return (silu(h @ t[pre + "gate"].T) * (h @ t[pre + "up"].T)) @ t[pre + "down"].T


def small_ff(h, t, pre: str) -> torch.Tensor:
    return relu2(h @ t[pre + "up"].T) @ t[pre + "down"].T


def choose_experts(z: torch.Tensor, correction: torch.Tensor, r: dict):
    """z [n, E] router logits.  Returns (chosen [n, top] indices, weights [n, top])."""
    n, E = z.shape
    s = torch.sigmoid(z)
    c = s + correction
    groups = r.get("groups")
    if groups is not None:
        count, keep = groups["count"], groups["keep"]
        per = E // count
        cg = c.reshape(n, count, per)
        gs = cg.topk(min(2, per), dim=-1).values.sum(-1)                # a group's score: its two largest choice scores
        best = gs.topk(keep, dim=-1).indices
        allowed = torch.zeros((n, count), dtype=torch.bool)
        allowed.scatter_(1, best, True)
        c = cg.masked_fill(~allowed[:, :, None], -math.inf).reshape(n, E)
    chosen = c.topk(r["top"], dim=-1).indices
    w = s.gather(1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20) * r["scale"]


def expert_ff(h, t, pre: str, mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    chosen, w = choose_experts(h @ t[pre + "router"].T, t[pre + "correction"], r)
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        for c in range(r["top"]):
            rows = (chosen[:, c] == e).nonzero()[:, 0]
            if len(rows):
                out[rows] += w[rows, c][:, None] * small_ff(h[rows], t, f"{pre}e{e}.")
    if mlp.get("shared") is not None:
        out = out + small_ff(h, t, pre + "shared.") * torch.sigmoid(h @ t[pre + "shared.sg"].T)
    return out


def run_order(cfg: dict) -> List[tuple]:
    """(layer, pass number if a pass begins with this run else None) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if loop is None:
        return [(i, None) for i in range(n)]
    a, b = loop["start"], loop["stop"]
    order = [(i, None) for i in range(a)]
    for t in range(loop["times"]):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg: dict, t: Dict[str, torch.Tensor], tokens, dtype=torch.float64, taps: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence from position 0.  ``taps`` (a list) receives the stream after every layer run."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in t.items()}
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x0 = embed(tokens, t["embed"], (cfg.get("embedding") or {}).get("scale", 1.0))
    x = x0.clone()
    for i, begins in run_order(cfg):
        if begins is not None:
            if begins > 0:
                x = x + x0
            x = x + t["loop.step"][begins]
        L, pre = cfg["layers"][i], f"l{i}."
        h = norm(x, t[pre + "norm1"], eps)
        if L["type"] == "parallel":
            x = x + parallel_mixer(h, t, pre + "mix.", L["mixer"], eps)
        elif L["type"] == "gla":
            x = x + gated_linear_attention(h, t, pre + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            h = norm(x, t[pre + "norm2"], eps)
            x = x + (dense_ff(h, t, pre + "mlp.") if L["mlp"]["kind"] == "dense" else expert_ff(h, t, pre + "mlp.", L["mlp"]))
        if taps is not None:
            taps.append(x.clone())
    z = norm(x, t["final.norm"], eps) @ t["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
