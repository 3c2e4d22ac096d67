"""The Tazizen decoder, plainly: float64 torch on the CPU, one function per mechanism, whole sequences at once (no
cache, no batching, no portions).  It shares nothing with the library; the tests compare the library with it.

A sequence's positions are 0 .. n-1.  `w` maps tensor names to float tensors, `c` is the configuration as the
model's config.json gives it."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """An RMS norm whose weight is stored around nought: unit_rms(x) * (1 + weight)."""
    return unit_rms(x, eps) * (1.0 + weight)


def frequencies(rot: dict):
    """Per pair i < dims/2: the angular frequency, and the factor on cosines and sines alike."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    pair_of = lambda turns: dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [n, heads, d]: channel i < dims/2 of every head is paired with channel i + dims/2; the rest pass."""
    if not rot:
        return x
    dims = rot["dims"]
    half = dims // 2
    f, magnitude = frequencies(rot)
    angle = positions.to(F64)[:, None] * f[None, :]
    cos, sin = (torch.cos(angle) * magnitude)[:, None, :], (torch.sin(angle) * magnitude)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def visible(n: int, window: Optional[int]) -> torch.Tensor:
    """[query, key]: key j is seen from position i when 0 <= i - j (< window)."""
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    see = j <= i
    if window:
        see = see & (i - j < window)
    return see


def softmax_one_more(scores: torch.Tensor, see: torch.Tensor, extra: Optional[float]) -> torch.Tensor:
    """Softmax over the seen keys; with `extra` the denominator also holds exp(extra) (a key without a value)."""
    s = scores.masked_fill(~see, -float("inf"))
    top = s.max(-1, keepdim=True).values
    if extra is not None:
        top = top.clamp(min=extra)
    e = torch.exp(s - top)
    denom = e.sum(-1, keepdim=True)
    if extra is not None:
        denom = denom + torch.exp(extra - top)
    return e / denom


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    dv = m.get("vdim", d)
    pos = torch.arange(n)
    q = (h @ w[p + "q"].T).view(n, H, d)
    k = (h @ w[p + "k"].T).view(n, G, d)
    v = (h @ w[p + "v"].T).view(n, G, dv)
    q = unit_rms(rotate_halves(q, pos, m.get("rot")), eps)          # the norm comes after the rotation, per head, no weight
    k = unit_rms(rotate_halves(k, pos, m.get("rot")), eps)
    see = visible(n, (m.get("mask") or {}).get("size"))
    heads = []
    for a in range(H):
        g = a // (H // G)
        prob = softmax_one_more((q[:, a] @ k[:, g].T) * m["scale"], see, 0.0)
        heads.append(prob @ v[:, g])
    joined = torch.cat(heads, dim=-1) * torch.sigmoid(h @ w[p + "g"].T)
    return joined @ w[p + "o"].T


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m.get("vdim", m["dim"]), m["kv_rank"]
    pos = torch.arange(n)
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(n, H, d + r)
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :R], eps) * w[p + "dkv.norm"]
    shared_key = rotate_halves(down[:, None, R:], pos, m.get("rot"))[:, 0]
    q_plain, q_rot = q[..., :d], rotate_halves(q[..., d:], pos, m.get("rot"))
    k_plain = (c @ w[p + "uk"].T).view(n, H, d)
    v = (c @ w[p + "uv"].T).view(n, H, dv)
    see = visible(n, (m.get("mask") or {}).get("size"))
    heads = []
    for a in range(H):
        scores = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ shared_key.T) * m["scale"]
        heads.append(softmax_one_more(scores, see, None) @ v[:, a])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def gated_unit(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = h @ w[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, r: dict):
    """-> chosen [n, top] (indices), weights [n, top], margin [n]: how far the last chosen corrected score lies above
    the best one left out (a small margin is a close call that rounding may turn)."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    groups = r.get("groups")
    if groups:
        per = E // groups["count"]
        by_group = choice.view(-1, groups["count"], per)
        score = by_group.topk(min(2, per), dim=-1).values.sum(-1)
        kept = torch.zeros_like(score, dtype=torch.bool)
        kept.scatter_(1, score.topk(groups["keep"], dim=-1).indices, True)
        choice = by_group.masked_fill(~kept[:, :, None], -float("inf")).reshape(-1, E)
    ranked = choice.sort(dim=-1, descending=True)
    chosen = ranked.indices[:, :top]
    margin = ranked.values[:, top - 1] - ranked.values[:, top] if top < E else torch.full((h.shape[0],), float("inf"), dtype=F64)
    if groups and groups["keep"] < groups["count"]:
        gs = score.sort(dim=-1, descending=True).values
        margin = torch.minimum(margin, gs[:, groups["keep"] - 1] - gs[:, groups["keep"]])
    picked = s.gather(1, chosen)
    weights = picked / (picked.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    return chosen, weights, margin


def experts(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict, margins: Optional[list] = None) -> torch.Tensor:
    chosen, weights, margin = route(h, w, p, f["router"])
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(h)
    for e in chosen.unique().tolist():
        rows, place = (chosen == e).nonzero(as_tuple=True)
        out[rows] += weights[rows, place, None] * gated_unit(h[rows], w, f"{p}e{e}.")
    if f.get("shared"):
        out = out + gated_unit(h, w, p + "shared.") * torch.sigmoid(h @ w[p + "shared.sg"].T)
    return out


def order_of_runs(c: dict) -> List[int]:
    n = len(c["layers"])
    loop = c.get("loop")
    if not loop:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop.get("times", 1) + list(range(loop["stop"], n))


def join_streams(xs: List[torch.Tensor], y_of, w: Dict[str, torch.Tensor], p: str) -> List[torch.Tensor]:
    """One sublayer on several copies of the stream: it reads sum_s in[s] x_s, and its result y moves every copy at
    once, x_t <- sum_s mix[s, t] x_s + out[t] y."""
    S = len(xs)
    a, b, M = w[p + "in"], w[p + "out"], w[p + "mix"]
    y = y_of(sum(a[s] * xs[s] for s in range(S)))
    return [sum(M[s, t] * xs[s] for s in range(S)) + b[t] * y for t in range(S)]


def forward(c: dict, w: Dict[str, torch.Tensor], tokens: List[int], after_runs: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab].  `after_runs` receives the stream (the sum of its copies) after every layer run, `margins`
    the routers' margins."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps = c["norm"]["eps"]
    x0 = w["embed"][torch.tensor(tokens)]
    hyper = "streams" in c
    xs = [x0.clone() for _ in range(c.get("streams", 1))]
    for i in order_of_runs(c):
        L, p = c["layers"][i], f"l{i}."
        mixer = attention if L["type"] == "attention" else latent_attention
        subs = [("1", lambda u: mixer(norm_around_zero(u, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps))]
        if L.get("mlp") is not None:
            subs.append(("2", lambda u: experts(norm_around_zero(u, w[p + "norm2"], eps), w, p + "mlp.", L["mlp"], margins)))
        for q, y_of in subs:
            xs = join_streams(xs, y_of, w, f"{p}hc{q}.") if hyper else [xs[0] + y_of(xs[0])]
        if after_runs is not None:
            after_runs.append(sum(xs))
    return norm_around_zero(sum(xs), w["final.norm"], eps) @ w["head"].T
