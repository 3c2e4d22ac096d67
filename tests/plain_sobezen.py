"""A plain, slow implementation of the Sobezen decoder in float64, one function per mechanism.  It shares no
code with the library: the tests compare the library against it.  Weights are a dict name -> tensor with the
design's own names ("embed", "l<i>.norm1", "l<i>.mix.<x>", "l<i>.mlp.<x>", "l<i>.ls1", "final.norm", "head")."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---------------------------------------------------------------- rotation
def pair_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i/n) for the n/2 pairs; with `scaling` the slow pairs are divided by `factor`, the fast ones
    kept, and a linear ramp over the pair index joins them."""
    n, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / n) for i in range(n // 2)]
    sc = rot.get("scaling")
    if sc:
        where = lambda turns: n * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), n - 1)
        for i in range(n // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / sc["factor"] * ramp + f[i] * (1.0 - ramp)
    return torch.tensor(f, dtype=F64)


def table_magnitude(rot: dict) -> float:
    sc = rot.get("scaling")
    return 0.1 * math.log(sc["factor"]) + 1.0 if sc else 1.0


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, d]: channels (2i, 2i + 1) of the first rot.dims channels turn by pos * f_i; the rest stay."""
    n = rot["dims"]
    angle = pos.to(F64)[:, None] * pair_frequencies(rot)[None, :]
    m = table_magnitude(rot)
    c, s = (torch.cos(angle) * m)[:, None, :], (torch.sin(angle) * m)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


# ---------------------------------------------------------------- attention
def causal_softmax(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, shares: Optional[list] = None) -> torch.Tensor:
    """q [T, H, d], k [T, H, d], v [T, H, dv]: position i sees every j <= i.  ``shares`` collects the weights [H, T, T]."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
    a = torch.softmax(s, -1)
    if shares is not None:
        shares.append(a)
    return torch.einsum("hij,jhd->ihd", a, v)


def keyed_attention(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, pos: torch.Tensor, shares: Optional[list] = None) -> torch.Tensor:
    """Grouped-query attention whose values are the keys as projected (bias added, not rotated)."""
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = k.clone()
    q, k = rotate_pairs(q, pos, m["rot"]), rotate_pairs(k, pos, m["rot"])
    k, v = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    return causal_softmax(q, k, v, m["scale"], shares).reshape(T, H * d) @ w[p + "o"].T


def latent_rows(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, pos: torch.Tensor, eps: float):
    """What a position leaves behind: the normed latent c [T, kv_rank] and the rotated key part [T, rot_dim]."""
    R = m["kv_rank"]
    both = h @ w[p + "dkv"].T
    c = rms_norm(both[:, :R], w[p + "dkv.norm"], eps)
    shared = rotate_pairs(both[:, None, R:], pos, m["rot"])[:, 0]
    return c, shared


def latent_attention(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, pos: torch.Tensor, eps: float, rows,
                     shares: Optional[list] = None) -> torch.Tensor:
    H, d, r, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = h.shape[0]
    c, shared = rows
    q = (rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps) @ w[p + "uq"].T).reshape(T, H, d + r)
    q = torch.cat([q[..., :d], rotate_pairs(q[..., d:], pos, m["rot"])], -1)
    k = torch.cat([(c @ w[p + "uk"].T).reshape(T, H, d), shared[:, None, :].expand(T, H, r)], -1)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    return causal_softmax(q, k, v, m["scale"], shares).reshape(T, H * dv) @ w[p + "o"].T


# ---------------------------------------------------------------- the gated delta rule
def short_conv(x: torch.Tensor, w: torch.Tensor, before: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], w [C, taps] (last column: the token's own); `before`: the taps - 1 rows ahead of x (zeros at a start)."""
    T, C = x.shape
    taps = w.shape[1]
    if before is None:
        before = torch.zeros(taps - 1, C, dtype=x.dtype)
    xp = torch.cat([before, x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + xp[j:j + T] * w[:, j][None, :]
    return y


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def unit_vector(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def delta_steps(q, k, v, beta, g, S=None):
    """q, k, g [T, H, d], v [T, H, dv], beta [T, H]; S [H, d, dv].  Per token: decay, then the write of what the
    state does not yet answer for this key, then the read-out (which sees that write)."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=F64) if S is None else S.clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = g[t][:, :, None] * S
        e = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * e[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def channel_delta(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float, survives: Optional[list] = None) -> torch.Tensor:
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = (unit_vector(q) * d ** -0.5).repeat_interleave(H // G, 1)
    k = unit_vector(k).repeat_interleave(H // G, 1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    step = torch.nn.functional.softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(T, H, d)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)
    o, _ = delta_steps(q, k, v, beta, g)
    if survives is not None:                           # how large a head's result is against the norm's eps
        survives.append((o * o).mean(-1).min(-1).values)
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    return (rms_norm(o, w[p + "norm"], eps) * gate).reshape(T, H * dv) @ w[p + "o"].T


# ---------------------------------------------------------------- feed-forward
def clamped_unit(w: Dict[str, torch.Tensor], p: str, f: dict, h: torch.Tensor) -> torch.Tensor:
    lim = f["limit"]
    g = torch.clamp(h @ w[p + "gate"].T + w[p + "gate.b"], max=lim)
    u = torch.clamp(h @ w[p + "up"].T + w[p + "up.b"], -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T + w[p + "down.b"]


# ---------------------------------------------------------------- the model
def forward(c: dict, w: Dict[str, torch.Tensor], tokens: List[int], stream_after: Optional[list] = None,
            survives: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps = c["norm"]["eps"]
    T = len(tokens)
    pos = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)] * c.get("embedding", {}).get("scale", 1.0)
    rows = {}
    for i, L in enumerate(c["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        if L["type"] == "attention":
            y = keyed_attention(w, p + "mix.", m, h, pos)
        elif L["type"] == "latent_attention":
            if m.get("kv_from") is None:
                rows[i] = latent_rows(w, p + "mix.", m, h, pos, eps)
            y = latent_attention(w, p + "mix.", m, h, pos, eps, rows[i if m.get("kv_from") is None else m["kv_from"]])
        elif L["type"] == "channel_delta":
            y = channel_delta(w, p + "mix.", m, h, eps, survives)
        else:
            raise ValueError(L["type"])
        x = x + y * w[p + "ls1"]
        if L["mlp"] is not None:
            x = x + clamped_unit(w, p + "mlp.", L["mlp"], rms_norm(x, w[p + "norm2"], eps)) * w[p + "ls2"]
        if stream_after is not None:
            stream_after.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T * c.get("logit_scale", 1.0)
