"""Small Sobezen configurations and random weights for the tests, made here (not by the library),
and the comparison rules."""
from __future__ import annotations

import math
from typing import Dict, List

import torch


def rot(dims, base, scaling=None):
    r = dict(dims=dims, base=base)
    if scaling:
        r["scaling"] = dict(factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
    return r


def attn(heads, kv, dim, rot_dims, base=10000.0, scale=None, scaling=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale if scale is not None else 1.0 / math.sqrt(dim),
             rot=rot(rot_dims, base, scaling))
    return dict(type="attention", mixer=m)


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=10000.0, scale=None, scaling=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank,
             scale=scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim), rot=rot(rot_dim, base, scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def delta(heads, kv, dim, vdim, conv):
    return dict(type="channel_delta", mixer=dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv))


def dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def layer(mixer, mlp):
    return dict(mlp=mlp, **mixer)


def config(vocab, width, eps, layers, embedding_scale=None, logit_scale=None):
    c = dict(architecture="Sobezen", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if embedding_scale is not None:
        c["embedding"] = dict(scale=embedding_scale)
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    return c


Y1 = (4.0, 64, 8.0, 1.0)          # a ramp that begins and ends inside the pairs
Y2 = (16.0, 4096, 32.0, 1.0)      # its first pairs keep their frequency (lo > 0)
Y3 = (2.5, 48, 4.0, 2.0)

# B1: every kind of layer; two query heads to a key head in the delta rule with values wider than keys, a partial
#     rotation, a latent layer that lends its rows to a later one across a delta layer, limits that bind.
# B2: sizes that are no multiple of 8 or 16, no embedding scale and no logit scale, a latent layer without scaling
#     that lends its rows to two layers, five taps, one key head for three query heads, a full rotation.
# B3: heads of 64 (the tiled kernels), two latent layers with rows of their own and one that borrows, four taps.
# B4: one tap (no state of the convolution), one delta head of 128 channels, as many key heads as query heads in
#     attention, a rotation of one pair, a latent of one head, a layer without feed-forward at the end.
# B5: widths that are multiples of 2 only (no 16-byte rows anywhere), six taps, delta heads of 10 with values of 6,
#     a scaled rotation on attention too.
# B6: delta layers only with feed-forwards, then attention without one: the orders a served model does not have.
CONFIGS: Dict[str, dict] = {
    "B1": config(150, 64, 1e-6,
                 [layer(delta(4, 2, 16, 24, 3), dense(96, 1.5)), layer(attn(4, 1, 32, 16, scale=0.2), None),
                  layer(latent(2, 24, 8, 40, 48, 20, base=5e4, scale=0.15, scaling=Y1), dense(80, 3.0)),
                  layer(delta(2, 2, 8, 8, 2), None),
                  layer(latent(2, 24, 8, 40, 48, 20, base=5e4, scale=0.15, scaling=Y1, kv_from=2), dense(72, 0.7))],
                 embedding_scale=8.0, logit_scale=0.5),
    "B2": config(131, 72, 1e-5,
                 [layer(latent(3, 16, 4, 12, 40, 24, scale=0.3), None), layer(attn(6, 2, 12, 12, base=500.0, scale=0.3), dense(50, 2.5)),
                  layer(latent(3, 16, 4, 12, 40, 24, scale=0.3, kv_from=0), dense(44, 1.0)), layer(delta(3, 1, 24, 10, 5), dense(60, 4.0)),
                  layer(latent(3, 16, 4, 12, 40, 24, scale=0.3, kv_from=0), None)]),
    "B3": config(300, 128, 2e-6,
                 [layer(attn(4, 2, 64, 32, base=1e5, scale=0.11), dense(160, 2.0)),
                  layer(latent(4, 64, 32, 64, 128, 96, base=1e6, scaling=Y2), dense(96, 6.0)), layer(delta(2, 2, 64, 64, 4), None),
                  layer(latent(2, 32, 16, 48, 64, 32, base=3e4, scale=0.2, scaling=Y1), None),
                  layer(latent(2, 32, 16, 48, 64, 32, base=3e4, scale=0.2, scaling=Y1, kv_from=3), dense(64, 1.2))],
                 embedding_scale=11.3, logit_scale=3.0),
    "B4": config(97, 48, 1e-5,
                 [layer(delta(1, 1, 128, 32, 1), dense(64, 2.0)), layer(attn(3, 3, 16, 2, scale=0.25), dense(40, 5.0)),
                  layer(latent(1, 8, 2, 8, 16, 8, scale=0.4), None)], embedding_scale=0.7),
    "B5": config(90, 50, 3e-6,
                 [layer(delta(3, 1, 10, 6, 6), None), layer(attn(6, 2, 18, 10, base=777.0, scale=0.25, scaling=Y3), dense(34, 0.9)),
                  layer(latent(5, 6, 6, 10, 22, 14, base=2e3, scale=0.33, scaling=Y3), dense(26, 2.2)),
                  layer(latent(5, 6, 6, 10, 22, 14, base=2e3, scale=0.33, scaling=Y3, kv_from=2), None)], logit_scale=1.5),
    "B6": config(180, 96, 1e-5,
                 [layer(delta(3, 3, 32, 16, 4), dense(72, 2.0)), layer(delta(4, 2, 48, 24, 3), dense(128, 1.0)),
                  layer(attn(2, 1, 64, 64, scale=0.15), None), layer(delta(6, 2, 16, 16, 2), None)], embedding_scale=9.8, logit_scale=2.5),
}
# the ranks of the low-rank inputs of decay and gate (the configuration does not give them: read from the tensors)
RANKS = {"B1": (8, 12), "B2": (5, 3), "B3": (16, 24), "B4": (24, 8), "B5": (3, 7), "B6": (7, 10)}


def tensor_shapes(c: dict, ranks=(-1, -1)) -> Dict[str, List[int]]:
    W = c["width"]
    ra, rg = ranks
    out = {"embed": [c["vocab"], W], "final.norm": [W], "head": [c["vocab"], W]}
    for i, L in enumerate(c["layers"]):
        m, p = L["mixer"], f"l{i}."
        out.update({p + "norm1": [W], p + "ls1": [W]})
        x = p + "mix."
        if L["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            out.update({x + "q": [H * d, W], x + "q.b": [H * d], x + "k": [G * d, W], x + "k.b": [G * d], x + "o": [W, H * d]})
        elif L["type"] == "latent_attention":
            H, d, r, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({x + "dq": [Q, W], x + "dq.norm": [Q], x + "uq": [H * (d + r), Q], x + "uk": [H * d, R], x + "uv": [H * dv, R],
                        x + "o": [W, H * dv]})
            if m.get("kv_from") is None:
                out.update({x + "dkv": [R + r, W], x + "dkv.norm": [R]})
        else:
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            out.update({x + "q": [G * d, W], x + "q.conv": [G * d, taps], x + "k": [G * d, W], x + "k.conv": [G * d, taps],
                        x + "v": [H * dv, W], x + "v.conv": [H * dv, taps], x + "b": [H, W], x + "A_log": [H], x + "norm": [dv],
                        x + "a1": [ra, W], x + "a2": [H * d, ra], x + "dt_bias": [H * d], x + "g1": [rg, W], x + "g2": [H * dv, rg],
                        x + "o": [W, H * dv]})
        f = L["mlp"]
        if f is None:
            continue
        out.update({p + "norm2": [W], p + "ls2": [W]})
        for n, shape in (("gate", [f["ff"], W]), ("up", [f["ff"], W]), ("down", [W, f["ff"]])):
            out[p + "mlp." + n] = shape
            out[p + "mlp." + n + ".b"] = shape[:1]
    return out


def random_weights(c: dict, seed: int = 0, ranks=(8, 8)) -> Dict[str, torch.Tensor]:
    """bfloat16-representable float32 tensors: matrices ~ N(0, 1/fan_in) times a factor that keeps the stream of
    order one (token rows are divided by the embedding's scale), norm weights around 1, layer scales around 0.6,
    biases around 0, decays spread from fast to slow."""
    g = torch.Generator().manual_seed(seed)
    scale = c.get("embedding", {}).get("scale", 1.0)
    out = {}
    for name, shape in tensor_shapes(c, ranks).items():
        r = lambda *s: torch.randn(*s, generator=g)
        if name.endswith(".conv"):
            t = 0.5 * r(shape)
        elif name.endswith("A_log"):
            t = 0.8 * r(shape) - 1.5
        elif name.endswith(".b") or name.endswith("dt_bias"):
            t = 0.5 * r(shape)
        elif name.endswith("ls1") or name.endswith("ls2"):
            t = 0.6 + 0.2 * r(shape)
        elif len(shape) == 1:
            t = 1.0 + 0.2 * r(shape)
        elif name == "embed":
            t = r(shape) / scale
        elif name.endswith("a2") or name.endswith("g2") or name.endswith("mix.b"):
            t = r(shape) * 2.0 / math.sqrt(shape[1])
        else:
            t = r(shape) * 1.3 / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16).float()
    return out


def tokens(c: dict, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(7000 + seed)
    return torch.randint(0, c["vocab"], (n,), generator=g).tolist()


def row_errors(got: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per position: the root mean square of the difference over the vocabulary, relative to the root mean square
    of the reference's logits (over everything)."""
    ref = ref.to(torch.float64)
    d = got.to(torch.float64).cpu() - ref
    return (d * d).mean(-1).sqrt() / (ref * ref).mean().sqrt()


# float32: rounding alone.  bfloat16: activations are rounded to 8 bits at every product's input.
TOL = {"float32": 3e-5, "bfloat16": 5e-2}


def check_rows(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str) -> None:
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    e = row_errors(got, ref)
    assert float(e.max()) < TOL[dtype], f"{what}: row error {float(e.max()):.3e} at position {int(e.argmax())} of {e.numel()} ({dtype})"
