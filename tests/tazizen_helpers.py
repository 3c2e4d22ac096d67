"""Small Tazizen configurations and random weights for the tests, made here (not by the library), and the
comparison rules."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rot(dims, base, scaling=None):
    r = dict(dims=dims, base=base)
    if scaling:
        r["scaling"] = dict(factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
    return r


def attn(heads, kv, dim, rot_dims, window=None, vdim=None, base=10000.0, scale=None, scaling=None):
    m = dict(heads=heads, dim=dim, scale=scale if scale is not None else 1.5 / math.sqrt(dim))
    if kv is not None:
        m["kv_heads"] = kv
    if vdim is not None:
        m["vdim"] = vdim
    if rot_dims:
        m["rot"] = rot(rot_dims, base, scaling)
    if window:
        m["mask"] = dict(size=window)
    return dict(type="attention", mixer=m)


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window=None, base=10000.0, scale=None, scaling=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank,
             scale=scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim), rot=rot(rot_dim, base, scaling))
    if window:
        m["mask"] = dict(size=window)
    return dict(type="latent_attention", mixer=m)


def moe(experts, top, ff, groups=None, scale=None, shared=None):
    r = dict(experts=experts, top=top)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    if scale is not None:
        r["scale"] = scale
    f = dict(kind="moe", expert=dict(ff=ff), router=r)
    if shared:
        f["shared"] = dict(ff=shared)
    return f


def layer(mixer, mlp):
    return dict(mlp=mlp, **mixer)


def config(vocab, width, eps, layers, streams=None, loop=None):
    c = dict(architecture="Tazizen", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if streams is not None:
        c["streams"] = streams
    if loop is not None:
        c["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return c


Y1 = (4.0, 64, 8.0, 1.0)          # a ramp that begins and ends inside the pairs
Y2 = (16.0, 4096, 32.0, 1.0)      # its first pairs keep their frequency (lo > 0)
Y3 = (2.5, 48, 4.0, 2.0)

# T1: two copies of the stream, a loop in the middle run twice, values narrower than keys, a layer without a
#     feed-forward, groups of two experts of which half are kept, windows shorter than a page.
# T2: three copies, sizes that are no multiple of 8, a latent layer without a window, an attention layer without one,
#     no shared expert, one expert chosen, no groups, no router scale.
# T3: one copy (its joining tensors are of size one), heads of 64 and 128 (the tiled kernels), windows that cross page
#     borders, a loop at the start run three times, four chosen of sixteen experts in four groups.
# T4: no `streams` key at all (the plain residual sum), no rotation in attention, as many key heads as query heads,
#     every expert chosen, one group.
# T5: five copies, heads of 80 (a prompt kernel but no single-token kernel), three query heads to one key head, windows of
#     exactly a page, a latent whose rows take the tensor-core kernels, two groups of which one is kept.
# T7: wider: four copies, a loop of three layers at the start run twice, every tiled kernel at once (heads of 64 and 128, latent
#     rows of 128 + 32 and 96 + 16), one of four groups kept.
# T6: a loop at the end run once, four query heads to a key head with heads of 32 (the single-token kernel), a rotation of
#     one pair, a scaled rotation in the latent layer, values wider than keys.
CONFIGS: Dict[str, dict] = {
    "T1": config(150, 64, 1e-6,
                 [layer(attn(4, 2, 16, 8, window=24, scaling=Y1), moe(8, 2, 24, groups=(4, 2), scale=2.5, shared=48)),
                  layer(latent(2, 16, 8, 16, 32, 24, window=17, base=5e4), None),
                  layer(attn(2, 1, 32, 32, window=70, vdim=24, base=500.0), moe(6, 2, 40, groups=(3, 1), scale=0.7))],
                 streams=2, loop=(1, 3, 2)),
    "T2": config(131, 72, 1e-5,
                 [layer(latent(3, 10, 6, 14, 40, 18, scale=0.3), moe(6, 3, 20, groups=(3, 2))),
                  layer(attn(6, 3, 12, 12, vdim=20, base=777.0), moe(5, 1, 36)),
                  layer(attn(3, None, 20, 10, window=9), None)], streams=3),
    "T3": config(300, 128, 2e-6,
                 [layer(attn(4, 2, 64, 32, window=100, base=1e5), moe(16, 4, 32, groups=(4, 2), scale=1.5, shared=64)),
                  layer(latent(4, 32, 16, 32, 64, 48, window=130, base=1e6, scaling=Y2), moe(8, 2, 64, shared=32)),
                  layer(attn(2, 2, 128, 64, window=65, scaling=Y2), moe(4, 2, 48, groups=(2, 1), scale=3.0))],
                 streams=1, loop=(0, 2, 3)),
    "T4": config(97, 48, 1e-5,
                 [layer(attn(3, 3, 16, 0), moe(4, 4, 24, groups=(1, 1), scale=2.0, shared=16)),
                  layer(latent(1, 8, 2, 8, 16, 8, window=33, scale=0.4), moe(3, 2, 40))]),
    "T5": config(90, 80, 3e-6,
                 [layer(latent(5, 16, 8, 24, 48, 32, window=64, base=2e3, scaling=Y3), moe(12, 2, 16, groups=(2, 1), scale=1.2, shared=40)),
                  layer(attn(3, 1, 80, 40, window=64, base=3e4, scaling=Y3), moe(12, 5, 16, groups=(3, 2), shared=24))],
                 streams=5),
    "T6": config(180, 96, 1e-5,
                 [layer(latent(2, 24, 4, 40, 80, 20, base=5e4, scale=0.2, scaling=Y1), moe(8, 3, 32, groups=(2, 2), scale=0.5)),
                  layer(attn(8, 2, 32, 2, window=40, scale=0.9), None),
                  layer(attn(4, 1, 32, 16, window=150, vdim=48), moe(9, 2, 28, groups=(3, 1), shared=56))],
                 streams=2, loop=(1, 3, 1)),
    "T7": config(500, 256, 1e-5,
                 [layer(latent(8, 64, 32, 64, 128, 96, window=48, base=1e6), moe(16, 2, 64, groups=(4, 1), scale=1.0, shared=128)),
                  layer(attn(8, 4, 128, 64, window=80, scaling=Y2), moe(16, 3, 64, groups=(2, 1), scale=2.0, shared=64)),
                  layer(latent(4, 32, 16, 32, 96, 64, window=200, base=1e4, scaling=Y1), None),
                  layer(attn(4, 4, 64, 64, window=31, vdim=64), moe(8, 2, 96))],
                 streams=4, loop=(0, 3, 2)),
}


def tensor_shapes(c: dict) -> Dict[str, List[int]]:
    W = c["width"]
    out = {"embed": [c["vocab"], W], "final.norm": [W], "head": [c["vocab"], W]}
    S = c.get("streams")
    for i, L in enumerate(c["layers"]):
        m, p = L["mixer"], f"l{i}."
        out[p + "norm1"] = [W]
        x = p + "mix."
        if L["type"] == "attention":
            H, d = m["heads"], m["dim"]
            G, dv = m.get("kv_heads", H), m.get("vdim", d)
            out.update({x + "q": [H * d, W], x + "k": [G * d, W], x + "v": [G * dv, W], x + "g": [H * dv, W], x + "o": [W, H * dv]})
        else:
            H, d, r, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({x + "dq": [Q, W], x + "dq.norm": [Q], x + "uq": [H * (d + r), Q], x + "dkv": [R + r, W], x + "dkv.norm": [R],
                        x + "uk": [H * d, R], x + "uv": [H * dv, R], x + "o": [W, H * dv]})
        if S is not None:
            out.update({p + "hc1.in": [S], p + "hc1.out": [S], p + "hc1.mix": [S, S]})
        f = L["mlp"]
        if f is None:
            continue
        out[p + "norm2"] = [W]
        if S is not None:
            out.update({p + "hc2.in": [S], p + "hc2.out": [S], p + "hc2.mix": [S, S]})
        y = p + "mlp."
        ff = f["expert"]["ff"]
        for e in range(f["router"]["experts"]):
            out.update({f"{y}e{e}.gate": [ff, W], f"{y}e{e}.up": [ff, W], f"{y}e{e}.down": [W, ff]})
        out.update({y + "router": [f["router"]["experts"], W], y + "correction": [f["router"]["experts"]]})
        if f.get("shared"):
            sf = f["shared"]["ff"]
            out.update({y + "shared.gate": [sf, W], y + "shared.up": [sf, W], y + "shared.down": [W, sf], y + "shared.sg": [1, W]})
    return out


def random_weights(c: dict, seed: int = 0, steady_choice: bool = False) -> Dict[str, torch.Tensor]:
    """bfloat16-representable float32 tensors: matrices ~ N(0, 1.3^2 / fan_in), norm weights around nought (they are
    applied as 1 + w), routers that spread their logits, corrections that matter, joins of the copies near the plain
    residual sum but with every entry different.  `steady_choice`: for bfloat16 runs of whole models."""
    g = torch.Generator().manual_seed(seed)
    S = c.get("streams", 1)
    out = {}
    for name, shape in tensor_shapes(c).items():
        r = lambda *s: torch.randn(*s, generator=g)
        if name.endswith("hc1.mix") or name.endswith("hc2.mix"):
            t = torch.eye(S) * 0.8 + 0.2 / S + 0.15 * r(shape)
        elif name.endswith(".in"):
            t = 1.0 / S + 0.3 * r(shape)
        elif name.endswith(".out"):
            t = 1.0 + 0.3 * r(shape)
        elif name.endswith("correction"):
            # steady_choice: corrections 0.6 apart in a random order, so that a router's choice mostly rests on them and
            # the noise of bfloat16 scores seldom turns it (tests/tazizen_helpers.py: check_rows says why)
            t = 0.6 * torch.randperm(shape[0], generator=g).float() if steady_choice else 0.3 * r(shape)
        elif name.endswith("dq.norm") or name.endswith("dkv.norm"):
            t = 1.0 + 0.2 * r(shape)
        elif len(shape) == 1:
            t = 0.2 * r(shape)
        elif name.endswith("router") or name.endswith("shared.sg"):
            t = r(shape) * 3.0 / math.sqrt(shape[1])
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


# float32: rounding alone.  bfloat16: activations are rounded to 8 bits at every product's input, and by the later layers
# a router's scores carry a hundredth or so of noise: where two experts' corrected scores (or two groups') lie closer than
# that the choice turns, which moves that position by far more than rounding does and, through the cache, those behind
# it (the fewer keys a position sees, the more).  So a bfloat16 run of a whole model is compared up to the first position
# whose closest choice (the plain implementation reports the margins) is narrower than SURE, and must be finite after;
# the weights for such runs space the corrections out so that this is seldom early (random_weights: steady_choice).
# The mechanisms themselves are compared in bfloat16 one by one, with the choice given, by the kernel tests.
TOL = {"float32": 3e-5, "bfloat16": 0.15}
SURE = 0.05


def check_rows(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, margin: Optional[torch.Tensor] = None) -> None:
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    e = row_errors(got, ref)
    if dtype == "float32":
        if margin is not None:
            e = e[margin > 1e-4]            # a choice closer than that is no test of anything
        if e.numel():
            assert float(e.max()) < TOL[dtype], f"{what}: row error {float(e.max()):.3e} at position {int(e.argmax())} of {e.numel()} ({dtype})"
        return
    if margin is not None:
        unsure = (margin <= SURE).nonzero()
        if unsure.numel():
            e = e[:int(unsure[0])]
    if e.numel() == 0:
        return
    assert float(e.max()) < TOL[dtype], f"{what}: row error {float(e.max()):.3e} at position {int(e.argmax())} of {e.numel()} ({dtype})"
    assert float(e.median()) < TOL[dtype] / 3, f"{what}: median row error {float(e.median()):.3e} ({dtype})"
