"""The mechanisms Sobezen adds, each alone (a part built from its description, run through the host library's part
handle) against the plain implementation's function for it: the rotation table of neighbouring pairs with the
ramp between kept and slowed frequencies, attention whose values are its keys, latent attention with rows of its
own and with borrowed rows, the delta rule with a decay per key channel and its carried state, the clamped gated
unit, and a sublayer's scale per channel.  Attention is run with a score scale that makes one key stand out for
almost every query, wherever it lies (far back, next to a page border, the query's own position), so that a mask or
a page one position off shows; prompts, portions and single tokens share the calls."""
import math

import pytest
import torch

import plain_sobezen as P
import sobezen_helpers as S
from test_parts_gpu import PAGE, Step, act, part, summed

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# on |got - ref| / (|ref| + mean |ref|), element by element
TOL = {"float32": 3e-5, "bfloat16": 3e-2}


def bf(t):
    return t.to(torch.bfloat16).float()


def close(got, ref, dtype, what, roundings=1.0):
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got.float()).all(), f"{what}: not finite"
    ref = ref.to(torch.float64)
    d = (got.to(torch.float64).cpu() - ref).abs()
    e = float((d / (ref.abs() + ref.abs().mean())).max())
    assert e < TOL[dtype] * roundings, f"{what}: error {e:.3e} ({dtype})"


def mixer_of(layers, i, dtype, seed, ranks=(6, 9), max_positions=1024):
    """Layer i's mixer of a model of `layers`, as the configuration's reader describes it, with weights of its own."""
    from libllm_b200 import _lib
    c = S.config(64, WIDTH, EPS, layers)
    spec = _lib.describe_model(c, dtype)["spec"]["layers"][i]["mixer"]
    w = {k: v for k, v in S.random_weights(c, seed, ranks).items() if k.startswith(f"l{i}.mix.")}
    m = part("mixer", spec, dtype, max_positions)
    m.load(w)
    return m, {k: v.double() for k, v in w.items()}, spec


WIDTH, EPS = 56, 1e-5


def run_in_portions(mixers, caches, x, portions, dtype, lens, state=None, slots=None):
    """Sequences of `lens` tokens of x (a list of [n, WIDTH]) brought in `portions` (a list of lists: new tokens per
    sequence and call, 0 = the sequence sits the call out) through every mixer of `mixers` in turn (they share the
    step; mixer j reads and writes caches[j]).  Returns per mixer and sequence the rows of the result."""
    done = [0] * len(lens)
    got = [[[] for _ in lens] for _ in mixers]
    pages = sum((n + PAGE - 1) // PAGE for n in lens) + 4
    for por in portions:
        seqs = [b for b in range(len(lens)) if por[b] > 0]
        step = Step([por[b] for b in seqs], [done[b] for b in seqs])
        # pages of a sequence stay its own from call to call: logical page j of sequence b is page (j * 5 + b * 2 + 1) % pages
        width = max((done[b] + por[b] + PAGE - 1) // PAGE for b in seqs)
        table = torch.tensor([[PAGE_OF[(b, j)] for j in range(width)] for b in seqs], dtype=torch.int32, device=DEV)
        if slots is not None:
            step.keep["seq_slot"].copy_(torch.tensor([slots[b] for b in seqs], dtype=torch.int32))
            step.json["slots"] = [slots[b] for b in seqs]
        xs = torch.cat([x[b][done[b]:done[b] + por[b]] for b in seqs]).to(DT[dtype]).to(DEV)
        for j, m in enumerate(mixers):
            call = dict(step=step.json, x=act(xs))
            if caches[j] is not None:
                k, v, writes = caches[j]
                call["cache"] = dict(k=k.data_ptr(), v=v.data_ptr() if v is not None else 0, n_pages=k.shape[0],
                                     page_table=table.data_ptr(), table_width=width, writes=writes)
            if state is not None:
                call["state"] = state
            out = summed(m.forward(call)["out"]).cpu()
            at = 0
            for b in seqs:
                got[j][b].append(out[at:at + por[b]])
                at += por[b]
        for b in seqs:
            done[b] += por[b]
    assert done == list(lens)
    return [[torch.cat(rows) for rows in per] for per in got]


# logical page j of sequence b -> a page of the store, scattered and never shared
PAGE_OF = {(b, j): 3 + b + 4 * j if j % 2 == 0 else 40 - b - 4 * j for b in range(4) for j in range(5)}
assert len(set(PAGE_OF.values())) == len(PAGE_OF) and min(PAGE_OF.values()) >= 0
N_PAGES = max(PAGE_OF.values()) + 1
LENS = [300, 66, 130]
# a prompt each; single tokens over the page border at 64 / 128 / 192 (the second sequence ends first); portions of
# two and three tokens; most of the rest of the first sequence in one portion; single tokens past 256 positions (where
# a token's keys are shared out over two runs); the last of it
PORTIONS = [[60, 63, 120]] + [[1, 1, 1]] * 3 + [[2, 0, 3], [1, 0, 1], [3, 0, 2], [1, 0, 1]] + [[200, 0, 0]] + [[1, 0, 0]] * 2 + [[28, 0, 0]]
assert [sum(p[b] for p in PORTIONS) for b in range(3)] == LENS


def sharp_inputs(seed, lens=LENS):
    g = torch.Generator().manual_seed(seed)
    return [bf(torch.randn(n, WIDTH, generator=g)) for n in lens]


def check_sharpness(shares, what):
    """The test means something only if most queries give most of their weight to one key, and those keys lie
    anywhere: many far back, some on either side of a page border, some the query's own position."""
    a = shares[0]                                       # [H, T, T]
    top, where = a.max(-1)
    T = a.shape[1]
    i = torch.arange(T)[None, :].expand_as(where)
    sharp = top > 0.6
    assert float(sharp.float().mean()) > 0.5, f"{what}: the scores are not sharp enough to show a misplaced key"
    far = (sharp & (i - where > 64)).sum()
    own = (sharp & (where == i) & (i > 0)).sum()
    edge = (sharp & ((where % PAGE == 0) | (where % PAGE == PAGE - 1)) & (i - where > 1)).sum()
    assert far > 20 and own > 3 and edge > 3, f"{what}: far {int(far)}, own {int(own)}, at a page's edge {int(edge)}"


# ---------------------------------------------------------------- the rotation's table
@pytest.mark.parametrize("rot", [S.rot(8, 5e4, S.Y1), S.rot(32, 1e6, S.Y2), S.rot(6, 2e3, S.Y3), S.rot(12, 500.0), S.rot(2, 1e4)])
def test_pair_table_holds_the_ramped_frequencies_and_the_magnitude(rot):
    """The position part of a latent layer: row p holds cos and sin of p * f_i, both times 0.1 ln(factor) + 1."""
    layers = [S.layer(S.latent(2, 8, rot["dims"], 8, 16, 8, base=rot["base"], scale=0.3,
                               scaling=tuple(rot["scaling"][k] for k in ("factor", "original", "fast", "slow")) if "scaling" in rot else None), None)]
    from libllm_b200 import _lib
    spec = _lib.describe_model(S.config(64, WIDTH, EPS, layers), "float32")["spec"]["layers"][0]["mixer"]["position"]
    assert spec["pairing"] == "interleaved"
    pos = part("position", spec, "float32", 300)
    pos.load({})
    table = pos.forward(dict(step=Step([1], [0]).json))["table"].torch().cpu().double()      # [positions, cosines | sines]
    n = rot["dims"]
    angle = torch.arange(300, dtype=torch.float64)[:, None] * P.pair_frequencies(rot)[None, :]
    m = P.table_magnitude(rot)
    assert table.shape == (300, n)
    assert float((table[:, :n // 2] - torch.cos(angle) * m).abs().max()) < 2e-5 * max(1.0, 300 * float(P.pair_frequencies(rot).max()))
    assert float((table[:, n // 2:] - torch.sin(angle) * m).abs().max()) < 2e-5 * max(1.0, 300 * float(P.pair_frequencies(rot).max()))
    if "scaling" in rot:
        assert abs(m - 1.0) > 0.05
        f_plain = P.pair_frequencies(dict(dims=n, base=rot["base"]))
        ratio = P.pair_frequencies(rot) / f_plain
        assert float(ratio.min()) < 0.99 and float(ratio.max()) <= 1.0        # some pair is slowed, none is sped up


# ---------------------------------------------------------------- latent attention
# heads, dim, rot_dim, vdim, kv_rank, q_rank, scale: sizes the tiled kernels take (five heads in a tile of 32 and
# values narrower than their tile; 34 heads over two tiles with a rotated part as wide as the rest) and sizes they
# do not (no 16-byte rows), which go the plain kernels' way
LATENT_SIZES = [(5, 24, 8, 40, 48, 20, 1.3), (34, 16, 16, 16, 32, 24, 2.0), (3, 6, 6, 10, 22, 14, 1.8)]


def latent_pair(sizes, dtype, seed):
    H, d, r, dv, R, Q, scale = sizes
    own = S.latent(H, d, r, dv, R, Q, base=3e3, scale=scale, scaling=S.Y1)
    lent = S.latent(H, d, r, dv, R, Q, base=3e3, scale=scale, scaling=S.Y1, kv_from=0)
    layers = [S.layer(own, None), S.layer(lent, None)]
    return layers, [mixer_of(layers, i, dtype, seed) for i in range(2)]


def plain_latent_pair(layers, weights, x, rounded):
    """Both layers over whole sequences: per layer and sequence the result, and the first layer's shares."""
    ref, shares = [[], []], []
    for xb in x:
        pos = torch.arange(xb.shape[0])
        h = xb.double()
        rows = P.latent_rows(weights[0], "l0.mix.", layers[0]["mixer"], h, pos, EPS)
        if rounded:
            rows = (bf(rows[0]).double(), bf(rows[1]).double())        # what a bfloat16 cache holds
        for i in range(2):
            sh = []
            ref[i].append(P.latent_attention(weights[i], f"l{i}.mix.", layers[i]["mixer"], h, pos, EPS, rows, sh))
            if i == 0:
                shares.append(sh)
    return ref, shares


@pytest.mark.parametrize("sizes", LATENT_SIZES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_with_sharp_scores(sizes, dtype):
    """Prompts from the first token, single tokens across page borders and past 256 positions, portions of two and
    three tokens and a long one behind cached rows, for three sequences at once; the second mixer has no rows of
    its own and reads the first's."""
    layers, built = latent_pair(sizes, dtype, 11)
    x = sharp_inputs(5)
    ref, shares = plain_latent_pair(layers, [b[1] for b in built], x, dtype == "bfloat16")
    check_sharpness(shares[0], "latent attention")
    row = sizes[4] + sizes[2]
    k = torch.zeros(N_PAGES, PAGE, row, dtype=DT[dtype], device=DEV)
    got = run_in_portions([b[0] for b in built], [(k, None, True), (k, None, False)], x, PORTIONS, dtype, LENS)
    for i in range(2):
        for b in range(len(LENS)):
            close(got[i][b], ref[i][b], dtype, f"latent layer {i}, sequence {b}", roundings=6.0 if dtype == "bfloat16" else 4.0)


@pytest.mark.parametrize("sizes", LATENT_SIZES[:2])
def test_latent_prompt_and_token_by_token_are_one_function(sizes):
    """The two forms of the kernel (heads materialised for a prompt; all heads over the cached rows otherwise) agree:
    a prompt at once against the same tokens one at a time."""
    layers, built = latent_pair(sizes, "bfloat16", 12)
    x = sharp_inputs(6, [150])
    row = sizes[4] + sizes[2]
    results = []
    for portions in ([[150]], [[1]] * 150, [[2]] * 75):
        k = torch.zeros(N_PAGES, PAGE, row, dtype=torch.bfloat16, device=DEV)
        results.append(run_in_portions([b[0] for b in built], [(k, None, True), (k, None, False)], x, portions, "bfloat16", [150]))
    for other in results[1:]:
        for i in range(2):
            close(other[i][0], results[0][i][0].double(), "bfloat16", f"latent layer {i} in single tokens", roundings=4.0)
