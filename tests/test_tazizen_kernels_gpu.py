"""The mechanisms Tazizen adds, each alone against the plain implementation's function for it: the pass over several
copies of the residual stream, the rotation followed by a unit norm per head, the softmax with one more key that has
no value in every attention kernel, the sliding window of latent attention in both of its forms, the choice of experts
among the best groups by corrected scores, the shared expert's gate.  Attention is run with scores sharp enough that
one key stands out for most queries, wherever it lies (far back, at a page border, at the window's edge, the query's
own position), so that a mask or a page one position off shows; prompts, portions and single tokens share the calls."""
import math

import pytest
import torch

import plain_tazizen as P
import tazizen_helpers as S
from test_parts_gpu import PAGE, Step, act, part, summed
from test_sobezen_kernels_gpu import LENS, N_PAGES, PORTIONS, WIDTH, bf, close, run_in_portions, sharp_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
EPS = 1e-5


def ops():
    from libllm_b200.csrc import ops as o
    return o


# ---------------------------------------------------------------- several copies of the residual stream
@pytest.mark.parametrize("S_,T,H,parts", [(1, 5, 48, 1), (2, 9, 64, 3), (3, 4, 50, 1), (4, 33, 256, 2), (5, 7, 72, 4), (8, 3, 2048, 1), (13, 6, 40, 2), (16, 2, 128, 1)])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_pass_over_the_copies_of_the_stream(S_, T, H, parts, out_dtype):
    """The pending result of one sublayer moves all copies, the next sublayer's input is joined and normed: in place;
    for chosen rows into a buffer of their own; from a stream whose copies are still all equal; and the plain sum."""
    o = ops()
    g = torch.Generator().manual_seed(S_ * 100 + T)
    r = lambda *s: torch.randn(*s, generator=g)
    x, delta = r(S_, T, H), r(parts, T, H)
    mix, outw, inw, nw = torch.eye(S_) + 0.3 * r(S_, S_), 1 + 0.3 * r(S_), 1.0 / S_ + 0.3 * r(S_), 1 + 0.2 * r(H)
    xs = [x[s].double() for s in range(S_)]
    w = {"in": inw.double(), "out": outw.double(), "mix": mix.double()}
    y = delta.double().sum(0)
    moved = [sum(w["mix"][s, t] * xs[s] for s in range(S_)) + w["out"][t] * y for t in range(S_)]
    joined = sum(w["in"][s] * moved[s] for s in range(S_))
    normed = P.unit_rms(joined, EPS) * nw.double()
    dev = lambda t: t.to(DEV).contiguous()
    # in place, with the norm
    xd, out = dev(x), torch.empty(T, H, dtype=DT[out_dtype], device=DEV)
    o.hyper_mix_norm(xd, dev(delta), dev(mix), dev(outw), dev(inw), dev(nw), EPS, out)
    close(xd.cpu(), torch.stack(moved), "float32", "the copies after the move")
    close(out.float().cpu(), normed, out_dtype, "joined and normed")
    # chosen rows, into a buffer of their own; the stream itself stays
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32)
    xd, few, out = dev(x), torch.zeros(S_, 3, H, device=DEV), torch.empty(3, H, dtype=DT[out_dtype], device=DEV)
    o.hyper_mix_norm(xd, dev(delta), dev(mix), dev(outw), dev(inw), dev(nw), EPS, out, rows=dev(rows), x_out=few)
    assert torch.equal(xd.cpu(), x)
    close(few.cpu(), torch.stack(moved)[:, rows.long()], "float32", "chosen rows of the copies")
    close(out.float().cpu(), normed[rows.long()], out_dtype, "chosen rows, joined and normed")
    # nothing pending, copies that are all equal to the first: they are written out, the join reads the first alone
    xd, out = dev(x), torch.empty(T, H, device=DEV)
    o.hyper_mix_norm(xd, None, None, None, dev(inw), None, 0.0, out, spread=False)
    close(xd.cpu(), x[:1].expand(S_, T, H), "float32", "copies spread from the first")
    close(out.cpu(), xs[0] * w["in"].sum(), "float32", "the join of equal copies")
    # the plain sum of the copies with the last result applied, no norm: what a model's last norm reads
    xd, out = dev(x), torch.empty(T, H, device=DEV)
    o.hyper_mix_norm(xd, dev(delta), dev(mix), dev(outw), None, None, 0.0, out)
    close(out.cpu(), sum(moved), "float32", "the sum of the copies")


def test_hyper_block_with_one_copy_and_unit_joins_is_the_prenorm_block():
    """in = out = mix = 1 and one copy: the block of kind "hyper" and the block of kind "prenorm" give the same stream."""
    c = S.config(64, 48, EPS, [S.layer(S.attn(3, 1, 16, 8, window=11), S.moe(4, 2, 24, shared=16))], streams=1)
    w = S.random_weights(c, 4)
    for k in list(w):
        if ".hc" in k:
            w[k] = torch.ones_like(w[k])
    toks = S.tokens(c, 30, 1)
    ref = P.forward(c, w, toks)
    plain_c = {k: v for k, v in c.items() if k != "streams"}
    close(P.forward(plain_c, {k: v for k, v in w.items() if ".hc" not in k}, toks), ref, "float32", "the plain functions agree")
    from libllm_b200.engine import Engine, StepItem
    for cfg, ws in ((c, w), (plain_c, {k: v for k, v in w.items() if ".hc" not in k})):
        e = Engine.from_tensors(cfg, ws, dtype="float32", max_tokens=128)
        s = e.open_sequence()
        got = torch.from_numpy(e.step([StepItem(s, toks, list(range(30)))]))
        S.check_rows(got, ref, "float32", "one copy with unit joins")


# ---------------------------------------------------------------- rotation, then a unit norm per head
@pytest.mark.parametrize("H,G,d,dv,rot", [(4, 2, 16, 16, 8), (3, 3, 12, 20, 12), (2, 1, 96, 40, 48), (1, 1, 256, 8, 2), (5, 1, 10, 6, 0)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_rotation_then_unit_heads(H, G, d, dv, rot, dtype):
    o = ops()
    g = torch.Generator().manual_seed(d)
    T, pad = 70, 5
    row = H * d + G * (d + dv)
    qkv = (torch.randn(T, row + pad, generator=g) * 3).to(DEV)
    r = S.rot(rot, 3e3, S.Y1) if rot else None
    table = None
    if rot:
        f, mag = P.frequencies(r)
        a = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
        table = torch.cat([torch.cos(a) * mag, torch.sin(a) * mag], -1).float().to(DEV)
    pos = torch.arange(130, 130 + T)
    step_pos = pos.to(torch.int32).to(DEV)
    tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    table_pages = torch.tensor([[7, 2, 5, 0]], dtype=torch.int32, device=DEV)
    kc = torch.zeros(8, G, PAGE, d, dtype=DT[dtype], device=DEV)
    vc = torch.zeros(8, G, PAGE, dv, dtype=DT[dtype], device=DEV)
    q_out = torch.empty(T, H * d, dtype=DT[dtype], device=DEV)
    o.rope_headnorm_place(qkv, q_out, H, G, d, dv, EPS, table, tok_seq, step_pos, table_pages, kc, vc, PAGE)
    x = qkv.cpu().double()
    q_ref = P.unit_rms(P.rotate_halves(x[:, :H * d].view(T, H, d), pos, r), EPS)
    k_ref = P.unit_rms(P.rotate_halves(x[:, H * d:H * d + G * d].view(T, G, d), pos, r), EPS)
    v_ref = x[:, H * d + G * d:row].view(T, G, dv)
    close(q_out.float().cpu().view(T, H, d), q_ref, dtype, "queries")
    pages = table_pages[0].cpu()[pos // PAGE]
    close(kc.float().cpu()[pages, :, pos % PAGE], k_ref, dtype, "keys in the cache")
    close(vc.float().cpu()[pages, :, pos % PAGE], v_ref, dtype, "values in the cache")


# ---------------------------------------------------------------- attention as the design has it, sharp scores
def mixer_of(layers, i, dtype, seed, max_positions=1024):
    from libllm_b200 import _lib
    c = S.config(64, WIDTH, EPS, layers, streams=2)
    spec = _lib.describe_model(c, dtype)["spec"]["layers"][i]["mixer"]
    w = {k: v for k, v in S.random_weights(c, seed).items() if k.startswith(f"l{i}.mix.")}
    m = part("mixer", spec, dtype, max_positions)
    m.load(w)
    return m, {k: v.double() for k, v in w.items()}, spec


# heads, key heads, head size, value size, rotated, window: the tiled kernels (64, 128; 32 with four query heads to a key
# head), sizes only the general kernel takes, windows shorter than a page, of a page, and over several
ATTENTION_SIZES = [(4, 2, 64, 64, 32, 100), (2, 2, 128, 128, 64, 65), (8, 2, 32, 32, 16, 64), (3, 1, 80, 80, 40, 150),
                   (2, 1, 24, 40, 12, 9), (3, 3, 16, 16, 0, None)]


@pytest.mark.parametrize("sizes", ATTENTION_SIZES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_with_unit_heads_a_key_without_value_window_and_gate(sizes, dtype):
    """Three sequences at once: prompts, single tokens across page borders and window edges, portions of two and three
    tokens, a long portion behind cached rows.  Unit heads make every score lie within +-scale * head size, so the
    scale sets how sharp the softmax is; the key without a value keeps its share wherever the real keys score low."""
    H, G, d, dv, rot, window = sizes
    layers = [S.layer(S.attn(H, G, d, rot, window=window, vdim=dv, base=3e3, scale=10.0 / d, scaling=S.Y1 if rot else None), None)]
    m, w, spec = mixer_of(layers, 0, dtype, 21)
    assert spec["head_norm"] == dict(eps=EPS) and spec["null_key"] == 0.0 and spec["out_gate"] == "l0.mix.g" and spec.get("window") == window
    x = sharp_inputs(9)
    ref = [P.attention(xb.double(), w, "l0.mix.", layers[0]["mixer"], EPS) for xb in x]
    k = torch.zeros(N_PAGES, G, PAGE, d, dtype=DT[dtype], device=DEV)
    v = torch.zeros(N_PAGES, G, PAGE, dv, dtype=DT[dtype], device=DEV)
    got = run_in_portions([m], [(k, v, True)], x, PORTIONS, dtype, LENS)
    for b in range(len(LENS)):
        close(got[0][b], ref[b], dtype, f"attention {sizes}, sequence {b}", roundings=6.0 if dtype == "bfloat16" else 4.0)


def test_the_key_without_value_takes_its_share():
    """Scores far below nought: almost all weight goes to the key that has no value, and the result shrinks by the
    factor the plain softmax gives; scores above nought: a small share."""
    for scale, sign in ((20.0 / 64, -1.0), (3.0 / 64, 1.0)):
        m = dict(heads=2, kv_heads=1, dim=64, scale=scale, mask=dict(size=50))
        T = 128
        g = torch.Generator().manual_seed(3)
        base = torch.randn(64, generator=g)
        q = (base[None, None, :] + 0.05 * torch.randn(T, 2, 64, generator=g))
        k = sign * (base[None, None, :] + 0.05 * torch.randn(T, 1, 64, generator=g))
        v = torch.randn(T, 1, 64, generator=g)
        qn, kn = P.unit_rms(q.double(), EPS), P.unit_rms(k.double(), EPS)
        see = P.visible(T, 50)
        ref = torch.stack([P.softmax_one_more((qn[:, a] @ kn[:, 0].T) * scale, see, 0.0) @ v[:, 0].double() for a in range(2)], 1)
        plain_ref = torch.stack([P.softmax_one_more((qn[:, a] @ kn[:, 0].T) * scale, see, None) @ v[:, 0].double() for a in range(2)], 1)
        ratio = float(ref.abs().mean() / plain_ref.abs().mean())
        assert ratio < 1e-6 if sign < 0 else 0.99 < ratio < 0.9999
        o = ops()
        for dtype in DTYPES:
            tdt = DT[dtype]
            kc = torch.zeros(4, 1, PAGE, 64, dtype=tdt, device=DEV)
            vc = torch.zeros_like(kc)
            kc[torch.arange(T) // PAGE, 0, torch.arange(T) % PAGE] = kn[:, 0].to(tdt).to(DEV)
            vc[torch.arange(T) // PAGE, 0, torch.arange(T) % PAGE] = v[:, 0].to(tdt).to(DEV)
            i32 = dict(dtype=torch.int32, device=DEV)
            qd = qn.reshape(T, 128).to(tdt).to(DEV)
            out = torch.empty(T, 128, dtype=tdt, device=DEV)
            table = torch.arange(4, **i32)[None]
            o.attention_generic(qd, out, kc, vc, torch.zeros(T, **i32), torch.arange(T, **i32), table, 2, 1, 64, PAGE, 50, scale, null_score=0.0)
            want = ref.reshape(T, 128)
            if sign > 0:
                close(out.float().cpu(), want, dtype, "general kernel", roundings=3.0)
            else:
                assert float((out.float().cpu() - want).abs().max()) < 1e-6
            if dtype != "bfloat16":
                continue
            start, past = torch.tensor([0, T], **i32), torch.zeros(1, **i32)
            for name, run in (("prompt kernel", lambda dst: o.attention_prefill(qd, dst, kc, vc, start, past, table, 1, T, 2, 1, 64, PAGE, 50, scale, null_score=0.0)),
                              ("tensor-core prompt kernel", lambda dst: o.attention_prefill_tc(qd, dst, kc, vc, start, past, table, 1, T, 2, 1, 64, PAGE, 50, scale, form=1, null_score=0.0)),
                              ("wide tensor-core prompt kernel", lambda dst: o.attention_prefill_tc(qd, dst, kc, vc, start, past, table, 1, T, 2, 1, 64, PAGE, 50, scale, form=2, null_score=0.0))):
                dst = torch.empty_like(out)
                run(dst)
                o.check_tc_status()
                if sign > 0:
                    close(dst.float().cpu(), want, dtype, name, roundings=3.0)
                else:
                    assert float((dst.float().cpu() - want).abs().max()) < 1e-6, name
            # the last token alone, its keys in one run and in two
            for n_splits in (1, 2):
                dst = torch.empty(1, 128, dtype=tdt, device=DEV)
                ws_o, ws_ml = torch.empty(2 * n_splits * 64, device=DEV), torch.empty(2 * n_splits * 2, device=DEV)
                o.attention_decode(qd[T - 1:], dst, kc, vc, torch.tensor([T - 1], **i32), table, 2, 1, 64, PAGE, 128 // n_splits, n_splits, 50, scale,
                                   ws_o, ws_ml, null_score=0.0)
                if sign > 0:
                    close(dst.float().cpu(), want[T - 1:], dtype, f"single-token kernel, {n_splits} runs", roundings=3.0)
                else:
                    assert float((dst.float().cpu() - want[T - 1:]).abs().max()) < 1e-6


# ---------------------------------------------------------------- latent attention with a window
# heads, unrotated, rotated, value size, kv_rank, q_rank, window: sizes the tensor-core forms take and sizes they do not
LATENT_SIZES = [(4, 32, 16, 32, 64, 48, 130), (5, 16, 8, 24, 48, 32, 64), (2, 16, 8, 16, 32, 24, 17), (3, 10, 6, 14, 40, 18, 70), (2, 24, 8, 40, 80, 20, None)]


@pytest.mark.parametrize("sizes", LATENT_SIZES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_with_a_window(sizes, dtype):
    H, d, r, dv, R, Q, window = sizes
    layers = [S.layer(S.latent(H, d, r, dv, R, Q, window=window, base=3e3, scale=2.5 / math.sqrt(d + r), scaling=S.Y1), None)]
    m, w, spec = mixer_of(layers, 0, dtype, 11)
    assert spec.get("window") == window and spec["position"]["pairing"] == "half"
    x = sharp_inputs(5)
    ref = [P.latent_attention(xb.double(), w, "l0.mix.", layers[0]["mixer"], EPS) for xb in x]
    k = torch.zeros(N_PAGES, PAGE, R + r, dtype=DT[dtype], device=DEV)
    got = run_in_portions([m], [(k, None, True)], x, PORTIONS, dtype, LENS)
    for b in range(len(LENS)):
        close(got[0][b], ref[b], dtype, f"latent attention {sizes}, sequence {b}", roundings=8.0 if dtype == "bfloat16" else 4.0)


@pytest.mark.parametrize("sizes", LATENT_SIZES[:2])
def test_latent_prompt_and_token_by_token_are_one_function(sizes):
    H, d, r, dv, R, Q, window = sizes
    layers = [S.layer(S.latent(H, d, r, dv, R, Q, window=window, base=3e3, scale=2.5 / math.sqrt(d + r)), None)]
    m, w, _ = mixer_of(layers, 0, "bfloat16", 12)
    x = sharp_inputs(6, [200])
    results = []
    for portions in ([[200]], [[1]] * 200, [[2]] * 100, [[150], [50]]):
        k = torch.zeros(N_PAGES, PAGE, R + r, dtype=torch.bfloat16, device=DEV)
        results.append(run_in_portions([m], [(k, None, True)], x, portions, "bfloat16", [200]))
    for other in results[1:]:
        close(other[0][0], results[0][0][0].double(), "bfloat16", "latent attention cut another way", roundings=4.0)


# ---------------------------------------------------------------- the choice of experts
@pytest.mark.parametrize("E,top,groups,scale", [(16, 3, (2, 1), 1.5), (8, 2, (4, 2), 2.5), (6, 3, (3, 2), 1.0), (12, 5, (3, 2), 0.5), (5, 1, None, 1.0),
                                                 (4, 4, (1, 1), 2.0), (64, 6, (8, 3), 1.0), (9, 2, (3, 1), 1.0), (6, 2, (6, 3), 1.0)])
def test_choice_among_the_best_groups_by_corrected_scores(E, top, groups, scale):
    o = ops()
    g = torch.Generator().manual_seed(E * 10 + top)
    T, W = 300, 32
    h = torch.randn(T, W, generator=g).double()
    w = {"router": torch.randn(E, W, generator=g).double() * 0.7, "correction": torch.randn(E, generator=g).double() * 0.4}
    r = dict(experts=E, top=top, scale=scale)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    chosen, weights, margin = P.route(h, w, "", r)
    logits = (h @ w["router"].T).float().to(DEV)
    got_c, got_w = o.moe_route_grouped(logits, top, w["correction"].float().to(DEV), groups[0] if groups else 1, groups[1] if groups else 1, 2,
                                       renormalize=True, norm_eps=1e-20, route_scale=scale)
    sure = margin > 1e-5
    assert int(sure.sum()) > T * 0.9
    assert torch.equal(got_c.cpu().long()[sure], chosen[sure]), "the chosen experts, in the order of their corrected scores"
    close(got_w.cpu()[sure], weights[sure], "float32", "weights")
    # corrections that push a whole group below nought must not bring it back: the others count as minus infinity
    if groups and groups[1] < groups[0]:
        low = w["correction"].clone()
        low[: E // groups[0]] -= 5.0
        c2, _, m2 = P.route(h, {**w, "correction": low}, "", r)
        g2, _ = o.moe_route_grouped(logits, top, low.float().to(DEV), groups[0], groups[1], 2, renormalize=True, norm_eps=1e-20, route_scale=scale)
        ok = m2 > 1e-5
        assert torch.equal(g2.cpu().long()[ok], c2[ok]) and int((g2.cpu() < E // groups[0]).sum()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("f", [S.moe(8, 2, 24, groups=(4, 2), scale=2.5, shared=48), S.moe(6, 3, 20, groups=(3, 2)), S.moe(16, 4, 32, groups=(4, 2), scale=1.5, shared=64),
                               S.moe(4, 4, 24, groups=(1, 1), scale=2.0, shared=16), S.moe(5, 1, 36)])
def test_routed_feed_forward_with_a_gated_shared_expert(f, dtype):
    from libllm_b200 import _lib
    c = S.config(64, WIDTH, EPS, [S.layer(S.attn(2, 1, 16, 8), f)], streams=2)
    spec = _lib.describe_model(c, dtype)["spec"]["layers"][0]["ff"]
    assert spec["norm_eps"] == 1e-20 and spec["route_scale"] == f["router"].get("scale", 1.0) and spec["correction"] == "l0.mlp.correction"
    assert ("shared_gate" in spec) == ("shared" in f) and spec["score"] == "sigmoid" and spec["renormalize"] is True
    w = {k: v for k, v in S.random_weights(c, 8).items() if k.startswith("l0.mlp.")}
    ff = part("feed_forward", spec, dtype)
    ff.load(w)
    for T in (1, 7, 200):
        g = torch.Generator().manual_seed(T)
        x = bf(torch.randn(T, WIDTH, generator=g))
        margins = []
        ref = P.experts(x.double(), {k: v.double() for k, v in w.items()}, "l0.mlp.", f, margins)
        out = summed(ff.forward(dict(step=Step([T], [0]).json, x=act(x.to(DT[dtype]).to(DEV))))["out"]).cpu()
        sure = margins[0] > (1e-4 if dtype == "float32" else 3e-2)
        if int(sure.sum()):
            close(out[sure], ref[sure], dtype, f"routed feed-forward, {T} tokens", roundings=4.0)
