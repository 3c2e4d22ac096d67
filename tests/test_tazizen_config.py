"""Tazizen's configuration, its description as parts, the order of its runs, the cache's books for its windows, and the
faults it names: what needs no GPU.  Also the plain implementation's small functions by hand."""
import copy
import math

import pytest
import torch

import plain_tazizen as P
import tazizen_helpers as S


def describe(c, dtype="bfloat16"):
    from libllm_b200 import _lib
    return _lib.describe_model(c, dtype)


@pytest.mark.parametrize("name", sorted(S.CONFIGS))
def test_tensors_asked_for_are_the_designs_names_and_shapes(name):
    c = S.CONFIGS[name]
    d = describe(c)
    assert {t["name"]: t["shape"] for t in d["tensor_needs"]} == S.tensor_shapes(c)
    roles = {t["name"]: t["role"] for t in d["tensor_needs"]}
    assert roles["l0.norm1"] == roles["final.norm"] == "vector" and roles["embed"] == roles["head"] == roles["l0.mix.o"] == "matrix"
    if "streams" in c:
        assert roles["l0.hc1.in"] == roles["l0.hc1.mix"] == "vector"        # 32-bit, whatever the engine's type
    assert d["capturable"]


@pytest.mark.parametrize("name", sorted(S.CONFIGS))
def test_looped_layers_run_in_a_row_each_with_a_cache_of_its_own(name):
    c = S.CONFIGS[name]
    sched = describe(c)["spec"]["schedule"]
    assert [e["layer"] for e in sched] == P.order_of_runs(c)
    assert all(e["cache_from"] is None and e["input_mix"] is None for e in sched)


def test_the_order_of_runs_by_hand():
    c = S.config(10, 8, 1e-5, [S.layer(S.attn(1, 1, 8, 2), None)] * 5, loop=(1, 3, 3))
    assert P.order_of_runs(c) == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert [e["layer"] for e in describe(c)["spec"]["schedule"]] == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    c["loop"] = dict(start=0, stop=5, times=2)
    assert [e["layer"] for e in describe(c)["spec"]["schedule"]] == list(range(5)) * 2
    c["loop"] = dict(start=2, stop=2, times=4)
    assert [e["layer"] for e in describe(c)["spec"]["schedule"]] == list(range(5))
    del c["loop"]
    assert [e["layer"] for e in describe(c)["spec"]["schedule"]] == list(range(5))


def test_every_constant_reaches_its_part():
    c = S.CONFIGS["T1"]
    spec = describe(c)["spec"]
    assert (spec["embedding"], spec["head"], spec["streams"], spec["embedding_scale"], spec["logit_scale"]) == ("embed", "head", 2, 1.0, 1.0)
    assert spec["final_norm"] == dict(kind="rmsnorm", size=64, eps=1e-6, weight="final.norm", weight_offset=1.0)
    L = spec["layers"]
    assert all(b["kind"] == "hyper" and b["streams"] == 2 and b["mixer_in"] == f"l{i}.hc1.in" and b["mixer_mix"] == f"l{i}.hc1.mix"
               for i, b in enumerate(L))
    assert L[0]["ff_out"] == "l0.hc2.out" and L[1]["ff"] is None and L[1]["ff_norm"] is None and "ff_in" not in L[1]
    assert L[0]["mixer_norm"]["weight_offset"] == 1.0 and L[0]["ff_norm"]["weight"] == "l0.norm2"
    a = L[0]["mixer"]
    assert (a["kind"], a["n_heads"], a["n_kv_heads"], a["head_dim"], a["v_head_dim"], a["scale"], a["window"]) == ("attention", 4, 2, 16, 16, 0.375, 24)
    assert a["head_norm"] == dict(eps=1e-6) and a["null_key"] == 0.0 and a["out_gate"] == "l0.mix.g" and a["v"] == "l0.mix.v"
    assert a["position"] == dict(kind="rope", head_dim=16, rotary_dim=8, theta=10000.0, pairing="half",
                                 scaling=dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=64.0, beta_fast=8.0, beta_slow=1.0,
                                              magnitude=0.1 * math.log(4.0) + 1.0))
    m = L[1]["mixer"]
    assert (m["kind"], m["n_heads"], m["head_dim"], m["rot_dim"], m["v_head_dim"], m["kv_rank"], m["q_rank"], m["eps"], m["window"]) == \
        ("latent_attention", 2, 16, 8, 16, 32, 24, 1e-6, 17)
    assert m["position"]["scaling"] is None and m["position"]["pairing"] == "half" and m["kv_down"] == "l1.mix.dkv"
    assert L[2]["mixer"]["v_head_dim"] == 24
    f = L[0]["ff"]
    assert (f["kind"], f["experts"], f["top"], f["score"], f["renormalize"], f["norm_eps"], f["route_scale"], f["weight_on"]) == \
        ("moe", 8, 2, "sigmoid", True, 1e-20, 2.5, "output")
    assert f["groups"] == dict(count=4, keep=2, top=2) and f["correction"] == "l0.mlp.correction" and f["shared_gate"] == "l0.mlp.shared.sg"
    assert f["expert"] == dict(intermediate=24, activation="silu", gate="l0.mlp.e{}.gate", up="l0.mlp.e{}.up", down="l0.mlp.e{}.down")
    assert f["shared"] == dict(kind="swiglu", hidden=64, intermediate=48, gate="l0.mlp.shared.gate", up="l0.mlp.shared.up", down="l0.mlp.shared.down")
    g = L[2]["ff"]
    assert "shared" not in g and "shared_gate" not in g and g["route_scale"] == 0.7
    # what the configuration leaves out
    t4 = describe(S.CONFIGS["T4"])["spec"]
    assert t4["streams"] == 1 and all(b["kind"] == "prenorm" for b in t4["layers"])
    assert t4["layers"][0]["mixer"]["position"] is None and "window" not in t4["layers"][0]["mixer"] and t4["layers"][0]["mixer"]["n_kv_heads"] == 3
    assert "groups" not in t4["layers"][1]["ff"] and t4["layers"][1]["ff"]["route_scale"] == 1.0


def test_faults_are_named():
    from libllm_b200.errors import ConfigError
    base = S.CONFIGS["T1"]

    def broken(change, match):
        c = copy.deepcopy(base)
        change(c)
        with pytest.raises(ConfigError, match=match):
            describe(c)

    broken(lambda c: c["layers"][0].update(type="conv"), "not known")
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of 'kv_heads'")
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "'dims'")
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "must equal 'rot_dim'")
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "'top' exceeds")
    broken(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "divide")
    broken(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=5), "'keep' exceeds")
    broken(lambda c: c["layers"][2]["mlp"]["router"].update(top=3), "fewer experts than 'top'")
    broken(lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not known")
    broken(lambda c: c["loop"].update(stop=4), "'start' <= 'stop'")
    broken(lambda c: c.pop("norm"), "norm")
    broken(lambda c: c.update(streams=0), "streams")
    broken(lambda c: c["layers"][0]["mixer"].pop("dim"), "dim")


def test_a_mixer_without_a_scale_takes_the_usual_one():
    c = copy.deepcopy(S.CONFIGS["T1"])
    del c["layers"][0]["mixer"]["scale"], c["layers"][1]["mixer"]["scale"]
    L = describe(c)["spec"]["layers"]
    assert L[0]["mixer"]["scale"] == 16 ** -0.5 and abs(L[1]["mixer"]["scale"] - 24 ** -0.5) < 1e-15


def test_the_caches_books_for_windows_of_looped_runs():
    """The runs of T1 (a loop of two layers run twice): runs with the same need share a group; a windowed group gives
    back the pages behind the window, for the latent rows (one key head, no values) as for keys and values."""
    from libllm_b200.cache import CacheBook
    attention = lambda w, d, dv, g: dict(kind="window", window=w, n_kv_heads=g, k_dim=d, v_dim=dv)
    rows = dict(kind="window", window=17, n_kv_heads=1, k_dim=40, v_dim=0)
    book = CacheBook([attention(24, 16, 16, 2), rows, attention(70, 32, 24, 1), rows, attention(70, 32, 24, 1)], capacity_tokens=64 * 8)
    by_runs = {tuple(g["runs"]): g for g in book.info()["groups"]}
    assert set(by_runs) == {(0,), (1, 3), (2, 4)}
    assert (by_runs[(1, 3)]["kind"], by_runs[(1, 3)]["window"], by_runs[(1, 3)]["k_dim"], by_runs[(1, 3)]["v_dim"]) == ("window", 17, 40, 0)
    slot = book.open()
    for n in (1, 17, 18, 64, 65, 80, 81, 134, 200, 330):
        book.reserve({slot: n})
        book.commit(slot, n)
        pages = book.info()["sequences"][str(slot)]["pages"]
        for g in book.info()["groups"]:
            first = max(0, n - g["window"] + 1) // 64
            index = book.info()["groups"].index(g)
            assert [p >= 0 for p in pages[index]] == [j >= first for j in range((n + 63) // 64)], (n, g["runs"])
        book.check()
    book.close(slot)
    assert all(g["pages_in_use"] == 0 for g in book.info()["groups"])


# ---------------------------------------------------------------- the plain functions by hand
def test_norm_around_zero_and_unit_rms():
    x = torch.tensor([[3.0, -4.0]], dtype=torch.float64)
    assert torch.allclose(P.unit_rms(x, 0.5), x / math.sqrt(12.5 + 0.5))
    assert torch.allclose(P.norm_around_zero(x, torch.tensor([0.5, -1.0], dtype=torch.float64), 0.5), torch.tensor([[1.5 * 3 / math.sqrt(13), 0.0]], dtype=torch.float64))


def test_rotation_pairs_channel_i_with_i_plus_half():
    rot = S.rot(4, 100.0)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 9.0]]], dtype=torch.float64)
    y = P.rotate_halves(x, torch.tensor([2]), rot)[0, 0]
    a0, a1 = 2 * 1.0, 2 * 100.0 ** -0.5
    assert torch.allclose(y, torch.tensor([math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                           3 * math.cos(a0) + math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 9.0], dtype=torch.float64))
    f, mag = P.frequencies(S.rot(8, 1e4, (4.0, 64, 8.0, 1.0)))
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-12 and torch.all(f[1:] < f[:-1])
    plain_f, _ = P.frequencies(S.rot(8, 1e4))
    assert torch.all(f <= plain_f + 1e-15) and torch.all(f >= plain_f / 4.0 - 1e-15)


def test_window_and_one_more_key():
    see = P.visible(5, 2)
    assert see.tolist() == [[True, False, False, False, False], [True, True, False, False, False], [False, True, True, False, False],
                            [False, False, True, True, False], [False, False, False, True, True]]
    s = torch.zeros(2, 2, dtype=torch.float64)
    p = P.softmax_one_more(s, torch.tensor([[True, False], [True, True]]), 0.0)
    assert torch.allclose(p, torch.tensor([[0.5, 0.0], [1 / 3, 1 / 3]], dtype=torch.float64))
    assert torch.allclose(P.softmax_one_more(s, torch.tensor([[True, False], [True, True]]), None), torch.tensor([[1.0, 0.0], [0.5, 0.5]], dtype=torch.float64))


def test_route_by_hand():
    # four experts in two groups of which one is kept; the correction decides the group, the weights ignore it
    w = {"router": torch.eye(4, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 2.0, -3.0], dtype=torch.float64)}
    h = torch.tensor([[2.0, 1.0, -1.0, 0.0]], dtype=torch.float64)
    s = torch.sigmoid(h[0])
    chosen, weights, _ = P.route(h, w, "", dict(experts=4, top=2, scale=3.0, groups=dict(count=2, keep=1)))
    # group scores: s0 + s1 = 1.61 against (s2 + 2) + (s3 - 3) = -0.23: the first group
    assert chosen.tolist() == [[0, 1]]
    assert torch.allclose(weights[0], 3.0 * s[:2] / s[:2].sum())
    chosen, _, _ = P.route(h, w, "", dict(experts=4, top=2))
    assert chosen.tolist() == [[2, 0]]                          # without groups: s2 + 2 is the largest corrected score
    w["correction"][3] = 0.5
    chosen, weights, _ = P.route(h, w, "", dict(experts=4, top=2, groups=dict(count=2, keep=1)))
    assert chosen.tolist() == [[2, 3]] and torch.allclose(weights[0], s[2:] / s[2:].sum())


def test_join_of_streams_by_hand():
    xs = [torch.tensor([[1.0, 0.0]], dtype=torch.float64), torch.tensor([[0.0, 2.0]], dtype=torch.float64)]
    w = {"in": torch.tensor([2.0, -1.0], dtype=torch.float64), "out": torch.tensor([1.0, 10.0], dtype=torch.float64),
         "mix": torch.tensor([[1.0, 3.0], [0.5, 1.0]], dtype=torch.float64)}
    seen = []
    out = P.join_streams(xs, lambda u: (seen.append(u.clone()), u * 0 + 1.0)[1], w, "")
    assert seen[0].tolist() == [[2.0, -2.0]]
    assert out[0].tolist() == [[1.0 + 1.0, 1.0 + 1.0]] and out[1].tolist() == [[3.0 + 10.0, 2.0 + 10.0]]
