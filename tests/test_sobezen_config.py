"""Sobezen's configuration, its description as parts, which run reads whose cache, and the faults it names: what
needs no GPU.  Also the plain implementation's small functions by hand."""
import copy
import math

import pytest
import torch

import plain_sobezen as P
import sobezen_helpers as S


def describe(c, dtype="bfloat16"):
    from libllm_b200 import _lib
    return _lib.describe_model(c, dtype)


@pytest.mark.parametrize("name", sorted(S.CONFIGS))
def test_tensors_asked_for_are_the_designs_names_and_shapes(name):
    c = S.CONFIGS[name]
    d = describe(c)
    want = S.tensor_shapes(c)                          # the ranks the configuration does not give are left open (-1)
    assert {t["name"]: t["shape"] for t in d["tensor_needs"]} == want
    roles = {t["name"]: t["role"] for t in d["tensor_needs"]}
    assert roles["l0.norm1"] == roles["l0.ls1"] == roles["final.norm"] == "vector"
    assert roles["embed"] == roles["head"] == roles["l0.mix.o"] == "matrix"
    assert d["capturable"]


@pytest.mark.parametrize("name", sorted(S.CONFIGS))
def test_every_layer_runs_once_and_borrowers_name_their_lender(name):
    c = S.CONFIGS[name]
    sched = describe(c)["spec"]["schedule"]
    assert [e["layer"] for e in sched] == list(range(len(c["layers"])))
    assert [e["cache_from"] for e in sched] == [L["mixer"].get("kv_from") for L in c["layers"]]
    assert all(e["input_mix"] is None for e in sched)


def test_every_constant_reaches_its_part():
    c = S.CONFIGS["B1"]
    spec = describe(c)["spec"]
    assert (spec["embedding"], spec["head"], spec["embedding_scale"], spec["logit_scale"], spec["logit_softcap"]) == ("embed", "head", 8.0, 0.5, 0.0)
    assert spec["position_table"] is None
    assert spec["final_norm"] == dict(kind="rmsnorm", size=64, eps=1e-6, weight="final.norm")
    L = spec["layers"]
    assert all(b["kind"] == "prenorm" and b["mixer_scale"] == f"l{i}.ls1" for i, b in enumerate(L))
    assert L[0]["ff_scale"] == "l0.ls2" and L[1]["ff"] is None and L[1]["ff_norm"] is None and "ff_scale" not in L[1]
    d = L[0]["mixer"]
    assert (d["kind"], d["n_heads"], d["n_kv_heads"], d["head_dim"], d["v_head_dim"], d["taps"]) == ("channel_delta", 4, 2, 16, 24, 3)
    assert (d["eps"], d["key_eps"], d["A_log"], d["dt_bias"], d["q_conv"]) == (1e-6, 1e-6, "l0.mix.A_log", "l0.mix.dt_bias", "l0.mix.q.conv")
    f = L[0]["ff"]
    assert (f["kind"], f["intermediate"], f["limit"], f["slope"], f["up_shift"]) == ("clamped_glu", 96, 1.5, 1.702, 1.0)
    assert (f["gate_bias"], f["up_bias"], f["down_bias"]) == ("l0.mlp.gate.b", "l0.mlp.up.b", "l0.mlp.down.b")
    a = L[1]["mixer"]
    assert (a["kind"], a["n_heads"], a["n_kv_heads"], a["head_dim"], a["scale"], a["values"], a["bias"]) == ("attention", 4, 1, 32, 0.2, "keys", True)
    assert "v" not in a and a["q_bias"] == "l1.mix.q.b" and a["k_bias"] == "l1.mix.k.b"
    assert a["position"] == dict(kind="rope", head_dim=32, rotary_dim=16, theta=10000.0, pairing="interleaved", scaling=None)
    m = L[2]["mixer"]
    assert (m["kind"], m["n_heads"], m["head_dim"], m["rot_dim"], m["v_head_dim"], m["kv_rank"], m["q_rank"], m["scale"], m["eps"]) == \
        ("latent_attention", 2, 24, 8, 40, 48, 20, 0.15, 1e-6)
    y = m["position"]["scaling"]
    assert (m["position"]["head_dim"], m["position"]["rotary_dim"], m["position"]["theta"]) == (8, 8, 5e4)
    assert (y["rope_type"], y["factor"], y["original_max_position_embeddings"], y["beta_fast"], y["beta_slow"]) == ("yarn", 4.0, 64, 8.0, 1.0)
    assert abs(y["magnitude"] - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert m["kv_down"] == "l2.mix.dkv" and m["kv_norm"] == "l2.mix.dkv.norm"
    assert "kv_down" not in L[4]["mixer"] and "kv_norm" not in L[4]["mixer"]
    # what the configuration leaves out: no scales, as many key heads as heads, values as wide as keys
    bare = copy.deepcopy(S.CONFIGS["B2"])
    for k in ("kv_heads", "vdim"):
        del bare["layers"][3]["mixer"][k]
    sb = describe(bare)["spec"]
    assert (sb["embedding_scale"], sb["logit_scale"]) == (1.0, 1.0)
    assert (sb["layers"][3]["mixer"]["n_kv_heads"], sb["layers"][3]["mixer"]["v_head_dim"]) == (3, 24)


@pytest.mark.parametrize("change, says", [
    (lambda c: c["layers"][0].update(type="conv_mixer"), "is not known"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=4), "earlier layer"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=1), "latent_attention layer"),
    (lambda c: c["layers"][4]["mixer"].update(kv_rank=40), "another 'kv_rank'"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=6), "must equal 'rot_dim'"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34), "at most"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=16), "values are the keys"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "is not known"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "at least one layer"),
])
def test_faults_are_named(change, says):
    from libllm_b200.errors import ConfigError
    c = copy.deepcopy(S.CONFIGS["B1"])
    change(c)
    with pytest.raises(ConfigError) as e:
        describe(c)
    assert says in str(e.value)


def test_a_borrower_of_a_borrower_is_refused():
    from libllm_b200.errors import ConfigError
    c = copy.deepcopy(S.CONFIGS["B2"])
    c["layers"][4]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError):
        describe(c)


# ---------------------------------------------------------------- the plain functions by hand
def test_pair_frequencies_by_hand():
    f = P.pair_frequencies(dict(dims=4, base=100.0))
    assert torch.allclose(f, torch.tensor([1.0, 0.1], dtype=torch.float64))
    # 8 channels, base 5e4, original 64: the ramp starts at pair 0 and is full from pair 1 on
    r = dict(dims=8, base=5e4, scaling=dict(factor=4.0, original=64, fast=8.0, slow=1.0))
    plain = [5e4 ** (-2.0 * i / 8) for i in range(4)]
    assert torch.allclose(P.pair_frequencies(r), torch.tensor([plain[0], plain[1] / 4, plain[2] / 4, plain[3] / 4], dtype=torch.float64))
    assert abs(P.table_magnitude(r) - 1.1386294361119891) < 1e-15 and P.table_magnitude(dict(dims=4, base=10.0)) == 1.0
    # a ramp in the middle: 16 channels, base 3e4: pairs 0, 1, 2.. get 0, 1/2, 1
    r = dict(dims=16, base=3e4, scaling=dict(factor=4.0, original=64, fast=8.0, slow=1.0))
    f0 = [3e4 ** (-2.0 * i / 16) for i in range(8)]
    want = [f0[0], f0[1] / 4 * 0.5 + f0[1] * 0.5] + [x / 4 for x in f0[2:]]
    assert torch.allclose(P.pair_frequencies(r), torch.tensor(want, dtype=torch.float64))


def test_rotation_turns_neighbours_and_leaves_the_rest():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]]], dtype=torch.float64)
    out = P.rotate_pairs(x, torch.tensor([3]), dict(dims=4, base=100.0))
    c0, s0, c1, s1 = math.cos(3.0), math.sin(3.0), math.cos(0.3), math.sin(0.3)
    assert torch.allclose(out[0, 0], torch.tensor([c0, s0, -2 * s1, 2 * c1, 5.0, 6.0], dtype=torch.float64))


def test_short_conv_by_hand():
    x = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    w = torch.tensor([[10.0, 100.0, 1.0]], dtype=torch.float64)
    assert P.short_conv(x, w).flatten().tolist() == [1.0, 102.0, 213.0]
    before = torch.tensor([[7.0], [8.0]], dtype=torch.float64)
    assert P.short_conv(x, w, before).flatten().tolist() == [871.0, 182.0, 213.0]


def test_delta_steps_by_hand():
    """One head, two key channels, one value channel: the decay acts on the rows of the key channels, the write
    removes what the decayed state already answers, the read-out sees the write."""
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]], dtype=torch.float64)
    k = torch.tensor([[[1.0, 0.0]], [[1.0, 1.0]]], dtype=torch.float64)
    v = torch.tensor([[[2.0]], [[3.0]]], dtype=torch.float64)
    beta = torch.tensor([[0.5], [1.0]], dtype=torch.float64)
    g = torch.tensor([[[0.9, 0.8]], [[0.5, 0.25]]], dtype=torch.float64)
    o, S_ = P.delta_steps(q, k, v, beta, g)
    # token 0: S = [[1], [0]], o = 1.  token 1: S <- [[.5], [0]]; u = 3 - .5 = 2.5; S = [[3], [2.5]]; o = 2.5
    assert o.flatten().tolist() == [1.0, 2.5] and S_.flatten().tolist() == [3.0, 2.5]


def test_clamped_unit_by_hand():
    w = {"gate": torch.tensor([[1.0], [1.0]]), "gate.b": torch.tensor([5.0, -1.0]), "up": torch.tensor([[1.0], [-1.0]]),
         "up.b": torch.tensor([0.0, -9.0]), "down": torch.tensor([[1.0, 10.0]]), "down.b": torch.tensor([0.25])}
    w = {k: v.double() for k, v in w.items()}
    y = P.clamped_unit(w, "", dict(limit=2.0), torch.tensor([[0.5]], dtype=torch.float64))
    g0, g1 = 2.0, -0.5                                  # 5.5 is cut to the limit from above only; -0.5 stays
    u0, u1 = 0.5, -2.0                                  # -9.5 is cut to -limit
    want = g0 / (1 + math.exp(-1.702 * g0)) * (u0 + 1) + 10 * g1 / (1 + math.exp(-1.702 * g1)) * (u1 + 1) + 0.25
    assert abs(float(y) - want) < 1e-12
