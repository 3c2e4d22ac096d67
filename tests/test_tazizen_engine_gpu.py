"""The Tazizen decoder through the engine (its step function, cache and scheduler) against the plain implementation,
in float32 and bfloat16, for every way of cutting the work: whole prompts, prompts then single tokens, portions of
prompts down to two tokens, unequal batches, pages and slots used again, long decoding across page borders and
window edges, the first tokens, other sizes, and greedy generation."""
import copy

import pytest
import torch

import plain_tazizen as P
import tazizen_helpers as S
from libllm_b200.engine import GREEDY, StepItem
from replay import replay_batch

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = sorted(S.CONFIGS)
_engines, _refs = {}, {}


def setup(name, dtype, max_tokens=4096, **kw):
    from libllm_b200.engine import Engine
    key = (name, dtype, max_tokens, tuple(sorted(kw.items())))
    if key not in _engines:
        c = S.CONFIGS[name]
        w = S.random_weights(c, seed=len(name) + ord(name[-1]), steady_choice=dtype == "bfloat16")
        _engines[key] = (Engine.from_tensors(c, w, dtype=dtype, max_tokens=max_tokens, **kw), c, w)
    return _engines[key]


def plain(name, c, w, toks):
    """-> logits, and per position the smallest margin of any router's choice"""
    key = (name, tuple(toks), float(w["final.norm"].sum() + sum(v.sum() for k, v in w.items() if k.endswith("correction"))))
    if key not in _refs:
        margins = []
        logits = P.forward(c, w, toks, margins=margins)
        _refs[key] = (logits, torch.stack(margins).min(0).values if margins else None)
    return _refs[key]


def compare(got, name, c, w, toks, dtype, what, rows=None):
    ref, margin = plain(name, c, w, toks)
    if rows is not None:
        ref, margin = ref[rows], margin[rows] if margin is not None else None
    S.check_rows(got, ref, dtype, what, margin)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(name, dtype):
    """Lengths from one token on, around the windows (9 to 150) and the page border (64)."""
    engine, c, w = setup(name, dtype)
    for i, n in enumerate([1, 2, 3, 9, 10, 17, 18, 25, 63, 64, 65, 71, 101, 131, 203]):
        toks = S.tokens(c, n, i)
        got = replay_batch(engine, [("r", toks, n)])["r"]
        compare(got, name, c, w, toks, dtype, f"{name} whole {n}")
    assert engine.pages_in_use() == [0] * len(engine.pages_in_use())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_models_cut_after_every_layer(name, dtype):
    """Models cut after 1, 2, .. layers (a loop keeps what is left of it) give the logits of the plain model cut at
    the same place: a fault shows at the first layer that has it."""
    from libllm_b200.engine import Engine
    c_full = S.CONFIGS[name]
    w_full = S.random_weights(c_full, seed=3, steady_choice=dtype == "bfloat16")
    toks = S.tokens(c_full, 90, 4)
    for n in range(1, len(c_full["layers"])):
        c = copy.deepcopy(c_full)
        c["layers"] = c["layers"][:n]
        if "loop" in c:
            c["loop"]["start"], c["loop"]["stop"] = min(c["loop"]["start"], n), min(c["loop"]["stop"], n)
        keep = tuple(f"l{i}." for i in range(n))
        w = {k: v for k, v in w_full.items() if not k.startswith("l") or k.startswith(keep)}
        engine = Engine.from_tensors(c, w, dtype=dtype, max_tokens=256)
        got = replay_batch(engine, [("r", toks, 60)])["r"]
        margins = []
        ref = P.forward(c, w, toks, margins=margins)
        S.check_rows(got, ref, dtype, f"{name}: the first {n} layers", torch.stack(margins).min(0).values if margins else None)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens_agrees_with_the_whole_prompt(name, dtype):
    """The same request as one prompt and as a prompt followed by single tokens, which pass page borders and carry every
    window over decoded tokens; also from a one-token prompt on."""
    engine, c, w = setup(name, dtype)
    for i, (n, n_prompt) in enumerate([(180, 100), (75, 35), (48, 1)]):
        toks = S.tokens(c, n, 20 + i)
        got = replay_batch(engine, [("r", toks, n_prompt)])["r"]
        compare(got, name, c, w, toks, dtype, f"{name} {n_prompt} + {n - n_prompt} single tokens")
        if dtype == "float32":
            whole = replay_batch(engine, [("r", toks, n)])["r"]
            S.check_rows(got, whole, dtype, f"{name}: decoding against the whole prompt", plain(name, c, w, toks)[1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_a_prompt(name, dtype):
    """A prompt brought in portions of several sizes, down to two tokens and one: a portion's first tokens look back
    into cached rows through every window."""
    engine, c, w = setup(name, dtype)
    toks = S.tokens(c, 212, 31)
    for sizes in ([64, 64, 64, 20], [2] * 20 + [57, 3, 100, 12], [7, 1, 42, 50, 2, 26, 70, 14], [1, 1, 1, 2, 1, 3, 203]):
        assert sum(sizes) == len(toks)
        slot = engine.open_sequence()
        rows, at = [], 0
        for n in sizes:
            rows.append(torch.from_numpy(engine.step([StepItem(slot, toks[at:at + n], list(range(n)))])))
            at += n
        engine.close_sequence(slot)
        compare(torch.cat(rows), name, c, w, toks, dtype, f"{name} portions {sizes[:4]}...")
    engine.cache_check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_against_each_request_alone(name, dtype):
    """Three batches of unequal requests on a cache that holds one batch at a time, so that pages and slots are used
    again; shorter requests end earlier; each request against the plain implementation and, in float32, against
    itself alone."""
    prompts, n_dec = [1, 70, 9, 131], 12
    cap = sum((p + n_dec + 4 + 63) // 64 * 64 for p in prompts)
    engine, c, w = setup(name, dtype, max_tokens=cap)
    alone, _, _ = setup(name, dtype)
    for b in range(3):
        reqs = []
        for j, p in enumerate(prompts):
            total = p + n_dec - (j if b % 2 == 0 else 3 - j)
            reqs.append((f"b{b}r{j}", S.tokens(c, total, 100 * b + j), p))
        got = replay_batch(engine, reqs)
        for rid, toks, p in reqs:
            compare(got[rid], name, c, w, toks, dtype, f"{name} batch {b} {rid}")
            if dtype == "float32" and b == 0:
                single = replay_batch(alone, [(rid, toks, p)])[rid]
                S.check_rows(got[rid], single, dtype, f"{name} {rid}: the batch changes the result", plain(name, c, w, toks)[1])
    assert engine.pages_in_use() == [0] * len(engine.pages_in_use())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["T1", "T3", "T5", "T6"])
def test_long_decoding(name, dtype):
    """One token a step for 330 steps: pages are taken as the rows grow over five page borders and given back as they
    leave the windows."""
    engine, c, w = setup(name, dtype)
    toks = S.tokens(c, 330, 77)
    got = replay_batch(engine, [("r", toks, 2)])["r"]
    compare(got, name, c, w, toks, dtype, f"{name} long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_beside_a_long_neighbour(dtype):
    engine, c, w = setup("T1", dtype)
    short, long_ = S.tokens(c, 3, 5), S.tokens(c, 90, 6)
    both = replay_batch(engine, [("l", long_, 60), ("s", short, 1)])
    compare(both["s"], "T1", c, w, short, dtype, "first tokens beside a long request")
    compare(both["l"], "T1", c, w, long_, dtype, "long neighbour")


@pytest.mark.parametrize("name", NAMES)
def test_what_the_cache_holds(name):
    """Every run of a looped layer has pages of its own; a latent layer holds one key head of kv_rank + rot_dim channels
    and no values, attention its heads with values of their own width; a window gives pages back."""
    engine, c, w = setup(name, "float32")
    slot = engine.open_sequence()
    engine.step([StepItem(slot, S.tokens(c, 330, 3), [329])])
    groups = engine.cache_info()["groups"]
    order = P.order_of_runs(c)
    assert sorted(r for g in groups for r in g["runs"]) == list(range(len(order)))
    for g in groups:
        held = set()
        for r in g["runs"]:
            L = c["layers"][order[r]]
            m = L["mixer"]
            if L["type"] == "latent_attention":
                assert (g["n_kv_heads"], g["k_dim"], g["v_dim"]) == (1, m["kv_rank"] + m["rot_dim"], 0), g
            else:
                assert (g["n_kv_heads"], g["k_dim"], g["v_dim"]) == (m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])), g
            window = (m.get("mask") or {}).get("size")
            assert g["window"] == window
            # after 330 tokens: the pages that hold positions 330 - window + 1 .. 329
            held.add(6 if not window else 330 // 64 - (330 - window + 1) // 64 + 1)
        n = held.pop()
        assert not held and g["pages_in_use"] in (n, n * len(g["runs"])), g
    engine.close_sequence(slot)
    engine.cache_check()
    assert engine.pages_in_use() == [0] * len(engine.pages_in_use())


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_cut_into_launch_sequences(dtype):
    """max_step_tokens below the prompts' lengths: the engine itself cuts inside a prompt."""
    engine, c, w = setup("T2", dtype, max_step_tokens=48)
    reqs = [("a", S.tokens(c, 150, 1), 150), ("b", S.tokens(c, 30, 2), 30)]
    got = replay_batch(engine, reqs)
    for rid, toks, _ in reqs:
        compare(got[rid], "T2", c, w, toks, dtype, f"cut {rid}")


@pytest.mark.parametrize("name", NAMES)
def test_the_last_row_alone(name):
    """A prompt of which only some places are wanted (the last layer then runs its feed-forward for those rows
    alone), and a portion of which nothing is wanted (its cache still moves on)."""
    engine, c, w = setup(name, "float32")
    toks = S.tokens(c, 77, 9)
    slot = engine.open_sequence()
    assert engine.step([StepItem(slot, toks[:40], [])]).shape[0] == 0
    got = torch.from_numpy(engine.step([StepItem(slot, toks[40:], [36, 0])]))
    engine.close_sequence(slot)
    compare(got, name, c, w, toks, "float32", f"{name} chosen rows", rows=[76, 40])


@pytest.mark.parametrize("name", ["T1", "T3", "T5"])
def test_greedy_generation_through_the_generation_loop(name):
    """engine.generate (scheduler, sampling, stop rule) in float32 against the plain implementation's own greedy
    loop, for prompts of unequal lengths in one call."""
    engine, c, w = setup(name, "float32")
    prompts = [S.tokens(c, n, 50 + n) for n in (5, 23, 1)]
    out = engine.generate(prompts, max_new_tokens=[10, 6, 12], sampling=GREEDY, stop_tokens=[])
    for p, got, n in zip(prompts, out, (10, 6, 12)):
        seq = list(p)
        for _ in range(n):
            logits = P.forward(c, w, seq)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < 1e-3:        # a close call is no test of anything
                break
            seq.append(int(logits.argmax()))
        want = seq[len(p):]
        assert got[:len(want)] == want, f"{name}: generated {got}, the plain loop {want}"
        assert len(got) == n


def tazizen_folder(tmp_path, name, seed, steady_choice=False):
    import json
    from helpers import write_safetensors
    c = S.CONFIGS[name]
    w = S.random_weights(c, seed, steady_choice)
    (tmp_path / "config.json").write_text(json.dumps(c))
    write_safetensors(str(tmp_path / "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in w.items()})
    return str(tmp_path), c, w


def test_the_model_folder_route_names_what_does_not_fit(tmp_path):
    """Weights written as a safetensors file and loaded by folder give the engine that tensors in memory give; an
    unexpected or missing tensor is named."""
    from libllm_b200.engine import Engine
    from libllm_b200.errors import WeightsError
    folder, c, w = tazizen_folder(tmp_path, "T2", 3)
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=256)
    toks = S.tokens(c, 40, 1)
    compare(replay_batch(engine, [("r", toks, 30)])["r"], "T2f", c, w, toks, "float32", "from a folder")
    del w["l1.mlp.correction"]
    w["l2.hc2.mix"] = torch.zeros(3, 3)
    with pytest.raises(WeightsError) as e:
        Engine.from_tensors(c, w, dtype="float32", max_tokens=256)
    assert e.value.missing == ["l1.mlp.correction"] and e.value.unexpected == ["l2.hc2.mix"]


def test_one_copy_of_the_stream_without_its_joining_tensors():
    """With one copy the joining tensors may be left out of the files: they count as 1, the plain residual sum."""
    from libllm_b200.engine import Engine
    c = S.CONFIGS["T3"]
    w = S.random_weights(c, 5)
    ones = {k: torch.ones_like(v) for k, v in w.items() if ".hc" in k}
    bare = {k: v for k, v in w.items() if ".hc" not in k}
    toks = S.tokens(c, 50, 2)
    got = replay_batch(Engine.from_tensors(c, bare, dtype="float32", max_tokens=256), [("r", toks, 40)])["r"]
    margins = []
    ref = P.forward(c, {**bare, **ones}, toks, margins=margins)
    S.check_rows(got, ref, "float32", "one copy, no joining tensors", torch.stack(margins).min(0).values)


def test_the_command_line_generates_from_a_tazizen_folder(tmp_path):
    """``bin/llm generate`` picks the model by config.json's ``architecture`` and builds what it needs."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, c, w = tazizen_folder(tmp_path, "T4", 8)
    prompt = S.tokens(c, 7, 800)
    out = subprocess.run([os.path.join(root, "bin", "llm"), "generate", "-m", folder, "--prompt-ids", ",".join(map(str, prompt)),
                          "--max-new-tokens", "4", "--temperature", "0", "--dtype", "float32", "--no-stop"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    got = [int(t) for t in out.stdout.strip().splitlines()[-1].split(",")]
    seq = list(prompt)
    for tok in got:
        logits = P.forward(c, w, seq)[-1]
        top2 = logits.topk(2)
        assert tok == int(top2.indices[0]) or float(top2.values[0] - top2.values[1]) < 1e-3
        seq.append(tok)
    assert len(got) == 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_of_a_tazizen_folder(dtype, tmp_path):
    """``bin/trace_run`` on a folder: two unequal requests that start together and go on by single tokens, then a
    third alone that uses their slots and pages again."""
    from test_entry_points_gpu import collect, run_trace, trace_of
    folder, c, w = tazizen_folder(tmp_path, "T3", 9, steady_choice=dtype == "bfloat16")
    first = [("a", S.tokens(c, 120, 1), 101), ("b", S.tokens(c, 40, 2), 7)]
    steps = trace_of(first)
    steps += trace_of([("c", S.tokens(c, 70, 3), 66)], first_step=len(steps))
    out_dir = str(tmp_path / "out")
    run_trace(folder, dtype, steps, out_dir, max_tokens=256)
    got = collect(steps, out_dir, c["vocab"])
    for rid, toks, _ in first + [("c", S.tokens(c, 70, 3), 66)]:
        compare(got[rid], "T3t", c, w, toks, dtype, f"trace {rid}")
