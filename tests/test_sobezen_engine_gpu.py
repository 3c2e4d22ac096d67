"""The Sobezen decoder through the engine (its step function, cache, state and scheduler) against the plain
implementation, in float32 and bfloat16, for every way of cutting the work: whole prompts, prompts then single
tokens, portions of prompts down to two tokens, unequal batches, pages and slots used again, long decoding across
page borders, the first tokens, other sizes, and greedy generation."""
import pytest
import torch

import plain_sobezen as P
import sobezen_helpers as S
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
        w = S.random_weights(c, seed=len(name) + ord(name[-1]), ranks=S.RANKS[name])
        _engines[key] = (Engine.from_tensors(c, w, dtype=dtype, max_tokens=max_tokens, **kw), c, w)
    return _engines[key]


def plain(name, c, w, toks):
    key = (name, tuple(toks))
    if key not in _refs:
        _refs[key] = P.forward(c, w, toks)
    return _refs[key]


def compare(got, name, c, w, toks, dtype, what):
    S.check_rows(got, plain(name, c, w, toks), dtype, what)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(name, dtype):
    """Lengths from one token on, around the convolutions' reach (1 to 6 taps) and the page border (64)."""
    engine, c, w = setup(name, dtype)
    for i, n in enumerate([1, 2, 3, 5, 6, 7, 11, 25, 63, 64, 65, 81, 128, 130, 203]):
        toks = S.tokens(c, n, i)
        got = replay_batch(engine, [("r", toks, n)])["r"]
        compare(got, name, c, w, toks, dtype, f"{name} whole {n}")
    assert engine.pages_in_use() == [0] * len(engine.pages_in_use())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_residual_stream_after_every_layer(name, dtype):
    """Models cut after 1, 2, .. layers (a borrower stays behind its lender) give the logits of the plain model cut
    at the same place: a fault shows at the first layer that has it."""
    from libllm_b200.engine import Engine
    import copy
    c_full = S.CONFIGS[name]
    w_full = S.random_weights(c_full, seed=3, ranks=S.RANKS[name])
    toks = S.tokens(c_full, 70, 4)
    for n in range(1, len(c_full["layers"])):
        c = copy.deepcopy(c_full)
        c["layers"] = c["layers"][:n]
        keep = tuple(f"l{i}." for i in range(n))
        w = {k: v for k, v in w_full.items() if not k.startswith("l") or k.startswith(keep)}
        engine = Engine.from_tensors(c, w, dtype=dtype, max_tokens=256)
        got = replay_batch(engine, [("r", toks, 50)])["r"]
        S.check_rows(got, P.forward(c, w, toks), dtype, f"{name}: the first {n} layers")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens_agrees_with_the_whole_prompt(name, dtype):
    """The same request as one prompt and as a prompt followed by single tokens (which pass a page border, with
    state carried from step to step); also from a one-token prompt on."""
    engine, c, w = setup(name, dtype)
    for i, (n, n_prompt) in enumerate([(140, 100), (75, 35), (48, 1)]):
        toks = S.tokens(c, n, 20 + i)
        got = replay_batch(engine, [("r", toks, n_prompt)])["r"]
        compare(got, name, c, w, toks, dtype, f"{name} {n_prompt} + {n - n_prompt} single tokens")
        if dtype == "float32":
            whole = replay_batch(engine, [("r", toks, n)])["r"]
            assert float(S.row_errors(got, whole).max()) < S.TOL[dtype], f"{name}: decoding differs from the whole prompt"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_a_prompt(name, dtype):
    """A prompt brought in portions of several sizes, down to two tokens and one (shorter than the convolutions'
    reach, so that their state is a mix of old and new rows)."""
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
    """Three batches of unequal requests on a cache that holds one batch at a time, so that pages, slots and the
    slots' state are used again; shorter requests end earlier; each request against the plain implementation and,
    in float32, against itself alone."""
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
                assert float(S.row_errors(got[rid], single).max()) < S.TOL[dtype], f"{name} {rid}: the batch changes the result"
    assert engine.pages_in_use() == [0] * len(engine.pages_in_use())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B1", "B2", "B3", "B5"])
def test_long_decoding(name, dtype):
    """One token a step for 330 steps: pages are taken as the rows grow over five page borders, borrowers read what
    their lender appended in the same step, the recurrent state is carried through every step."""
    engine, c, w = setup(name, dtype)
    toks = S.tokens(c, 330, 77)
    got = replay_batch(engine, [("r", toks, 2)])["r"]
    compare(got, name, c, w, toks, dtype, f"{name} long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_beside_a_long_neighbour(dtype):
    engine, c, w = setup("B1", dtype)
    short, long_ = S.tokens(c, 3, 5), S.tokens(c, 90, 6)
    both = replay_batch(engine, [("l", long_, 60), ("s", short, 1)])
    compare(both["s"], "B1", c, w, short, dtype, "first tokens beside a long request")
    compare(both["l"], "B1", c, w, long_, dtype, "long neighbour")


@pytest.mark.parametrize("name", NAMES)
def test_what_the_cache_holds(name):
    """A latent layer with rows of its own holds one key head of kv_rank + rot_dim channels and no values; a layer
    that borrows holds nothing; attention holds its rotated keys and, as values, the keys as projected."""
    engine, c, w = setup(name, "float32")
    slot = engine.open_sequence()
    engine.step([StepItem(slot, S.tokens(c, 130, 3), [129])])
    info = engine.cache_info()
    groups = info["groups"]
    own = [i for i, L in enumerate(c["layers"])
           if L["type"] == "attention" or (L["type"] == "latent_attention" and L["mixer"].get("kv_from") is None)]
    assert sorted(r for g in groups for r in g["runs"]) == own          # a borrower and the delta rule own no pages
    assert all(g["pages_in_use"] == 3 * len(g["runs"]) or g["pages_in_use"] == 3 for g in groups), groups
    for g in groups:
        for r in g["runs"]:
            m = c["layers"][r]["mixer"]
            if c["layers"][r]["type"] == "latent_attention":
                assert (g["n_kv_heads"], g["k_dim"], g["v_dim"]) == (1, m["kv_rank"] + m["rot_dim"], 0), g
            else:
                assert (g["n_kv_heads"], g["k_dim"], g["v_dim"]) == (m["kv_heads"], m["dim"], m["dim"]), g
    engine.close_sequence(slot)
    engine.cache_check()
    assert engine.pages_in_use() == [0] * len(engine.pages_in_use())


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_cut_into_launch_sequences(dtype):
    """max_step_tokens below the prompts' lengths: the engine itself cuts inside a prompt, and the state goes on
    from piece to piece."""
    engine, c, w = setup("B2", dtype, max_step_tokens=48)
    reqs = [("a", S.tokens(c, 150, 1), 150), ("b", S.tokens(c, 30, 2), 30)]
    got = replay_batch(engine, reqs)
    for rid, toks, _ in reqs:
        compare(got[rid], "B2", c, w, toks, dtype, f"cut {rid}")


@pytest.mark.parametrize("name", NAMES)
def test_the_last_row_alone(name):
    """A prompt of which only some places are wanted (the last layer then runs its feed-forward for those rows
    alone), and a portion of which nothing is wanted (its cache and state still move on)."""
    engine, c, w = setup(name, "float32")
    toks = S.tokens(c, 77, 9)
    ref = plain(name, c, w, toks)
    slot = engine.open_sequence()
    assert engine.step([StepItem(slot, toks[:40], [])]).shape[0] == 0
    got = torch.from_numpy(engine.step([StepItem(slot, toks[40:], [36, 0])]))
    engine.close_sequence(slot)
    S.check_rows(got, ref[[76, 40]], "float32", f"{name} chosen rows")


def test_a_slot_used_again_starts_from_zero_state():
    """A sequence that takes the slot of a finished one must not see its recurrent or convolution state."""
    engine, c, w = setup("B6", "float32", max_tokens=256)
    a, b = S.tokens(c, 50, 1), S.tokens(c, 33, 2)
    s1 = engine.open_sequence()
    engine.step([StepItem(s1, a, [49])])
    engine.close_sequence(s1)
    s2 = engine.open_sequence()
    assert s2 == s1
    got = torch.from_numpy(engine.step([StepItem(s2, b, list(range(33)))]))
    engine.close_sequence(s2)
    S.check_rows(got, plain("B6", c, w, b), "float32", "a slot used again")


@pytest.mark.parametrize("name", ["B1", "B3", "B5"])
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


def sobezen_folder(tmp_path, name, seed):
    import json
    from helpers import write_safetensors
    c = S.CONFIGS[name]
    w = S.random_weights(c, seed, S.RANKS[name])
    (tmp_path / "config.json").write_text(json.dumps(c))
    write_safetensors(str(tmp_path / "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in w.items()})
    return str(tmp_path), c, w


def test_the_model_folder_route_names_what_does_not_fit(tmp_path):
    """Weights written as a safetensors file and loaded by folder give the engine that tensors in memory give; an
    unexpected or missing tensor is named (a borrower must not bring a latent projection of its own); the ranks of the
    low-rank inputs are taken from the stored tensors."""
    from libllm_b200.engine import Engine
    from libllm_b200.errors import WeightsError
    folder, c, w = sobezen_folder(tmp_path, "B2", 3)
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=256)
    toks = S.tokens(c, 40, 1)
    S.check_rows(replay_batch(engine, [("r", toks, 30)])["r"], P.forward(c, w, toks), "float32", "from a folder")
    del w["l1.mlp.up.b"]
    w["l2.mix.dkv"] = torch.zeros(44, 72)
    with pytest.raises(WeightsError) as e:
        Engine.from_tensors(c, w, dtype="float32", max_tokens=256)
    assert e.value.missing == ["l1.mlp.up.b"] and e.value.unexpected == ["l2.mix.dkv"]


def test_the_command_line_generates_from_a_sobezen_folder(tmp_path):
    """``bin/llm generate`` picks the model by config.json's ``architecture`` and builds what it needs."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, c, w = sobezen_folder(tmp_path, "B4", 8)
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
def test_trace_replay_of_a_sobezen_folder(dtype, tmp_path):
    """``bin/trace_run`` on a folder: two unequal requests that start together and go on by single tokens, then a
    third alone that uses their slots, pages and state again."""
    from test_entry_points_gpu import collect, run_trace, trace_of
    folder, c, w = sobezen_folder(tmp_path, "B3", 9)
    first = [("a", S.tokens(c, 120, 1), 101), ("b", S.tokens(c, 40, 2), 7)]
    steps = trace_of(first)
    steps += trace_of([("c", S.tokens(c, 70, 3), 66)], first_step=len(steps))
    out_dir = str(tmp_path / "out")
    run_trace(folder, dtype, steps, out_dir, max_tokens=256)
    got = collect(steps, out_dir, c["vocab"])
    for rid, toks, _ in first + [("c", S.tokens(c, 70, 3), 66)]:
        S.check_rows(got[rid], P.forward(c, w, toks), dtype, f"trace {rid}")
