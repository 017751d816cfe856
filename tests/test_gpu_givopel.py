"""The Givopel decoder through the library's engine, cache and entry points, against the plain implementation
(tests/plain/givopel.py): whole prompts, token-by-token decoding, prompts cut into portions down to two tokens,
batches of unequal requests, slots and blocks that are used again, long decoding through captured steps, and
greedy generation through the scheduler."""
import numpy as np
import pytest

from givopel_cases import CASES, make_case
from helpers import random_prompts, scaled_error

pytestmark = pytest.mark.gpu
# Of the logit scale.  The 32-bit runs are the sharp ones.  The test models' sharp attention and unit-norm branch
# outputs multiply a rounding error by about 1.6 with every layer run (measured in 32-bit: 3e-7 of the stream after
# the first run, 5e-6 after the seventh; in bfloat16 0.003 and 0.075), so whole models of seven runs get wider
# bounds than single mechanisms do (2e-5 and 3e-2 there).  A wrong key, a lost state or a token that is one off
# moves the logits by 0.2 or more of their scale.
TOL = {"float32": 5e-5, "bfloat16": 0.1}


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    root = tmp_path_factory.mktemp("givopel")
    return {name: make_case(root, name) for name in CASES}


def _plain(config, weights, tokens):
    from plain import givopel
    return givopel.forward(config, weights, tokens)


def _engine(folder, dtype, tokens=64 * 24):
    from xeno_rt_b200.engine import Engine
    from xeno_rt_b200.engine.model import Model
    return Engine(Model.load(folder, dtype=dtype), tokens)


def _run_cut(engine, tokens, cuts):
    """All logits of ``tokens`` fed in portions of the sizes ``cuts``."""
    from xeno_rt_b200.engine import StepEntry
    slot = engine.open_slot()
    parts, at = [], 0
    for size in cuts:
        parts.append(engine.step([StepEntry(slot, tokens[at:at + size], list(range(size)))]).cpu().numpy())
        at += size
    assert at == len(tokens)
    engine.close_slot(slot)
    return np.concatenate(parts)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_prompts_portions_and_decoding_give_the_plain_logits(cases, name, dtype):
    folder, config, weights = cases[name]
    engine = _engine(folder, dtype)
    n = 330 if name == "wide" else 200
    tokens = random_prompts(config["vocab"], [n], seed=1)[0]
    want = _plain(config, weights, tokens)
    tol = TOL[dtype]
    whole = _run_cut(engine, tokens, [n])
    assert scaled_error(whole, want) < tol
    # the first tokens alone (a state that starts at zero, convolutions that reach before the start)
    assert scaled_error(whole[:4], want[:4]) < tol
    # most of it in one step, the rest token by token: across a block's edge (192) in the long case
    assert scaled_error(_run_cut(engine, tokens, [n - 40] + [1] * 40), want) < tol
    # portions of several sizes, down to two tokens and one, shorter than the convolutions reach
    cuts = [2, 1, 2, 3, 59, 64, 5, 2]
    assert scaled_error(_run_cut(engine, tokens, cuts + [n - sum(cuts)]), want) < tol
    # token by token from the first one
    assert scaled_error(_run_cut(engine, tokens[:70], [1] * 70), want[:70]) < tol
    if dtype == "float32":  # how the tokens are cut changes nothing but rounding
        assert scaled_error(_run_cut(engine, tokens, [n - 40] + [1] * 40), whole) < 2e-6
    engine.check_errors()
    engine.cache.check()
    assert engine.cache.blocks_free() == engine.cache.n_blocks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["loop-middle", "wide"])
def test_unequal_batches_equal_each_request_alone_and_slots_are_used_again(cases, name, dtype):
    from xeno_rt_b200.engine import StepEntry
    folder, config, weights = cases[name]
    engine = _engine(folder, dtype, 64 * 16)
    tol = TOL[dtype]
    lengths = [1, 150, 7, 66, 129]
    decode = 12
    prompts = random_prompts(config["vocab"], [k + decode for k in lengths], seed=4)
    want = [_plain(config, weights, p) for p in prompts]
    for turn in range(2):  # the second turn takes the slots, blocks and states that the first gave back
        slots = [engine.open_slot() for _ in prompts]
        got = [[] for _ in prompts]
        out = engine.step([StepEntry(s, p[:k], list(range(k))) for s, p, k in zip(slots, prompts, lengths)]).cpu().numpy()
        at = 0
        for i, k in enumerate(lengths):
            got[i].append(out[at:at + k])
            at += k
        live = list(range(len(prompts)))
        for step in range(decode):
            if step == 5:  # a shorter request ends earlier; its slot is closed while the others go on
                engine.close_slot(slots[live.pop(0)])
            out = engine.step([StepEntry(slots[i], [prompts[i][lengths[i] + step]], [0]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1])
        for i in live:
            engine.close_slot(slots[i])
        for i in range(len(prompts)):
            rows = np.concatenate(got[i])
            assert scaled_error(rows, want[i][:len(rows)]) < tol, (turn, i)
        engine.cache.check()
    engine.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(cases, dtype):
    """300 single-token steps after a short prompt: the states and the keys of token 0 still count at the end."""
    folder, config, weights = cases["loop-middle"]
    engine = _engine(folder, dtype)
    assert engine.use_graphs and engine.model.graph_safe
    tokens = random_prompts(config["vocab"], [305], seed=9)[0]
    want = _plain(config, weights, tokens)
    assert scaled_error(_run_cut(engine, tokens, [5] + [1] * 300), want) < TOL[dtype]
    # the first tokens matter at the end: the same tail after another beginning gives other logits
    other = _plain(config, weights, [(t + 1) % config["vocab"] for t in tokens[:5]] + tokens[5:])
    assert scaled_error(other[-1:], want[-1:]) > 0.2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(cases, dtype):
    from xeno_rt_b200 import GenerateRequest, Runtime
    from plain import givopel
    folder, config, weights = cases["loop-middle"]
    prompts = random_prompts(config["vocab"], [3, 70, 20], seed=6)
    session = Runtime.load(folder, dtype=dtype).new_session()
    requests = [GenerateRequest(p, max_tokens=10, temperature=0.0, repetition_penalty=1.0, stop_ids=()) for p in prompts]
    results, stats = session.generate_batch(requests)
    tol = TOL[dtype]
    for p, r in zip(prompts, results):
        assert len(r.tokens) == 10 and r.finish_reason == "length"
        want = givopel.forward(config, weights, list(p) + list(r.tokens))
        scale = np.abs(want).max()
        for i, token in enumerate(r.tokens):  # the plain model's best token wherever its lead is beyond rounding
            row = want[len(p) + i - 1]
            top = np.sort(row)[-2:]
            if top[1] - top[0] > 2 * tol * scale:
                assert int(token) == int(np.argmax(row)), (i, token)
    session.backend.engine.cache.check()


def test_a_model_without_a_file_is_drawn_from_a_seed(cases):
    """Random weights on the device need the ranks in the configuration; the model then steps like any other."""
    import copy
    from xeno_rt_b200.core import ConfigError
    from xeno_rt_b200.engine import Engine, StepEntry
    from xeno_rt_b200.engine.model import Model
    config = copy.deepcopy(CASES["loop-middle"][0])
    with pytest.raises(ConfigError):
        Model.random(config, seed=1)
    config["layers"][0]["mixer"]["decay_rank"] = 8
    for i in (1, 2):
        config["layers"][i]["mixer"]["right"].update(decay_rank=8, gate_rank=8)
    engine = Engine(Model.random(config, seed=1), 256)
    slot = engine.open_slot()
    a = engine.step([StepEntry(slot, [1, 2, 3, 4], [3])])
    b = engine.step([StepEntry(slot, [5], [0])])
    assert a.shape == (1, config["vocab"]) and bool(a.isfinite().all()) and bool(b.isfinite().all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(cases, tmp_path, dtype):
    """``bin/trace_run`` on a Givopel folder: five requests of unequal lengths start as one batch and are decoded
    together, the shorter ones end earlier, and the cache is asked for no more than the tokens they hold (every
    request's last block of 64 is partly empty)."""
    import json
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, config, weights = cases["no-loop"]
    lengths, tails = [3, 70, 1, 65, 20], [4, 9, 2, 9, 6]
    prompts = random_prompts(config["vocab"], [k + t for k, t in zip(lengths, tails)], seed=21)
    want = [_plain(config, weights, p) for p in prompts]
    steps = [{"step": 0, "entries": [{"id": f"q{i}", "tokens": p[:k], "want": list(range(k))}
                                     for i, (p, k) in enumerate(zip(prompts, lengths))], "end": []}]
    for n in range(max(tails)):
        live = [i for i, t in enumerate(tails) if n < t]
        steps.append({"step": n + 1, "entries": [{"id": f"q{i}", "tokens": [prompts[i][lengths[i] + n]],
                                                  "want": [0] if n % 2 == 0 else []} for i in live],
                      "end": [f"q{i}" for i in live if n == tails[i] - 1]})
    out = tmp_path / dtype
    proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
                           "--max-tokens", str(sum(len(p) for p in prompts))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got = {i: [] for i in range(len(prompts))}
    rows = {i: [] for i in range(len(prompts))}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if not wanted:
            assert not (out / f"{s['step']}.f32").exists()
            continue
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, config["vocab"])
        assert data.shape[0] == wanted
        at = 0
        for e in s["entries"]:
            i = int(e["id"][1:])
            first = 0 if s["step"] == 0 else lengths[i] + s["step"] - 1
            got[i].append(data[at:at + len(e["want"])])
            rows[i] += [first + w for w in e["want"]]
            at += len(e["want"])
    for i in range(len(prompts)):
        assert scaled_error(np.concatenate(got[i]), want[i][rows[i]]) < TOL[dtype], i
