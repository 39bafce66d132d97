"""The Sofunex decoder through the library's engine, cache and entry points, against the plain implementation
(tests/plain/sofunex.py): the residual stream after every layer run, whole prompts, token-by-token decoding, prompts
cut into portions down to two tokens, batches of unequal requests, slots, blocks and states that are used again,
windows that pass over decoded tokens and give their blocks back, long decoding through captured steps, greedy
generation through the scheduler, the command line and the trace replay program."""
import copy
import os

import numpy as np
import pytest

from helpers import random_prompts, scaled_error
from sofunex_cases import CASES, make_case, random_config, random_weights, write_folder

pytestmark = pytest.mark.gpu
# Of the logit scale.  The 32-bit runs are the sharp ones: a window that is one token off, a lost state or a tap
# that reads the wrong token moves the logits by far more (the tests below say by how much).
TOL = {"float32": 3e-5, "bfloat16": 0.08}
# A routing decision whose lead is this small may fall the other way in the compute dtype; from such a token on only
# the typical position is held to the bound (the design's own close call, no fault).
MARGIN = {"float32": 1e-4, "bfloat16": 0.05}


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    root = tmp_path_factory.mktemp("sofunex")
    return {name: make_case(root, name) for name in CASES}


def _plain(config, weights, tokens, dtype, streams=None):
    """(logits, the first position at which a routing decision is a close call in ``dtype``)."""
    from plain import sofunex
    margins = np.full(len(tokens), np.inf)
    logits = sofunex.forward(config, weights, tokens, streams=streams, margins=margins)
    hit = np.nonzero(margins < MARGIN[dtype])[0]
    return logits, (int(hit[0]) if len(hit) else len(tokens))


def _check(got, want, close, dtype, rows=None):
    rows = list(range(len(got))) if rows is None else list(rows)
    scale = np.abs(want).max()
    err = np.abs(got.astype(np.float64) - want[rows]).max(-1) / scale
    strict = np.array([r < close for r in rows])
    assert not strict.any() or err[strict].max() < TOL[dtype], (err[strict].max(), int(np.argmax(err * strict)))
    assert np.isfinite(err).all()
    if len(rows) >= 20:  # a handful of rows after a close call has no typical position
        assert np.median(err) < TOL[dtype]


def _engine(folder, dtype, tokens=64 * 24):
    from xeno_rt_b200.engine import Engine
    from xeno_rt_b200.engine.model import Model
    return Engine(Model.load(folder, dtype=dtype), tokens)


def _run_cut(engine, tokens, cuts):
    from xeno_rt_b200.engine import StepEntry
    slot = engine.open_slot()
    parts, at = [], 0
    for size in cuts:
        parts.append(engine.step([StepEntry(slot, tokens[at:at + size], list(range(size)))]).cpu().numpy())
        at += size
    assert at == len(tokens)
    engine.close_slot(slot)
    return np.concatenate(parts)


def _with_windows(config, by: int):
    other = copy.deepcopy(config)
    for layer in other["layers"]:
        mask = layer["mixer"]["left"].get("mask")
        if mask:
            mask["size"] = max(1, mask["size"] + by)
    return other


@pytest.mark.parametrize("name", list(CASES))
def test_the_stream_after_every_layer_run_is_the_plain_one(cases, name):
    """In 32-bit, layer run by layer run (a layer of a loop counts every time): the first that differs names the
    mechanism at fault."""
    import torch
    from xeno_rt_b200.engine import StepEntry
    folder, config, weights = cases[name]
    engine = _engine(folder, "float32")
    model = engine.model
    kept, original = [], list(model.arrangements)

    def wrap(fn):
        def run(parts, x, ctx, stores, owns):
            fn(parts, x, ctx, stores, owns)
            kept.append(x.clone())
        for key in ("first_norm", "reads_stream"):
            if hasattr(fn, key):
                setattr(run, key, getattr(fn, key))
        return run
    model.arrangements = [wrap(fn) for fn in original]
    tokens = random_prompts(config["vocab"], [150], seed=2)[0]
    want = []
    _plain(config, weights, tokens, "float32", streams=want)
    slot = engine.open_slot()
    engine.step([StepEntry(slot, tokens, [0])])
    engine.close_slot(slot)
    model.arrangements = original
    assert len(kept) == len(want) == len(model.spec.schedule)
    for i, (got, ref) in enumerate(zip(kept, want)):
        assert got.dtype == torch.float32  # the stream itself is 32-bit
        assert np.abs(got.cpu().numpy() - ref).max() < 3e-5 * max(1.0, np.abs(ref).max()), i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_prompts_portions_and_decoding_give_the_plain_logits(cases, name, dtype):
    folder, config, weights = cases[name]
    engine = _engine(folder, dtype)
    n = 330 if name == "wide" else 230
    tokens = random_prompts(config["vocab"], [n], seed=1)[0]
    want, close = _plain(config, weights, tokens, dtype)
    if dtype == "float32":
        # what a fault would look like here: every window one key wider or narrower moves the logits by far more
        # than the bound
        from plain import sofunex
        for by in (1, -1):
            off = sofunex.forward(_with_windows(config, by), weights, tokens)
            assert np.abs(off - want).max() / np.abs(want).max() > 20 * TOL[dtype]
    whole = _run_cut(engine, tokens, [n])
    _check(whole, want, close, dtype)
    # most of it in one step, the rest token by token: the windows pass over decoded tokens, across a block's edge
    decoded = _run_cut(engine, tokens, [n - 100] + [1] * 100)
    _check(decoded, want, close, dtype)
    # portions of several sizes, down to two tokens and one: every portion's first tokens read the convolutions'
    # and the shift's state, and the scan goes on from the state that the portion before left
    cuts = [2, 1, 2, 3, 59, 64, 5, 2]
    portions = _run_cut(engine, tokens, cuts + [n - sum(cuts)])
    _check(portions, want, close, dtype)
    # token by token from the first one
    _check(_run_cut(engine, tokens[:70], [1] * 70), want[:70], close, dtype)
    if dtype == "float32":  # how the tokens are cut changes nothing but rounding
        assert scaled_error(decoded, whole) < 3e-6 and scaled_error(portions, whole) < 3e-6
    engine.check_errors()
    engine.cache.check()
    assert engine.cache.blocks_free() == engine.cache.n_blocks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_unequal_batches_equal_each_request_alone_and_slots_are_used_again(cases, name, dtype):
    from xeno_rt_b200.engine import StepEntry
    folder, config, weights = cases[name]
    engine = _engine(folder, dtype, 64 * 16)
    lengths = [1, 150, 7, 66, 129]
    decode = 12
    prompts = random_prompts(config["vocab"], [k + decode for k in lengths], seed=4)
    want = [_plain(config, weights, p, dtype) for p in prompts]
    alone = _run_cut(engine, prompts[3], [lengths[3]] + [1] * decode)
    for turn in range(2):  # the second turn takes the slots, blocks and states that the first gave back, in another order
        slots = [engine.open_slot() for _ in prompts]
        if turn:
            slots = slots[::-1]
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
            _check(np.concatenate(got[i]), want[i][0], want[i][1], dtype)
        if dtype == "float32":  # what else is in the batch changes nothing but rounding
            assert scaled_error(np.concatenate(got[3]), alone) < 3e-6
        engine.cache.check()
        assert engine.cache.blocks_free() == engine.cache.n_blocks
    engine.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps_gives_the_blocks_behind_the_windows_back(cases, dtype):
    """300 single-token steps after a short prompt.  The windows (40, 70, 5 and 90 keys; the looped layers hold a cache
    for every pass) leave whole cache blocks behind, which go back to the pool while the sequence lives; the states
    of the scans, the convolutions and the shifts are carried through every captured step; the logits stay the plain
    ones to the end."""
    from xeno_rt_b200.engine import StepEntry
    folder, config, weights = cases["mixed"]
    engine = _engine(folder, dtype)
    assert engine.use_graphs and engine.model.graph_safe
    tokens = random_prompts(config["vocab"], [305], seed=9)[0]
    want, close = _plain(config, weights, tokens, dtype)
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, tokens[:5], list(range(5)))]).cpu().numpy()]
    rows += [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in tokens[5:]]
    _check(np.concatenate(rows), want, close, dtype)
    # a block of positions 64 b .. 64 b + 63 is done once 64 b + 63 <= 305 - window
    held = sorted(len(g.held_blocks(slot, 5)) for g in engine.cache.kv_groups)
    assert held == [1, 1, 2, 2], held
    free_now = engine.cache.blocks_free()
    engine.cache.check()
    engine.close_slot(slot)
    assert engine.cache.blocks_free() == engine.cache.n_blocks > free_now
    engine.check_errors()


def test_what_the_cache_holds_for_a_layer(cases):
    """Keys at the larger of key and value size (rounded up to 16) with the layer's window, the convolutions' last
    taps - 1 product rows, the scan's matrix a head, and the shift's row; a place of a loop owns all of it again."""
    from xeno_rt_b200.cache import KVNeed, StateNeed
    from xeno_rt_b200.engine.model import Model
    folder, config, weights = cases["mixed"]
    needs = Model.load(folder, dtype="bfloat16").cache_needs()
    assert len(needs) == 8 and needs[1] == needs[3] == needs[5] and needs[2] == needs[4]
    first = needs[0]
    assert first["mixer_shift"] == StateNeed((64,), "float32")
    (keys, taps), scan = first["mixer"]
    assert keys == KVNeed(2, 16, 40, 0) and taps == StateNeed((2, 4 * 16 + 2 * 2 * 16), "float32")
    assert scan == StateNeed((2, 32, 32), "float32")
    (keys, taps), scan = needs[1]["mixer"]
    assert keys == KVNeed(3, 32, 70, 0) and taps == StateNeed((1, (3 + 2 * 3) * 32), "float32") and scan == StateNeed((4, 16, 16), "float32")
    odd = Model.load(cases["odd"][0], dtype="float32").cache_needs()
    assert odd[0]["mixer"][0] == KVNeed(3, 32, 1, 0)          # one tap: no state of the convolution
    assert odd[1]["mixer"][0] == KVNeed(2, 32, None, 0)       # no window, no convolution


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(cases, dtype):
    from plain import sofunex
    from xeno_rt_b200 import GenerateRequest, Runtime
    folder, config, weights = cases["mixed"]
    prompts = random_prompts(config["vocab"], [3, 70, 20], seed=6)
    session = Runtime.load(folder, dtype=dtype).new_session()
    requests = [GenerateRequest(p, max_tokens=10, temperature=0.0, repetition_penalty=1.0, stop_ids=()) for p in prompts]
    results, stats = session.generate_batch(requests)
    tol = 0.1 if dtype == "bfloat16" else 1e-4
    for p, r in zip(prompts, results):
        assert len(r.tokens) == 10 and r.finish_reason == "length"
        want = sofunex.forward(config, weights, list(p) + list(r.tokens))
        scale = np.abs(want).max()
        for i, token in enumerate(r.tokens):  # the plain model's best token wherever its lead is beyond rounding
            row = want[len(p) + i - 1]
            top = np.sort(row)[-2:]
            if top[1] - top[0] > 2 * tol * scale:
                assert int(token) == int(np.argmax(row)), (i, token)
    session.backend.engine.cache.check()


def test_the_command_line_generates_what_the_session_generates(cases):
    """``xrt generate --model DIR`` picks the design by config.json: greedy tokens equal the session's; sampling with
    a seed repeats itself and differs from another seed."""
    import subprocess
    import sys
    from xeno_rt_b200 import GenerateRequest, Runtime
    folder, config, _ = cases["odd"]
    prompts = random_prompts(config["vocab"], [4, 31], seed=8)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    xrt = [sys.executable, os.path.join(root, "bin", "xrt"), "generate", "--model", folder, "--dtype", "float32",
           "--max-tokens", "9", "--stop-ids", "", "--prompt-ids", ",".join(map(str, prompts[0])),
           "--prompt-ids", ",".join(map(str, prompts[1]))]
    greedy = subprocess.run(xrt + ["--temperature", "0", "--repetition-penalty", "1.0"], capture_output=True, text=True,
                            timeout=600)
    assert greedy.returncode == 0, greedy.stderr
    session = Runtime.load(folder, dtype="float32").new_session()
    results, _ = session.generate_batch([GenerateRequest(p, max_tokens=9, temperature=0.0, repetition_penalty=1.0,
                                                         stop_ids=()) for p in prompts])
    lines = [list(map(int, l.split(","))) for l in greedy.stdout.strip().splitlines() if l]
    assert lines == [list(r.tokens) for r in results]
    sampled = [subprocess.run(xrt + ["--temperature", "1.3", "--top-k", "20", "--seed", seed], capture_output=True,
                              text=True, timeout=600) for seed in ("5", "5", "6")]
    assert all(run.returncode == 0 for run in sampled)
    assert sampled[0].stdout == sampled[1].stdout != sampled[2].stdout


def test_a_model_without_a_file_is_drawn_from_a_seed():
    from xeno_rt_b200.engine import Engine, StepEntry
    from xeno_rt_b200.engine.model import Model
    engine = Engine(Model.random(CASES["odd"][0], seed=1), 256)
    slot = engine.open_slot()
    a = engine.step([StepEntry(slot, [1, 2, 3, 4], [3])])
    b = engine.step([StepEntry(slot, [5], [0])])
    assert a.shape == (1, CASES["odd"][0]["vocab"]) and bool(a.isfinite().all()) and bool(b.isfinite().all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(cases, tmp_path, dtype):
    """``bin/trace_run`` on a Sofunex folder: five requests of unequal lengths start as one batch and are decoded
    together, the shorter ones end earlier."""
    import json
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, config, weights = cases["odd"]
    lengths, tails = [3, 70, 1, 65, 20], [4, 9, 2, 9, 6]
    prompts = random_prompts(config["vocab"], [k + t for k, t in zip(lengths, tails)], seed=21)
    want = [_plain(config, weights, p, dtype) for p in prompts]
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
        _check(np.concatenate(got[i]), want[i][0], want[i][1], dtype, rows[i])


def test_decode_steps_of_many_sequences_sort_their_experts_rows_inside_the_captured_step(cases):
    """11 sequences a step (16 rows with padding): enough (token, choice) pairs an expert for the grouped products,
    which run inside the captured step with the row counts staying on the device; the padding rows count as rows of
    some expert and change nothing, and no state of any slot is touched by them."""
    from xeno_rt_b200.engine import StepEntry
    folder, config, weights = cases["wide"]
    engine = _engine(folder, "bfloat16", 64 * 16)
    assert engine.use_graphs and engine.model.graph_safe
    lengths = [3, 9, 17, 5, 11, 2, 8, 13, 4, 6, 21]
    decode = 6
    prompts = random_prompts(config["vocab"], [k + decode for k in lengths], seed=12)
    want = [_plain(config, weights, p, "bfloat16") for p in prompts]
    slots = [engine.open_slot() for _ in prompts]
    got = [[] for _ in prompts]
    out = engine.step([StepEntry(s, p[:k], list(range(k))) for s, p, k in zip(slots, prompts, lengths)]).cpu().numpy()
    at = 0
    for i, k in enumerate(lengths):
        got[i].append(out[at:at + k])
        at += k
    for step in range(decode):
        out = engine.step([StepEntry(slots[i], [prompts[i][lengths[i] + step]], [0]) for i in range(len(prompts))]).cpu().numpy()
        for i in range(len(prompts)):
            got[i].append(out[i:i + 1])
    for i in range(len(prompts)):
        _check(np.concatenate(got[i]), want[i][0], want[i][1], "bfloat16")
        engine.close_slot(slots[i])
    engine.check_errors()
    engine.cache.check()


@pytest.mark.parametrize("seed", range(6))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Other sizes, orders, loops and options than the named cases, in 32-bit: whole, cut and decoded, and three
    unequal requests at a time."""
    from xeno_rt_b200.engine import StepEntry
    rng = np.random.default_rng(100 + seed)
    config = random_config(rng)
    weights = random_weights(config, 200 + seed)
    folder = write_folder(str(tmp_path / "drawn"), config, weights)
    engine = _engine(folder, "float32", 64 * 12)
    prompts = random_prompts(config["vocab"], [150, 9, 77], seed=seed)
    want = [_plain(config, weights, p, "float32") for p in prompts]
    _check(_run_cut(engine, prompts[0], [150]), *want[0], "float32")
    _check(_run_cut(engine, prompts[0], [2, 63, 1, 70] + [1] * 14), *want[0], "float32")
    slots = [engine.open_slot() for _ in prompts]
    heads = [140, 4, 70]
    got = [[] for _ in prompts]
    out = engine.step([StepEntry(s, p[:k], list(range(k))) for s, p, k in zip(slots, prompts, heads)]).cpu().numpy()
    at = 0
    for i, k in enumerate(heads):
        got[i].append(out[at:at + k])
        at += k
    for step in range(5):
        out = engine.step([StepEntry(slots[i], [prompts[i][heads[i] + step]], [0]) for i in range(3)]).cpu().numpy()
        for i in range(3):
            got[i].append(out[i:i + 1])
    for i in range(3):
        _check(np.concatenate(got[i]), want[i][0][:heads[i] + 5], want[i][1], "float32")
        engine.close_slot(slots[i])
    engine.check_errors()
    engine.cache.check()
