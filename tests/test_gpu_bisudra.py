"""The Bisudra decoder through the engine against the plain implementation: whole prompts, every token decoded one by
one from the first, the last tokens decoded one by one (long enough for pages to fill and for every window to pass over
decoded tokens), prompts cut into portions down to two tokens, batches of unequal requests with a cache so small that
slots (and with them the convolutions' inputs) and pages are used again, the replay program itself, and greedy
generation through the engine's own entry point.  Both precisions."""
import os
import subprocess
import sys

import pytest
import torch

import plain_bisudra
from bisudra_helpers import CONFIGS, assert_logits, make_bisudra_dir, plain_inputs, reference
from conftest import ROOT, random_prompts
from replay_helpers import (max_live_tokens, read_rows, run_in_process, trace_batches, trace_tail_one_by_one,
                            trace_whole, write_trace)

pytestmark = pytest.mark.gpu

LENGTHS = [1, 2, 33, 64, 65, 131, 40, 200, 70, 260]
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E", "F"])
def setup(request, session_tmp):
    d = make_bisudra_dir(session_tmp, CONFIGS[request.param], seed=11)
    cfg, weights = plain_inputs(d)
    prompts = random_prompts(cfg["vocab"], LENGTHS, seed=23)
    requests = {f"r{i}": p for i, p in enumerate(prompts)}
    refs = {rid: reference(cfg, weights, toks) for rid, toks in requests.items()}
    return d, cfg, weights, requests, refs


def _check(got, refs, dtype, what):
    by_req: dict = {}
    for (rid, pos), row in got.items():
        by_req.setdefault(rid, []).append((pos, row))
    for rid, items in by_req.items():
        items.sort()
        assert_logits(torch.stack([r for _, r in items]), refs[rid][[p for p, _ in items]], dtype, f"{what} request {rid}")


@DTYPES
@pytest.mark.parametrize("cut", ["whole", "one by one", "tail150", "batches3", "batches8"])
def test_replay_cuts_match_plain(setup, tmp_path, dtype, cut):
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, requests, refs = setup
    if cut == "whole":
        steps, rows = trace_whole(requests)
    elif cut == "one by one":
        few = {r: requests[r] for r in ("r1", "r5", "r6")}
        steps, rows = trace_tail_one_by_one(few, 10 ** 6)
    elif cut == "tail150":
        steps, rows = trace_tail_one_by_one(requests, 150)
    elif cut == "batches3":
        steps, rows = trace_batches(requests, 3)
    else:
        steps, rows = trace_batches(requests, 8, prompt_fraction=0.3)
    model = load_model(d, dtype)
    run_in_process(model, steps, tmp_path, max_live_tokens(steps))  # the smallest cache the trace is promised
    _check(read_rows(tmp_path, rows, cfg["vocab"]), refs, dtype, cut)


@DTYPES
@pytest.mark.parametrize("sizes", [[2], [2, 3, 1, 7], [64], [63, 2], [5, 128]], ids=str)
def test_prompts_in_portions(setup, dtype, sizes):
    """A prompt fed in portions (the sizes repeat) gives at every position what the whole prompt gives; two requests
    advance together through portions of different sizes (a portion shorter than the convolution's reach among them)."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, requests, refs = setup
    model = load_model(d, dtype)
    cache = model.new_cache(64 * 12)
    step = StepFunction(model, cache)
    pair = ["r7", "r5"]                          # 200 and 131 tokens
    slots = {r: cache.acquire() for r in pair}
    at = {r: 0 for r in pair}
    got = {r: [] for r in pair}
    k = 0
    while any(at[r] < len(requests[r]) for r in pair):
        inputs, who = [], []
        for j, r in enumerate(pair):
            n = sizes[(k + j) % len(sizes)]
            toks = requests[r][at[r]:at[r] + n]
            if toks:
                inputs.append(SequenceInput(slots[r], toks, list(range(len(toks)))))
                who.append((r, len(toks)))
        out = step(inputs).cpu()
        off = 0
        for r, n in who:
            got[r].append(out[off:off + n].clone())
            off += n
            at[r] += n
        k += 1
    for r in pair:
        assert_logits(torch.cat(got[r]), refs[r], dtype, f"portions {sizes} request {r}")
        cache.release(slots[r])
    cache.check_invariants()


@DTYPES
def test_a_step_cut_into_passes(setup, dtype):
    """A step with more tokens than one pass may hold runs as several passes that continue what the earlier pass left
    in the cache and in the convolutions' inputs; every pass keeps the levels of its own tokens."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, requests, refs = setup
    model = load_model(d, dtype)
    cache = model.new_cache(64 * 16)
    ids = ["r9", "r2", "r5", "r0"]
    wants = {r: sorted({0, len(requests[r]) // 3, len(requests[r]) - 1}) for r in ids}
    for limits in (dict(max_pass_tokens=96, max_sequence_chunk=8192), dict(max_pass_tokens=16384, max_sequence_chunk=40)):
        step = StepFunction(model, cache, **limits)
        slots = {r: cache.acquire() for r in ids}
        out = step([SequenceInput(slots[r], requests[r], wants[r]) for r in ids]).cpu()
        off = 0
        for r in ids:
            n = len(wants[r])
            assert_logits(out[off:off + n], refs[r][wants[r]], dtype, f"passes {limits} request {r}")
            off += n
        for r in ids:
            cache.release(slots[r])
    cache.check_invariants()


@DTYPES
def test_recorded_and_unrecorded_decode_steps_agree(setup, dtype):
    """Decode steps replayed from a recording give what the same steps give launch by launch."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, requests, refs = setup
    model = load_model(d, dtype)
    outs = []
    for graphs in (True, False):
        cache = model.new_cache(64 * 8)
        step = StepFunction(model, cache, use_graphs=graphs)
        ids = ["r2", "r4"]
        slots = {r: cache.acquire() for r in ids}
        step([SequenceInput(slots[r], requests[r][:20], []) for r in ids])
        rows = [step([SequenceInput(slots[r], [requests[r][p]], [0]) for r in ids]).cpu().clone() for p in range(20, 33)]
        outs.append(torch.stack(rows))
        for j, r in enumerate(ids):
            assert_logits(outs[-1][:, j], refs[r][20:33], dtype, f"decode steps, graphs {graphs}, request {r}")
    assert float((outs[0] - outs[1]).abs().max()) <= 1e-5 * float(outs[0].abs().max())


def test_decode_steps_read_in_the_step_kernel(session_tmp):
    """In a step of one token per sequence a layer's last kernel applies the next block's input convolution: only the
    first block launches one; a layer is one kernel per sublayer result, and the mix over the levels has none of its own
    behind level 0."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model
    from gpullama3.java_b200.kernels import ops

    d = make_bisudra_dir(session_tmp, CONFIGS["A"], seed=11)
    model = load_model(d, torch.bfloat16)
    cache = model.new_cache(64 * 4)
    step = StepFunction(model, cache, use_graphs=False)
    slots = [cache.acquire(), cache.acquire()]
    step([SequenceInput(slots[0], [5, 6, 7], []), SequenceInput(slots[1], [8], [])])
    ops.profile_start()
    step([SequenceInput(s, [9], [0]) for s in slots])
    table = ops.profile_stop()
    layers = CONFIGS["A"]["layers"]
    assert table["b200_causal_conv"][0] == 1
    assert table["b200_depth_average"][0] == 1
    assert table["b200_gated_norm_step"][0] == sum(2 + (L["mlp"] is not None) for L in layers)    # mixer, feed-forward, token input
    assert "b200_cast_rows" not in table
    ops.profile_start()
    step([SequenceInput(slots[0], [9, 3], [1]), SequenceInput(slots[1], [4], [0])])     # a portion: every block reads for itself
    assert ops.profile_stop()["b200_causal_conv"][0] == len(layers)


def test_which_models_run_short_prompts_as_recorded_passes(session_tmp):
    from gpullama3.java_b200.engine.trace import load_model

    safe = {name: load_model(make_bisudra_dir(session_tmp, CONFIGS[name], seed=11), torch.bfloat16).pad_safe for name in CONFIGS}
    assert safe == {"A": False, "B": False, "C": False, "D": False, "E": False, "F": True}


@DTYPES
def test_logits_do_not_depend_on_the_batch(setup, dtype):
    """A request's logits in a batch of unequal requests are those it has alone, within the rounding of one product (the
    products' tiles depend on the number of rows), for prompts and for decoded tokens, also in a slot and pages that
    another request has left."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, requests, refs = setup
    model = load_model(d, dtype)
    cache = model.new_cache(64 * 12)
    step = StepFunction(model, cache, use_graphs=False)

    def run(ids):
        slots = {r: cache.acquire() for r in ids}
        out = {r: [] for r in ids}
        head = {r: min(len(requests[r]) - 1, 37) for r in ids}
        got = step([SequenceInput(slots[r], requests[r][:head[r]], [head[r] - 1]) for r in ids]).cpu()
        for j, r in enumerate(ids):
            out[r].append(got[j].clone())
        for k in range(12):
            live = [r for r in ids if head[r] + k < len(requests[r])]
            if not live:
                break
            got = step([SequenceInput(slots[r], [requests[r][head[r] + k]], [0]) for r in live]).cpu()
            for j, r in enumerate(live):
                out[r].append(got[j].clone())
        for r in ids:
            cache.release(slots[r])
        return {r: torch.stack(v) for r, v in out.items()}

    together = run(["r6", "r3", "r7", "r2"])
    for r in ("r7", "r3", "r6"):            # alone, in slots and pages the batch has given back
        alone = run([r])[r]
        assert together[r].shape == alone.shape
        # (a routed layer's products run over other rows' tiles in a batch: within rounding of one product)
        tol = 0.0 if dtype == torch.float32 else 2e-2
        assert float((together[r] - alone).abs().max()) <= tol * float(alone.abs().max()) + (1e-4 * float(alone.abs().max()) if dtype == torch.float32 else 0.0)
    cache.check_invariants()


def test_trace_run_program(setup, tmp_path):
    """The program itself, as a user starts it: steps on standard input, 'done <step>' lines out, and a cache sized
    from the tokens alone (no allowance for partly filled pages)."""
    d, cfg, weights, requests, refs = setup
    few = {r: requests[r] for r in ("r2", "r0", "r4", "r6")}
    steps, rows = trace_batches(few, 4)
    trace = tmp_path / "trace.jsonl"
    write_trace(trace, steps)
    out = tmp_path / "out"
    env = dict(os.environ, PYTHON=sys.executable)
    with open(trace) as f:
        p = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out),
                            "--max-tokens", str(sum(len(t) for t in few.values()))], stdin=f, capture_output=True,
                           text=True, env=env, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    _check(read_rows(out, rows, cfg["vocab"]), refs, torch.float32, "trace_run")


@DTYPES
def test_greedy_generation_through_the_engine(setup, dtype):
    """``Engine.generate`` (the scheduler's batches, recorded decode steps, the argmax kernel): every generated token
    is the plain implementation's greedy choice given the tokens before it (bfloat16: within rounding of the best)."""
    from gpullama3.java_b200.engine.api import Engine

    d, cfg, weights, requests, refs = setup
    prompts = [requests[r] for r in ("r2", "r0", "r6", "r4", "r1")]
    engine = Engine.from_folder(d, dtype="float32" if dtype == torch.float32 else "bfloat16", max_tokens=64 * 8, max_batch=3)
    got = engine.generate(prompts, max_new_tokens=12, stop_ids=())
    for p, g in zip(prompts, got):
        assert len(g) == 12
        ref = reference(cfg, weights, list(p) + list(g))
        for i, tok in enumerate(g):
            row, moved = ref.logits[len(p) - 1 + i], ref.moved[len(p) - 1 + i]
            slack = 1e-4 * float(row.abs().max()) if dtype == torch.float32 else 0.05 * float(row.abs().max()) + 3.0 * float(moved.max())
            assert float(row.max() - row[tok]) <= slack, (p, g, i)


def test_command_line(setup, tmp_path):
    """``bin/llama-b200`` on a Bisudra folder: greedy tokens are the plain implementation's, and random weights fill a
    configuration."""
    import json

    d, cfg, weights, requests, refs = setup
    env = dict(os.environ, PYTHON=sys.executable)
    prompt = requests["r2"][:9]
    cmd = [str(ROOT / "bin" / "llama-b200"), "--model", str(d), "--dtype", "float32", "--temperature", "0", "-n", "5",
           "--stream", "false", "--prompt", " ".join(map(str, prompt))]
    p = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    got = list(map(int, p.stdout.split()))
    assert len(got) == 5
    logits = plain_bisudra.forward(cfg, weights, prompt + got)
    for i, tok in enumerate(got):
        row = logits[len(prompt) - 1 + i]
        assert float(row.max() - row[tok]) <= 1e-4 * float(row.abs().max())
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    p = subprocess.run([str(ROOT / "bin" / "llama-b200"), "--config", str(tmp_path / "config.json"), "--random-weights", "3",
                        "--prompt", "1 2 3", "--prompt", "4 5", "-n", "4", "--seed", "1", "--temperature", "0.8",
                        "--top-p", "0.9"], capture_output=True, text=True, env=env, timeout=900)
    assert p.returncode == 0 and len(p.stdout.split()) == 8, p.stderr[-2000:]
