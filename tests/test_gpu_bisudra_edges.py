"""Keys at the edges of Bisudra's windows (just inside and just outside, in prompts and in decoding, windows shorter
than a page and longer than two), keys far back over many pages with peaked scores, page borders, the first tokens of a
sequence, the reach of the input convolution, the rotation's position, the second map and lambda, and long decoding.
Each test first shows on the plain implementation that the thing it probes moves the logits by far more than the
tolerance (a window one token shorter or longer, the far keys hidden, the positions shifted, a tap removed, the second
map's weight changed), so that an engine that got it wrong could not pass.  The window model's score scale is small:
its attention is nearly flat, so every visible key carries weight and the edge key cannot hide behind a peak; the far-key
model's is large, so that single far keys carry the result."""
import copy

import pytest
import torch

import plain_bisudra
from bisudra_helpers import assert_logits, make_bisudra_dir, plain_inputs
from conftest import random_prompts

pytestmark = pytest.mark.gpu
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])


def _att(heads, kv_heads, dim, vdim, scale, diff, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


WINDOWS = {
    "architecture": "Bisudra", "vocab": 64, "width": 32, "norm": {"eps": 1e-6}, "canon": {"taps": 2}, "token_side": {"dim": 6},
    "initializer_range": 0.1,
    "layers": [
        {"type": "attention", "mixer": _att(2, 1, 16, 32, 0.02, 0.3, window=17, rot=(100.0, 8)), "mlp": {"kind": "dense", "ff": 48}},
        {"type": "attention", "mixer": _att(1, 1, 32, 32, 0.02, 0.6, window=140), "mlp": None},
    ],
}
FAR = {
    "architecture": "Bisudra", "vocab": 64, "width": 32, "norm": {"eps": 1e-6}, "canon": {"taps": 3}, "token_side": {"dim": 7},
    "initializer_range": 0.1,
    "layers": [
        {"type": "attention", "mixer": _att(2, 2, 16, 16, 1.5, 0.4, window=690, rot=(3000.0, 16)), "mlp": {"kind": "dense", "ff": 48}},
        {"type": "attention", "mixer": _att(2, 1, 8, 32, 1.1, 0.5, rot=(500.0, 4)),
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 3, "top": 1}}},
    ],
}


def _run(model_dir, dtype, tokens, prompt_len, chunk=None):
    """Logits at every position: the first ``prompt_len`` tokens as a prompt (in portions of ``chunk``), the rest one
    token a step."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    model = load_model(model_dir, dtype)
    cache = model.new_cache(64 * (len(tokens) // 64 + 2))
    step = StepFunction(model, cache)
    slot = cache.acquire()
    out, at = [], 0
    while at < len(tokens):
        n = 1 if at >= prompt_len else min(chunk or prompt_len, prompt_len - at)
        out.append(step([SequenceInput(slot, tokens[at:at + n], list(range(n)))]).cpu().clone())
        at += n
    cache.release(slot)
    cache.check_invariants()
    return torch.cat(out)


def _moved(a, b, scale):
    """Per position: how far two sets of logits are apart, in units of the float32 tolerance."""
    return (a - b).abs().amax(dim=1) / (5e-5 * scale)


@DTYPES
@pytest.mark.parametrize("prompt_len, chunk", [(330, None), (150, None), (150, 7), (3, None)])
def test_windows_in_prompts_and_in_decoding(session_tmp, dtype, prompt_len, chunk):
    d = make_bisudra_dir(session_tmp, WINDOWS, seed=2)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [330], seed=3)[0]
    ref = plain_bisudra.forward(cfg, weights, tokens)
    scale = float(ref.abs().max())
    for layer, size in ((0, 17), (1, 140)):
        for other in (size - 1, size + 1):
            c2 = copy.deepcopy(cfg)
            c2["layers"][layer]["mixer"]["mask"]["size"] = other
            moved = _moved(plain_bisudra.forward(c2, weights, tokens), ref, scale)[size + 2:]
            # (the second layer spreads its weight over 140 keys: one of them moves the logits less, still several
            # times what the float32 comparison allows)
            assert float((moved > (20 if layer == 0 else 4)).float().mean()) > 0.9, (layer, other, moved.median())
    assert_logits(_run(d, dtype, tokens, prompt_len, chunk), ref, dtype, f"windows, prompt of {prompt_len}")


@DTYPES
@pytest.mark.parametrize("prompt_len, chunk", [(700, None), (520, 130), (64, None)])
def test_far_keys_over_many_pages(session_tmp, dtype, prompt_len, chunk):
    """700 tokens: eleven pages of keys with peaked scores in both maps; the second layer has no window at all."""
    d = make_bisudra_dir(session_tmp, FAR, seed=4)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [700], seed=5)[0]
    ref = plain_bisudra.forward(cfg, weights, tokens)
    scale = float(ref.abs().max())
    for layer, size in ((0, 400), (1, 300)):
        hidden = copy.deepcopy(cfg)
        hidden["layers"][layer]["mixer"]["mask"] = {"size": size}        # attention that cannot see far back
        moved = _moved(plain_bisudra.forward(hidden, weights, tokens), ref, scale)[450:]
        assert float((moved > 20).float().mean()) > 0.9, (layer, moved.median())
    got = _run(d, dtype, tokens, prompt_len, chunk)
    assert_logits(got, ref, dtype, f"far keys, prompt of {prompt_len}")
    assert_logits(got[:4], ref[:4], dtype, "the first tokens")
    edges = [63, 64, 65, 127, 128, 129, 191, 192, 193]
    assert_logits(got[edges], ref[edges], dtype, "positions at pages' borders")


@DTYPES
def test_positions_taps_the_second_map_and_the_levels(session_tmp, dtype):
    """What the plain implementation loses when a mechanism is taken out, the engine must have: the rotation's position
    (the same tokens one place later), the convolution's oldest tap, the second map's weight lambda, the mix over the
    levels, the token input's own columns of the table, and the gate on a sublayer's result."""
    d = make_bisudra_dir(session_tmp, FAR, seed=6)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [150], seed=7)[0]
    ref = plain_bisudra.forward(cfg, weights, tokens)
    scale = float(ref.abs().max())
    shifted = plain_bisudra.forward(cfg, weights, [tokens[0]] + tokens)[1:]
    assert float((_moved(shifted, ref, scale)[8:] > 20).float().mean()) > 0.9
    changes = {
        "tap": lambda n, t: t * torch.tensor([0.0, 1.0, 1.0]) if n.endswith("canon1") else t,
        "lambda": lambda n, t: t * 0.5 if n.endswith("mix.lq2") else t,
        "levels": lambda n, t: torch.cat([t[:1] * 0.0, t[1:]]) if n.endswith(".dwa") else t,
        "gate": lambda n, t: t * 0.0 if n.endswith("rg1.b") or n.endswith("rg2.b") else t,
        "token input": lambda n, t: torch.roll(t, 7, dims=1) if n == "side.embed" else t,
    }
    for what, change in changes.items():
        other = {n: change(n, t) for n, t in weights.items()}
        moved = _moved(plain_bisudra.forward(cfg, other, tokens), ref, scale)[4:]
        assert float((moved > 20).float().mean()) > 0.9, (what, moved.median())
    assert_logits(_run(d, dtype, tokens, 90, 31), ref, dtype, "mechanisms")


@DTYPES
def test_long_decoding(session_tmp, dtype):
    """Four tokens of prompt, then 400 decoded one by one: windows pass over decoded tokens, pages fill and are let go
    of, and every step reads the convolution's inputs the step before it left."""
    d = make_bisudra_dir(session_tmp, WINDOWS, seed=8)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [404], seed=9)[0]
    ref = plain_bisudra.forward(cfg, weights, tokens)
    assert_logits(_run(d, dtype, tokens, 4), ref, dtype, "long decoding")
