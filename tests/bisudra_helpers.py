"""Small Bisudra configurations for the tests, and model folders with random weights made so that faults show.

The configurations differ from one another in every size and option: heads per kv head (1, 2, 3 and 4) and kv heads (1 to
3), maps smaller than, as large as and larger than half the values, two maps that fill a size the tensor-core attention
kernels take and ones that are widened, rotation of a part of a map, of all of it and none, windows shorter than a
page, longer than two and none, score scales that are not 1 / sqrt(dim), a constant ``diff`` on both sides of one half,
input convolutions of 1 to 4 taps and none, token inputs of few numbers, of a number that is no multiple of 8, and none,
layers without feed-forward, dense and routed ones in every order, one expert of several and several of many."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _att(heads, kv_heads, dim, vdim, scale, diff, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


BISUDRA_A = {
    "architecture": "Bisudra", "vocab": 160, "width": 64, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
    "token_side": {"dim": 12}, "initializer_range": 0.08,
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 16, 32, 0.3, 0.4, window=40, rot=(5000.0, 8)), "mlp": _moe(32, 6, 2)},
        {"type": "attention", "mixer": _att(2, 2, 24, 16, 0.17, 0.7, window=130, rot=(100.0, 24)), "mlp": None},
        {"type": "attention", "mixer": _att(6, 2, 8, 24, 0.5, 0.2, rot=(10000.0, 2)), "mlp": _dense(96)},
    ],
}
BISUDRA_B = {
    "architecture": "Bisudra", "vocab": 200, "width": 96, "norm": {"eps": 1e-6}, "canon": {"taps": 2},
    "initializer_range": 0.06,
    "layers": [
        {"type": "attention", "mixer": _att(3, 3, 32, 64, 0.11, 0.5, window=64), "mlp": _dense(40)},
        {"type": "attention", "mixer": _att(4, 1, 16, 16, 0.25, 0.9, window=65, rot=(300.0, 16)), "mlp": _moe(24, 9, 4)},
    ],
}
BISUDRA_C = {
    "architecture": "Bisudra", "vocab": 96, "width": 48, "norm": {"eps": 1e-6}, "token_side": {"dim": 5},
    "initializer_range": 0.1,
    "layers": [
        {"type": "attention", "mixer": _att(3, 1, 40, 48, 0.2, 0.1, window=7, rot=(50.0, 10)), "mlp": _moe(16, 3, 1)},
        {"type": "attention", "mixer": _att(1, 1, 64, 128, 0.09, 0.6, rot=(1000000.0, 32)), "mlp": _moe(16, 2, 2)},
        {"type": "attention", "mixer": _att(8, 2, 8, 8, 0.4, 0.3, window=1), "mlp": _dense(64)},
        {"type": "attention", "mixer": _att(2, 1, 16, 40, 0.3, 0.5, window=200, rot=(10.0, 4)), "mlp": None},
    ],
}
# rows wide enough for the kernels that keep a token's row in registers over several rounds, a token input wider than
# one round of a warp, and a single tap (a convolution that reads no earlier input)
BISUDRA_D = {
    "architecture": "Bisudra", "vocab": 120, "width": 640, "norm": {"eps": 1e-5}, "canon": {"taps": 1},
    "token_side": {"dim": 40}, "initializer_range": 0.04,
    "layers": [
        {"type": "attention", "mixer": _att(2, 1, 32, 64, 0.2, 0.5, window=96, rot=(10000.0, 16)), "mlp": _dense(256)},
        {"type": "attention", "mixer": _att(4, 2, 64, 128, 0.12, 0.25, window=33, rot=(500.0, 64)), "mlp": _moe(128, 4, 2)},
    ],
}
# sizes off every kernel's grid of fast cases: a width and head sizes that are no multiples of 8, sixteen and twenty-four
# maps on one kv head, as many kv heads as heads, values wider than two maps, every expert chosen, five taps
BISUDRA_E = {
    "architecture": "Bisudra", "vocab": 77, "width": 50, "norm": {"eps": 1e-5}, "canon": {"taps": 5},
    "token_side": {"dim": 3}, "initializer_range": 0.1,
    "layers": [
        {"type": "attention", "mixer": _att(8, 1, 12, 10, 0.21, 0.55, window=50, rot=(1000.0, 6)), "mlp": _dense(30)},
        {"type": "attention", "mixer": _att(12, 1, 6, 20, 0.33, 0.15), "mlp": _moe(10, 5, 5)},
        {"type": "attention", "mixer": _att(5, 5, 32, 72, 0.1, 0.45, window=300, rot=(10000.0, 32)), "mlp": None},
    ],
}
# nothing routed and no convolution: every part lets a short prompt run as a recorded pass padded to a whole page
BISUDRA_F = {
    "architecture": "Bisudra", "vocab": 90, "width": 72, "norm": {"eps": 1e-5}, "token_side": {"dim": 9},
    "initializer_range": 0.09,
    "layers": [
        {"type": "attention", "mixer": _att(2, 1, 32, 64, 0.15, 0.35, window=80, rot=(2000.0, 12)), "mlp": _dense(100)},
        {"type": "attention", "mixer": _att(3, 3, 16, 24, 0.3, 0.65, rot=(700.0, 16)), "mlp": None},
        {"type": "attention", "mixer": _att(4, 2, 24, 40, 0.2, 0.5, window=31), "mlp": _dense(56)},
    ],
}
CONFIGS = {"A": BISUDRA_A, "B": BISUDRA_B, "C": BISUDRA_C, "D": BISUDRA_D, "E": BISUDRA_E, "F": BISUDRA_F}


ROUTER_BIAS_STD = 1.0


def make_bisudra_dir(tmp_path: Path, config_json: dict, seed: int = 0, edit=None) -> Path:
    """A model folder with random bfloat16 weights.  Norm weights get a visible spread, norm biases and the gates'
    biases too; the four vectors behind lambda are large enough for lambda to differ from ``diff`` in the first digit; the routers'
    biases lie wide apart, so that few choices are close calls.
    ``edit(tensors)`` may change the float32 tensors before they are rounded and written."""
    from gpullama3.java_b200.config import config_from_dict
    from gpullama3.java_b200.weights import random_checkpoint, write_safetensors

    cfg = config_from_dict(config_json)
    tag = abs(hash(json.dumps([config_json, seed, getattr(edit, "__name__", None)], sort_keys=True))) % 10 ** 10
    out = Path(tmp_path) / f"bisudra_{tag}"
    if (out / "model.safetensors").is_file():
        return out
    out.mkdir(parents=True, exist_ok=True)
    where = "cuda" if torch.cuda.is_available() else "cpu"
    tensors = {}
    for n, t in random_checkpoint(cfg, seed, dtype=torch.float32, norm_std=0.2, device=where):
        tensors[n] = t.cpu().to(torch.float32)
    for name in tensors:
        if name.rsplit(".", 1)[-1] in ("lq1", "lk1", "lq2", "lk2"):
            tensors[name] = tensors[name] * 3.0
        if name.endswith(".router.b"):       # wide apart: most choices are then far from a tie, the input still decides some
            tensors[name] = tensors[name] * (ROUTER_BIAS_STD / 0.02)
    if edit is not None:
        edit(tensors)
    (out / "config.json").write_text(json.dumps(cfg.to_dict(), indent=2))
    write_safetensors(out / "model.safetensors", {n: t.to(torch.bfloat16) for n, t in tensors.items()})
    return out


def plain_inputs(model_dir: Path):
    """config.json as a dict and the weights by checkpoint name as float32, read with the safetensors package (not with
    the product's reader)."""
    from safetensors.torch import load_file

    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    weights = {k: v.to(torch.float32) for k, v in load_file(str(Path(model_dir) / "model.safetensors")).items()}
    return cfg, weights


class Reference:
    """The plain implementation's logits of a request and, per position and logit, how far they move when what every
    product reads and returns is rounded to bfloat16: a sublayer's result is gated and normed before it joins the stream,
    so where it is small by chance the norm magnifies any rounding, and a routed layer's choice can flip; the plain
    implementation shows both itself."""

    def __init__(self, logits: torch.Tensor, moved: torch.Tensor, settled: torch.Tensor | None = None):
        """``settled`` [T] bool: no routed layer had a close call at this position or at one before it (a close call:
        the last chosen expert's logit leads the best one left out by less than CLOSE_CALL of what a relative change
        of the router's input could undo).  Behind a close call a bfloat16 run may have picked the other expert, and
        attention carries that to every later position."""
        self.logits, self.moved = logits, moved
        self.settled = settled if settled is not None else torch.ones(logits.shape[0], dtype=torch.bool)

    def __getitem__(self, index):
        return Reference(self.logits[index], self.moved[index], self.settled[index])


def reference(cfg, weights, tokens) -> Reference:
    import plain_bisudra

    margins: list = []
    exact = plain_bisudra.forward(cfg, weights, tokens, margins=margins)
    rounded = plain_bisudra.forward(cfg, weights, tokens, reads=lambda h: h.to(torch.bfloat16).to(h.dtype))
    close = torch.zeros(exact.shape[0], dtype=torch.bool)
    for m in margins:
        close |= m < CLOSE_CALL
    settled = torch.cumsum(close.to(torch.int64), dim=0) == 0
    return Reference(exact, (rounded - exact).abs(), settled)


CLOSE_CALL = 0.03


def assert_logits(got: torch.Tensor, ref, dtype, what: str = "") -> None:
    """float32: accumulation-order noise only, at every position.  bfloat16: the engine rounds activations between its
    kernels, the plain implementation does not round at all; what is allowed is a few roundings' worth relative to the
    largest logit plus, against a ``Reference``, three times what the roundings of its products move the plain
    implementation's own result at that position; a small share of positions may lie outside (a routing that flipped)."""
    moved = settled = None
    if isinstance(ref, Reference):
        ref, moved, settled = ref.logits, ref.moved.detach().to("cpu", torch.float64), ref.settled
    got = got.detach().to("cpu", torch.float64)
    ref = ref.detach().to("cpu", torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = float(ref.abs().max()) + 1e-30
    err = (got - ref).abs()
    if dtype == torch.float32:
        allowed = 5e-5 * scale + (1e-3 * moved.amax(dim=-1) if moved is not None else 0.0)
        worst = err.amax(dim=-1)
        over = worst - allowed
        assert float(over.max()) <= 0.0, (f"{what}: max err {float(worst.max()):.3e} vs scale {scale:.3e} "
                                          f"(position {int(over.argmax())})")
        return
    if settled is not None and dtype != torch.float32:
        # behind a routed layer's close call the run may have picked the other expert: those positions must be sane,
        # the ones before it are held to the bound (the float32 run is held to it everywhere)
        assert float(err.max()) <= 2.0 * scale, f"{what}: max err {float(err.max()):.3e} vs scale {scale:.3e}"
        if not bool(settled.any()):
            return
        err, ref = err[settled], ref[settled]
        moved = moved[settled] if moved is not None else None
    worst, mean = err.amax(dim=-1), err.mean(dim=-1)
    if moved is None:
        bad = (worst > 0.08 * scale) | (mean > 0.012 * scale)
    else:
        bad = (worst > 0.08 * scale + 3.0 * moved.amax(dim=-1)) | (mean > 0.012 * scale + 3.0 * moved.mean(dim=-1))
    allowed = max(1, int(0.12 * bad.numel())) if bad.numel() >= 3 else 0
    assert int(bad.sum()) <= allowed, (f"{what}: {int(bad.sum())} of {bad.numel()} positions outside "
                                       f"(max err {float(err.max()):.3e}, scale {scale:.3e})")
    typical = 0.04 * scale + (3.0 * float(moved.amax(dim=-1).median()) if moved is not None else 0.0)
    assert float(worst.median()) <= typical, f"{what}: median of the worst errors {float(worst.median()):.3e} vs scale {scale:.3e}"
