"""Bisudra's mechanisms one at a time, each against its function of the plain implementation: the kernel that gates
and norms a sublayer's result into the stream, the mix over the levels, the token input's gate, the activation with its
bias, the rows of two maps laid side by side, the difference of two maps with its norm and gate, differential attention
as a part alone (prompts, portions and single tokens, with a score made to stand out so that one far key carries the
result), the dense feed-forward, the router with its bias, and the block alone."""

import pytest
import torch

import plain_bisudra as P
from gpullama3.java_b200.cache import KVCacheNeed, SequenceCache

pytestmark = pytest.mark.gpu
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
F = torch.float64
DEV = "cuda"


def _close(got, ref, dtype, what, f32=2e-5, bf16=2e-2):
    got, ref = got.detach().cpu().to(F), ref.detach().cpu().to(F)
    scale = float(ref.abs().max()) + 1e-30
    err = float((got - ref).abs().max())
    assert err <= (f32 if dtype == torch.float32 else bf16) * scale, f"{what}: {err:.3e} vs scale {scale:.3e}"


def _ctx(cache, dtype, slots, token_lists):
    from gpullama3.java_b200.engine.step import build_context
    start = [cache.length(s) for s in slots]
    cache.reserve([(s, len(t)) for s, t in zip(slots, token_lists)])
    ctx, _ = build_context(dtype, torch.device(DEV), cache, slots, start, token_lists, [])
    return ctx


@DTYPES
@pytest.mark.parametrize("rows, dim", [(5, 48), (3, 640), (300, 1024), (2, 8192), (2, 8448), (7, 1), (4, 257)])
@pytest.mark.parametrize("gated, centred, result_bias", [(True, True, True), (True, True, False), (False, False, False), (True, False, True)])
@pytest.mark.parametrize("pad, gate_type", [(3, None), (4, None), (8, torch.float32)], ids=["ragged", "whole fours", "32-bit gate"])
def test_gated_norm_into_the_stream(dtype, rows, dim, gated, centred, result_bias, pad, gate_type):
    """``pad``: further columns of the gate's rows (rows of whole fours go four numbers at a time)."""
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(rows * dim + gated)
    x, y = torch.randn(rows, dim, generator=g) * 4, torch.randn(rows, dim, generator=g) * 0.01 + 0.02
    r = (torch.randn(rows, dim + pad, generator=g) * 2).to(gate_type or dtype)
    w, b, rb, yb = (torch.randn(dim, generator=g) for _ in range(4))
    yb = yb * 0.01
    xd, yd = x.to(DEV), y.to(DEV)
    cast = torch.empty((rows, dim), dtype=dtype, device=DEV)
    ops.gated_norm_step(yd, w.to(DEV), b.to(DEV) if centred else None, xd, 1e-5, gate=r.to(DEV) if gated else None,
                        gate_bias=rb.to(DEV) if gated else None, y_bias=yb.to(DEV) if result_bias else None, cast=cast,
                        center=centred)
    z = y.to(F) + (yb.to(F) if result_bias else 0.0)
    if gated:
        z = z * torch.sigmoid(r[:, :dim].to(F) + rb.to(F))
    normed = P.layer_norm(z, w.to(F), b.to(F), 1e-5) if centred else P.over_root_mean_square(z, 1e-5) * w.to(F)
    ref = x.to(F) + normed
    _close(xd, ref, torch.float32, "stream", f32=2e-5 if dim > 1 else 1e-3)
    assert float(yd.abs().max()) == 0.0
    assert torch.equal(cast.float().cpu(), xd.cpu().to(dtype).float())


@DTYPES
@pytest.mark.parametrize("rows, dim, levels", [(5, 48, 1), (3, 640, 4), (130, 100, 9), (1, 7, 2)])
def test_mix_over_the_levels(dtype, rows, dim, levels):
    """Level after level: what each round leaves as the stream is the mix of everything kept so far."""
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(rows + dim)
    kept = torch.full((levels + 1, rows, dim), float("nan"), device=DEV)
    results = []
    for n in range(levels + 1):
        newest = torch.randn(rows, dim, generator=g) * (n + 1)
        c = torch.randn(n + 1, generator=g)
        x = newest.to(DEV)
        cast = torch.empty((rows, dim), dtype=dtype, device=DEV)
        ops.depth_average(kept, n, c.to(DEV), x, cast=cast)
        results.append(newest.to(F))
        _close(x, P.depth_average(results, c.to(F)), torch.float32, f"level {n}", f32=1e-5)
        assert torch.equal(kept[n].cpu(), newest) and torch.equal(cast.float().cpu(), x.cpu().to(dtype).float())


@DTYPES
@pytest.mark.parametrize("rows, dim, n", [(5, 48, 1), (3, 640, 4), (9, 50, 3), (2, 8448, 2)])
def test_last_step_of_a_layer_files_its_level_and_mixes(dtype, rows, dim, n):
    """The norm-and-add kernel with levels: what it leaves equals the plain step followed by the plain mix."""
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(rows + dim + n)
    x, y = torch.randn(rows, dim, generator=g) * 4, torch.randn(rows, dim, generator=g)
    w, c = torch.randn(dim, generator=g), torch.randn(n + 1, generator=g)
    kept = torch.randn(n + 2, rows, dim, generator=g)
    levels = kept.to(DEV)
    xd, yd = x.to(DEV), y.to(DEV)
    cast = torch.empty((rows, dim), dtype=dtype, device=DEV)
    ops.gated_norm_step(yd, w.to(DEV), None, xd, 1e-5, center=False, cast=cast, levels=levels, n=n, coefficients=c.to(DEV))
    newest = x.to(F) + P.over_root_mean_square(y.to(F), 1e-5) * w.to(F)
    ref = P.depth_average([kept[j].to(F) for j in range(n)] + [newest], c.to(F))
    _close(xd, ref, torch.float32, "stream", f32=1e-5)
    _close(levels[n], newest, torch.float32, "level", f32=1e-5)
    assert torch.equal(levels[n + 1].cpu(), kept[n + 1]) and torch.equal(levels[:n].cpu(), kept[:n])
    assert torch.equal(cast.float().cpu(), xd.cpu().to(dtype).float()) and float(yd.abs().max()) == 0.0


@DTYPES
@pytest.mark.parametrize("rows, n, width, columns", [(5, 12, 16, 36), (3, 5, 8, 5), (70, 40, 40, 200), (2, 1, 8, 3)])
def test_token_gate(dtype, rows, n, width, columns):
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(rows + n)
    a = (torch.randn(rows, width + 8, generator=g) * 2).to(dtype)
    table = torch.randn(30, columns, generator=g).to(dtype)
    lo = columns - n
    tokens = torch.randint(0, 30, (rows,), generator=g, dtype=torch.int32)
    out = torch.full((rows, width), float("nan"), dtype=dtype, device=DEV)
    ops.token_gate_rows(a.to(DEV), tokens.to(DEV), table.to(DEV)[:, lo:lo + n], out, n)
    ref = P.gelu_tanh(a[:, :n].to(F)) * table[tokens.long()][:, lo:lo + n].to(F)
    _close(out[:, :n], ref, dtype, "gated numbers", f32=1e-5, bf16=1e-2)
    assert width == n or float(out[:, n:].float().abs().max()) == 0.0


@DTYPES
def test_bias_and_squared_relu(dtype):
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(5)
    u = (torch.randn(9, 2100, generator=g) * 3).to(dtype)
    b = torch.randn(2100, generator=g)
    ud = u.to(DEV)
    ops.bias_act_rows(ud, b.to(DEV))
    _close(ud, P.squared_relu(u.to(F) + b.to(F)), dtype, "activation", f32=1e-6, bf16=1e-2)


@DTYPES
@pytest.mark.parametrize("heads, d, d_pad, gated", [(4, 32, 32, True), (3, 24, 64, True), (1, 128, 128, False), (5, 8, 32, True)])
def test_difference_of_two_maps(dtype, heads, d, d_pad, gated):
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(heads * d)
    T = 11
    maps = torch.randn(T, heads, 2, d_pad, generator=g).to(dtype)
    gate = (torch.randn(T, heads * d + 5, generator=g) * 2).to(dtype)
    out = torch.empty((T, heads * d), dtype=dtype, device=DEV)
    lam, diff, eps = 0.83, 0.3, 1e-5
    ops.differential_heads(maps.reshape(T, -1).to(DEV), gate.to(DEV) if gated else None, out, heads, d, d_pad, lam, 1.0 - diff, eps)
    o = maps[:, :, 0, :d].to(F) - lam * maps[:, :, 1, :d].to(F)
    ref = P.over_root_mean_square(o, eps) * (1.0 - diff)
    if gated:
        ref = ref * torch.sigmoid(gate[:, :heads * d].to(F)).reshape(T, heads, d)
    _close(out, ref.reshape(T, -1), dtype, "heads", f32=1e-5, bf16=1e-2)


def _mixer(hidden, H, G, d, dv, scale, diff, window, rot, dtype, seed, loud=None):
    """A differential attention part with random weights and the plain implementation's view of them.  ``loud``: scale
    on the query and key norms' weights, which makes the scores peaked (one key carries the result)."""
    from gpullama3.java_b200.parts import DifferentialAttention, NoPositionEncoding, RotaryPositionEncoding

    position = RotaryPositionEncoding(d, rot[0], "interleaved", rotary_dim=rot[1]) if rot else NoPositionEncoding()
    att = DifferentialAttention(hidden, H, G, d, dv, scale, diff, 1e-5, position, window)
    specs = att.parameters()
    assert specs["q"].shape == (H * 2 * d, hidden) and specs["k"].shape == (G * 2 * d, hidden) and specs["v"].shape == (G * dv, hidden)
    g = torch.Generator().manual_seed(seed)
    w = {k: (torch.randn(s.shape, generator=g) * 0.2).to(torch.bfloat16) for k, s in specs.items()}
    for n in ("q_norm", "k_norm"):
        w[n] = (1.0 + 0.3 * torch.randn(d, generator=g)).to(torch.bfloat16) * (loud or 1.0)
    att.load(w, dtype, DEV)
    names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "lq1": "lq1", "lk1": "lk1",
             "lq2": "lq2", "lk2": "lk2"}
    W = {"x.mix." + names[k]: t.to(F) for k, t in w.items()}
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale, "diff": diff}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return att, W, m, g


SHAPES = [  # hidden, heads, kv heads, dim per map, value dim, scale, diff, window, (rotation base, dims)
    (72, 4, 2, 16, 32, 0.3, 0.4, None, (1e4, 16)),
    (40, 3, 1, 32, 64, 0.11, 0.5, 50, (500.0, 8)),
    (100, 6, 3, 24, 16, 0.25, 0.8, 64, None),
    (64, 2, 2, 64, 128, 0.125, 0.2, 65, (1e6, 64)),
    (48, 8, 1, 8, 8, 0.5, 0.6, 3, (10.0, 2)),
    (56, 1, 1, 40, 56, 0.2, 0.1, 129, (100.0, 20)),
    (64, 2, 1, 72, 200, 0.1, 0.3, 70, (1e4, 36)),      # rows of 208 numbers: wider than any tensor-core attention kernel takes
]


@DTYPES
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s[:5])))
def test_differential_attention_alone(dtype, shape):
    """Three sequences of unequal length as one prompt step; then the same sequences in portions and single tokens."""
    hidden, H, G, d, dv, scale, diff, window, rot = shape
    att, W, m, g = _mixer(hidden, H, G, d, dv, scale, diff, window, rot, dtype, seed=H * d)
    D = att.row_dim
    assert att.cache_need() == KVCacheNeed(G, D, window) and D >= max(2 * d, dv)
    lens = [70, 5, 131]
    xs = [torch.randn(n, hidden, generator=g).to(dtype).float() for n in lens]
    refs = [P.differential_attention(x.to(F), W, "x.", m, 1e-5) for x in xs]
    lam = P.differential_weight(W, "x.", diff)
    assert abs(att.weight - lam) <= 1e-5 * max(1.0, abs(lam))
    for portions in ([lens], [[64, 3, 100], [1, 1, 1], [1, 1, 1], [4, 0, 29]]):
        cache = SequenceCache({0: att.cache_need()}, max_tokens=64 * 8, dtype=dtype, device=DEV, window_slack=128)
        slots = [cache.acquire() for _ in lens]
        at = [0, 0, 0]
        got = [[] for _ in lens]
        for step in portions:
            live = [i for i, n in enumerate(step) if n]
            ctx = _ctx(cache, dtype, [slots[i] for i in live], [[0] * step[i] for i in live])
            y = torch.zeros(sum(step), hidden, device=DEV)
            att.forward(torch.cat([xs[i][at[i]:at[i] + step[i]] for i in live]).to(dtype).to(DEV), ctx, cache.view(0), y)
            o = 0
            for i in live:
                got[i].append(y[o:o + step[i]].cpu())
                o += step[i]
                at[i] += step[i]
                cache.commit(slots[i], step[i])
        for i in range(3):
            n = at[i]
            _close(torch.cat(got[i]), refs[i][:n], dtype, f"sequence {i}, {len(portions)} steps", f32=5e-5, bf16=4e-2)


@DTYPES
def test_one_far_key_carries_the_result(dtype):
    """Peaked scores: with loud norm weights the softmax of each map rests on one or two keys, anywhere among 300."""
    hidden, H, G, d, dv = 48, 2, 1, 16, 32
    att, W, m, g = _mixer(hidden, H, G, d, dv, 0.9, 0.5, None, (1e4, 8), dtype, seed=3, loud=4.0)
    x = torch.randn(300, hidden, generator=g).to(dtype).float()
    ref = P.differential_attention(x.to(F), W, "x.", m, 1e-5)
    hidden_keys = P.differential_attention(x.to(F), W, "x.", dict(m, mask={"size": 150}), 1e-5)
    assert float((hidden_keys[200:] - ref[200:]).abs().amax(dim=1).median()) > 0.1 * float(ref.abs().max())
    cache = SequenceCache({0: att.cache_need()}, max_tokens=64 * 6, dtype=dtype, device=DEV, window_slack=128)
    slot = cache.acquire()
    got = []
    for lo, hi in [(0, 250)] + [(t, t + 1) for t in range(250, 300)]:
        ctx = _ctx(cache, dtype, [slot], [[0] * (hi - lo)])
        y = torch.zeros(hi - lo, hidden, device=DEV)
        att.forward(x[lo:hi].to(dtype).to(DEV), ctx, cache.view(0), y)
        got.append(y.cpu())
        cache.commit(slot, hi - lo)
    # (bfloat16: a rounding of a query or key moves a peaked score by a tenth and with it a softmax weight; a few
    # positions feel that, the typical one does not)
    _close(torch.cat(got), ref, dtype, "peaked scores", f32=1e-4, bf16=0.2)
    worst = (torch.cat(got).to(F) - ref).abs().amax(dim=1)
    assert float(worst.median()) <= (1e-4 if dtype == torch.float32 else 2e-2) * float(ref.abs().max())


@DTYPES
def test_dense_feed_forward_alone(dtype):
    from gpullama3.java_b200.parts import DenseFeedForward

    ff = DenseFeedForward(hidden_size=72, intermediate_size=200)
    g = torch.Generator().manual_seed(2)
    w = {k: (torch.randn(s.shape, generator=g) * 0.2).to(torch.bfloat16) for k, s in ff.parameters().items()}
    ff.load(w, dtype, DEV)
    x = torch.randn(9, 72, generator=g).to(dtype).float()
    W = {"x.mlp.up": w["up"].to(F), "x.mlp.up.b": w["up_bias"].to(F), "x.mlp.down": w["down"].to(F), "x.mlp.down.b": w["down_bias"].to(F)}
    ref = P.dense_feed_forward(x.to(F), W, "x.")

    class Ctx:
        def __init__(self):
            self.dtype = dtype

        def empty(self, shape, dt):
            return torch.empty(tuple(shape), dtype=dt, device=DEV)

    y = torch.zeros(9, 72, device=DEV)
    ff.forward(x.to(dtype).to(DEV), Ctx(), y)
    _close(y, ref, dtype, "dense feed-forward", f32=2e-5, bf16=3e-2)
    y.zero_()
    ff.forward(x.to(dtype).to(DEV), Ctx(), y, add_result_bias=False)
    _close(y + ff.result_bias(), ref, dtype, "without its last bias", f32=2e-5, bf16=3e-2)


@pytest.mark.parametrize("experts, top, width", [(10, 3, 64), (5, 1, 40), (7, 7, 33), (64, 8, 128)])
def test_router_with_bias(experts, top, width):
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(experts)
    h = torch.randn(50, width, generator=g)
    W = {"x.mlp.router": torch.randn(experts, width, generator=g).to(F), "x.mlp.router.b": (3 * torch.randn(experts, generator=g)).to(F)}
    chosen = torch.empty((50, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((50, top), dtype=torch.float32, device=DEV)
    ops.moe_route(h.to(DEV), W["x.mlp.router"].float().to(DEV), chosen, weights, 1, 1, 0.0, None, W["x.mlp.router.b"].float().to(DEV))
    ref_c, ref_w = P.router_choice(h.to(F), W, "x.", top)
    assert torch.equal(chosen.cpu().long(), ref_c)       # (largest first, as the plain implementation's order)
    _close(weights, ref_w, torch.float32, "weights", f32=1e-5)
    without = torch.empty_like(chosen)
    ops.moe_route(h.to(DEV), W["x.mlp.router"].float().to(DEV), without, weights, 1, 1, 0.0)
    assert not torch.equal(without.cpu(), chosen.cpu())      # the bias decides


@DTYPES
@pytest.mark.parametrize("taps, side, mlp", [(3, 10, "dense"), (0, 0, None), (1, 8, "moe"), (4, 0, "dense")])
def test_block_alone(dtype, taps, side, mlp):
    """One block between a random stream and the plain implementation's layer function, in two steps that continue one
    another (the second brings one token per sequence), with the mix over two levels behind it."""
    from gpullama3.java_b200.config.base import LayerSpec, PartSpec
    from gpullama3.java_b200.parts import build_block

    hidden, vocab = 64, 50
    mix = {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 24, "scale": 0.3, "diff": 0.45, "mask": {"size": 9}, "rot": {"base": 100.0, "dims": 4}}
    norm = PartSpec("norm", "layernorm", {"dim": hidden, "eps": 1e-5})
    parts = {"mixer": PartSpec("mixer", "differential_attention", {
        "hidden_size": hidden, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16, "value_dim": 24, "scale": 0.3, "diff": 0.45,
        "norm_eps": 1e-5, "window": 9,
        "position": PartSpec("position", "rope", {"head_dim": 16, "theta": 100.0, "pairing": "interleaved", "rotary_dim": 4})}),
        "mixer_norm": norm}
    record = None
    if mlp == "dense":
        parts.update(feed_forward=PartSpec("feed_forward", "dense", {"hidden_size": hidden, "intermediate_size": 40}), feed_forward_norm=norm)
        record = {"kind": "dense", "ff": 40}
    elif mlp == "moe":
        parts.update(feed_forward=PartSpec("feed_forward", "routed", {"hidden_size": hidden, "intermediate_size": 16, "n_experts": 3,
                                                                       "top": 2, "weight_eps": 0.0, "router_bias": True}),
                     feed_forward_norm=norm)
        record = {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 2}}
    block = build_block(LayerSpec("gated_residual", parts, {"hidden_size": hidden, "conv_taps": taps, "side_dim": side,
                                                            "side_columns": (side, 3 * side), "vocab_size": vocab, "side_eps": 1e-5,
                                                            "depth": (0, 1)}))
    from gpullama3.java_b200.parts.base import all_parts
    g = torch.Generator().manual_seed(taps + side)
    W, by_part = {}, {}
    plain_names = {"mixer_conv": "l1.canon1", "mixer_gate": "l1.rg1", "mixer_gate_bias": "l1.rg1.b", "feed_forward_gate": "l1.rg2",
                   "feed_forward_gate_bias": "l1.rg2.b", "side_table": "side.embed", "side_gate": "l1.side.gate",
                   "side_proj": "l1.side.proj", "side_norm": "l1.side.norm", "depth_mix": "l1.dwa",
                   "mixer_norm.weight": "l1.norm1", "mixer_norm.bias": "l1.norm1.b", "feed_forward_norm.weight": "l1.norm2",
                   "feed_forward_norm.bias": "l1.norm2.b", "feed_forward.up": "l1.mlp.up", "feed_forward.up_bias": "l1.mlp.up.b",
                   "feed_forward.down": "l1.mlp.down", "feed_forward.down_bias": "l1.mlp.down.b",
                   "feed_forward.router": "l1.mlp.router", "feed_forward.router_bias": "l1.mlp.router.b"}
    for path, part in [("", block)] + [(p + ".", q) for p, q in all_parts(block).items()]:
        mine = {}
        for k, s in part.parameters().items():
            std = 1.0 if k in ("side_table",) else 0.3
            t = (torch.randn(s.shape, generator=g) * std + (1.0 if "norm" in path + k and "bias" not in k else 0.0)).to(torch.bfloat16)
            mine[k] = t
            name = path + k
            if name.startswith("mixer.") and name != "mixer.position":
                plain = "l1.mix." + {"q_norm": "q.norm", "k_norm": "k.norm"}.get(k, k)
            elif name.startswith("feed_forward.e"):
                plain = "l1.mlp." + k
            else:
                plain = plain_names[name]
            W[plain] = t.to(F)
        part.load(mine, dtype, DEV)
    config = {"norm": {"eps": 1e-5}, "canon": {"taps": taps} if taps else None, "token_side": {"dim": side} if side else None,
              "layers": [None, {"mixer": mix, "mlp": record}]}
    lens = [21, 6]
    tokens = [torch.randint(0, vocab, (n,), generator=g) for n in lens]
    xs = [(torch.randn(n, hidden, generator=g) * 3).float() for n in lens]
    refs = []
    for x, t in zip(xs, tokens):
        X = P.layer(x.to(F), t, W, config, 1)
        refs.append(P.depth_average([x.to(F), X], W["l1.dwa"]))
    cache = SequenceCache({0: block.cache_need()}, max_tokens=64 * 4, dtype=dtype, device=DEV, window_slack=64)
    slots = [cache.acquire() for _ in lens]
    got = [[], []]
    for step in ([20, 5], [1, 1]):
        at = [sum(r.shape[0] for r in got[i]) for i in range(2)]
        toks = [tokens[i][at[i]:at[i] + step[i]].tolist() for i in range(2)]
        ctx = _ctx(cache, dtype, slots, toks)
        stream = torch.cat([xs[i][at[i]:at[i] + step[i]] for i in range(2)]).to(DEV)
        handed = block.forward(stream, ctx, cache.view(0))
        assert torch.equal(handed.data.float(), stream.to(dtype).float())
        o = 0
        for i in range(2):
            got[i].append(stream[o:o + step[i]].cpu())
            o += step[i]
            cache.commit(slots[i], step[i])
    for i in range(2):
        _close(torch.cat(got[i]), refs[i], dtype, f"sequence {i}", f32=5e-5, bf16=5e-2)
