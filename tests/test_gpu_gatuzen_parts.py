"""Gatuzen's mechanisms one at a time, each against its function of the plain implementation: the norm in groups, the
kernel between two sublayers, the convolution in its general form, the scan without the delta correction in both of its
uses, the gated output norm with the gate first, rotation by position with stretched frequencies, routing by table,
and one-layer models that hold nothing but one kind of mixer (with a far key made to stand out for the attention)."""
import pytest
import torch

import plain_gatuzen as P
from conftest import random_prompts
from gatuzen_helpers import assert_logits, make_gatuzen_dir, plain_inputs

pytestmark = pytest.mark.gpu
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
F = torch.float64


def _close(got, ref, dtype, what, f32=2e-5, bf16=2e-2):
    got, ref = got.detach().cpu().to(F), ref.detach().cpu().to(F)
    scale = float(ref.abs().max()) + 1e-30
    err = float((got - ref).abs().max())
    assert err <= (f32 if dtype == torch.float32 else bf16) * scale, f"{what}: {err:.3e} vs scale {scale:.3e}"


@DTYPES
@pytest.mark.parametrize("rows, dim, groups", [(5, 48, 3), (3, 50, 1), (1300, 1024, 4), (7, 5000, 2), (2, 7, 7), (4, 96, 16)])
def test_norm_in_groups(dtype, rows, dim, groups):
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(rows + dim)
    x = torch.randn(rows, dim, generator=g) * torch.linspace(0.1, 30.0, dim)     # the parts differ in size by far
    w = torch.randn(dim, generator=g)
    out = torch.empty((rows, dim), dtype=dtype, device="cuda")
    ops.group_rmsnorm(x.cuda(), w.cuda(), out, 1e-5, groups)
    _close(out, P.grouped_rms_norm(x.to(F), w.to(F), groups, 1e-5), dtype, "norm in groups", f32=1e-5, bf16=1e-2)
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32)
    out2 = torch.empty((2, dim), dtype=dtype, device="cuda")
    ops.group_rmsnorm(x.cuda(), w.cuda(), out2, 1e-5, groups, pick.cuda())
    assert torch.equal(out2.cpu(), out.cpu()[pick.long()])


@pytest.mark.parametrize("rows, dim, groups", [(5, 48, 3), (300, 1024, 4), (3, 50, 1), (2, 2048, 1), (3, 384, 3), (4, 8192, 2),
                                               (2, 3072, 4), (5, 1280, 2), (3, 128, 1), (2, 8320, 1)])
@pytest.mark.parametrize("offset, follows", [(False, False), (True, True), (False, True)])
def test_between_two_sublayers(rows, dim, groups, offset, follows):
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(rows * dim)
    x, y = torch.randn(rows, dim, generator=g) * 4, torch.randn(rows, dim, generator=g) * 0.01
    wb, wn, off = torch.randn(dim, generator=g), torch.randn(dim, generator=g), torch.randn(dim, generator=g)
    xd, yd = x.cuda(), y.cuda()
    out = torch.empty((rows, dim), dtype=torch.float32, device="cuda") if follows else None
    ops.sandwich_step(yd, wb.cuda(), 0.7, xd, 1e-5, groups, offset=off.cuda() if offset else None,
                      next_weight=wn.cuda() if follows else None, out=out)
    ref = x.to(F) + 0.7 * P.grouped_rms_norm(y.to(F), wb.to(F), groups, 1e-5) + (off.to(F) if offset else 0.0)
    _close(xd, ref, torch.float32, "stream", f32=1e-6)
    assert float(yd.abs().max()) == 0.0
    if follows:
        _close(out, P.grouped_rms_norm(ref, wn.to(F), groups, 1e-5), torch.float32, "next input", f32=1e-5)


@DTYPES
@pytest.mark.parametrize("taps, channels", [(4, 48), (1, 50), (2, 7), (3, 1024)])
@pytest.mark.parametrize("bias, act, add", [(False, None, True), (True, "silu", False)])
def test_convolution_carries_its_inputs(dtype, taps, channels, bias, act, add):
    """Three sequences of 9, 1 and 30 tokens, cut into steps of unequal portions (one shorter than the taps)."""
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(taps * channels)
    lens = [9, 1, 30]
    xs = [torch.randn(n, channels, generator=g).to(dtype).float() for n in lens]
    w = torch.randn(channels, taps, generator=g)
    b = torch.randn(channels, generator=g) if bias else None
    refs = []
    for x in xs:
        r = P.causal_conv(x.to(F), w.to(F), b.to(F) if bias else None)
        r = P.silu(r) if act else r
        refs.append(r + x.to(F) if add else r)
    state = torch.zeros(5, max(taps - 1, 1) * channels + 3, device="cuda")
    slots = [4, 0, 2]
    got = [[] for _ in lens]
    at = [0, 0, 0]
    for portions in ([2, 1, 5], [1, 0, 1], [6, 0, 24]):
        live = [i for i, n in enumerate(portions) if n]
        x = torch.cat([xs[i][at[i]:at[i] + portions[i]] for i in live]).to(dtype).cuda()
        cu = torch.tensor([0] + list(torch.tensor([portions[i] for i in live]).cumsum(0)), dtype=torch.int32).cuda()
        seq = torch.cat([torch.full((portions[i],), j, dtype=torch.int32) for j, i in enumerate(live)]).cuda()
        out = torch.empty_like(x)
        ops.causal_conv(x, w.cuda(), state, torch.tensor([slots[i] for i in live], dtype=torch.int32).cuda(), seq, cu, out,
                        channels, bias=b.cuda() if bias else None, activation=act, add_input=add)
        o = 0
        for i in live:
            got[i].append(out[o:o + portions[i]].float().cpu())
            o += portions[i]
            at[i] += portions[i]
    for i in range(3):
        _close(torch.cat(got[i]), refs[i], dtype, f"sequence {i}", f32=1e-5, bf16=2e-2)


@DTYPES
@pytest.mark.parametrize("taps, channels", [(4, 64), (2, 1024), (1, 50), (5, 36), (3, 7)])
@pytest.mark.parametrize("form", ["added", "bias and silu", "silu alone"])
def test_convolution_token_by_token(dtype, taps, channels, form):
    """Three sequences: a first portion of 5, 1 and 0 tokens in one step, then one token each per step (the kernel that
    also moves the state on), one sequence ending early and its slot taken by a new one."""
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(taps + channels)
    lens = [17, 9, 12, 6]
    xs = [torch.randn(n, channels, generator=g).to(dtype).float() for n in lens]
    w = torch.randn(channels, taps, generator=g)
    b = torch.randn(channels, generator=g) if form == "bias and silu" else None
    refs = []
    for x in xs:
        r = P.causal_conv(x.to(F), w.to(F), b.to(F) if b is not None else None)
        refs.append(r + x.to(F) if form == "added" else P.silu(r))
    state = torch.zeros(4, max(taps - 1, 1) * channels, device="cuda")
    slot = {0: 3, 1: 0, 2: 2, 3: 0}          # sequence 3 takes sequence 1's slot when that has ended
    got = [[] for _ in lens]
    at = [0, 0, 0, 0]

    def run(portions):
        live = [i for i in portions if portions[i]]
        x = torch.cat([xs[i][at[i]:at[i] + portions[i]] for i in live]).to(dtype).cuda()
        cu = torch.tensor([0] + list(torch.tensor([portions[i] for i in live]).cumsum(0)), dtype=torch.int32).cuda()
        seq = torch.cat([torch.full((portions[i],), j, dtype=torch.int32) for j, i in enumerate(live)]).cuda()
        out = torch.empty_like(x)
        kw = dict(bias=b.cuda() if b is not None else None, activation=None if form == "added" else "silu", add_input=form == "added")
        if form == "silu alone":
            ops.causal_conv_silu(x, w.cuda(), state, torch.tensor([slot[i] for i in live], dtype=torch.int32).cuda(), seq, cu, out, channels)
        else:
            ops.causal_conv(x, w.cuda(), state, torch.tensor([slot[i] for i in live], dtype=torch.int32).cuda(), seq, cu, out, channels, **kw)
        o = 0
        for i in live:
            got[i].append(out[o:o + portions[i]].float().cpu())
            o += portions[i]
            at[i] += portions[i]

    run({0: 5, 1: 1})
    while any(at[i] < lens[i] for i in (0, 1, 2)):
        run({i: 1 for i in (0, 1, 2) if at[i] < lens[i]})
        if at[1] == lens[1] and at[3] == 0:
            state[slot[3]].zero_()           # (what handing out a slot does)
            run({3: 2})
    while at[3] < lens[3]:
        run({3: 1})
    for i in range(4):
        _close(torch.cat(got[i]), refs[i], dtype, f"sequence {i}", f32=1e-5, bf16=2e-2)


@DTYPES
@pytest.mark.parametrize("dim, groups, taps", [(256, 2, 4), (1024, 4, 2), (384, 1, 1), (2048, 4, 4), (1280, 2, 5), (8192, 8, 3)])
@pytest.mark.parametrize("offset", [False, True])
def test_step_that_reads_for_the_next_sublayer(dtype, dim, groups, taps, offset):
    """Token by token for three sequences: the stream takes the normed result, and what the next sublayer reads is the
    normed stream plus its convolution over the tokens so far, the older inputs kept per slot."""
    from gpullama3.java_b200.kernels import ops

    assert ops.sandwich_step_conv_fits(dim, groups)
    g = torch.Generator().manual_seed(dim + taps)
    n, steps = 3, 7
    wb, wn, off = torch.randn(dim, generator=g), torch.randn(dim, generator=g), torch.randn(dim, generator=g)
    cw = torch.randn(dim, taps, generator=g)
    xs = torch.randn(steps, n, dim, generator=g) * 3
    ys = torch.randn(steps, n, dim, generator=g) * 0.02
    slots = torch.tensor([4, 1, 2], dtype=torch.int32)
    state = torch.zeros(6, max(taps - 1, 1) * dim, device="cuda")
    hs, outs = [], []
    for k in range(steps):
        xd, yd = xs[k].cuda(), ys[k].cuda()
        out = torch.empty((n, dim), dtype=dtype, device="cuda")
        ops.sandwich_step_conv(yd, wb.cuda(), 0.7, xd, 1e-5, groups, wn.cuda(), out, cw.cuda(), state, slots.cuda(),
                               offset=off.cuda() if offset else None, update_state=True)
        ref = xs[k].to(F) + 0.7 * P.grouped_rms_norm(ys[k].to(F), wb.to(F), groups, 1e-5) + (off.to(F) if offset else 0.0)
        _close(xd, ref, torch.float32, "stream", f32=1e-6)
        assert float(yd.abs().max()) == 0.0
        hs.append(P.grouped_rms_norm(ref, wn.to(F), groups, 1e-5))
        outs.append(out.float().cpu())
    h = torch.stack(hs)                       # [steps, n, dim]
    for i in range(n):
        ref = h[:, i] + P.causal_conv(h[:, i], cw.to(F), None)
        _close(torch.stack([o[i] for o in outs]), ref, dtype, f"sequence {i}", f32=1e-5, bf16=1e-2)
    # a step that must not write leaves the state as it is
    before = state.clone()
    ops.sandwich_step_conv(ys[0].cuda(), wb.cuda(), 0.7, xs[0].cuda(), 1e-5, groups, wn.cuda(),
                           torch.empty((n, dim), dtype=dtype, device="cuda"), cw.cuda(), state, slots.cuda(), update_state=False)
    assert torch.equal(state, before)


@DTYPES
@pytest.mark.parametrize("taps, channels", [(4, 64), (2, 520), (7, 36), (1, 8), (9, 12), (4, 30)])
@pytest.mark.parametrize("form", ["added", "bias and silu", "silu alone"])
def test_convolution_over_long_steps(dtype, taps, channels, form):
    """Steps of 154 and 200 tokens (threads then take runs of tokens): four sequences whose borders fall inside a run,
    one of a single token, the second step reading what the first left in the slots; input rows wider than the
    channels.  32-bit inputs with a rounded result as well as equal types."""
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(taps * channels + len(form))
    lens = [150, 3, 200, 1]
    xs = [torch.randn(n, channels, generator=g).to(dtype).float() for n in lens]
    w = torch.randn(channels, taps, generator=g)
    b = torch.randn(channels, generator=g) if form == "bias and silu" else None
    refs = []
    for x in xs:
        r = P.causal_conv(x.to(F), w.to(F), b.to(F) if b is not None else None)
        refs.append(r + x.to(F) if form == "added" else P.silu(r))
    in_dtype = torch.float32 if form == "added" else dtype
    state = torch.zeros(6, max(taps - 1, 1) * channels + 4, device="cuda")
    slots = [5, 1, 0, 3]
    got, at = [[] for _ in lens], [0] * 4
    for portions in ([61, 2, 90, 1], [89, 1, 110, 0]):
        live = [i for i, n in enumerate(portions) if n]
        x = torch.zeros(sum(portions), channels + 8, dtype=in_dtype, device="cuda")
        x[:, :channels] = torch.cat([xs[i][at[i]:at[i] + portions[i]] for i in live]).to(in_dtype)
        cu = torch.tensor([0] + list(torch.tensor([portions[i] for i in live]).cumsum(0)), dtype=torch.int32).cuda()
        seq = torch.cat([torch.full((portions[i],), j, dtype=torch.int32) for j, i in enumerate(live)]).cuda()
        out = torch.empty((sum(portions), channels), dtype=dtype, device="cuda")
        slot_ids = torch.tensor([slots[i] for i in live], dtype=torch.int32).cuda()
        if form == "silu alone":
            ops.causal_conv_silu(x, w.cuda(), state, slot_ids, seq, cu, out, channels)
        else:
            ops.causal_conv(x, w.cuda(), state, slot_ids, seq, cu, out, channels, bias=b.cuda() if b is not None else None,
                            activation=None if form == "added" else "silu", add_input=form == "added")
        o = 0
        for i in live:
            got[i].append(out[o:o + portions[i]].float().cpu())
            o += portions[i]
            at[i] += portions[i]
    for i in range(4):
        _close(torch.cat(got[i]), refs[i], dtype, f"sequence {i}", f32=1e-5, bf16=2e-2)
    assert float(state[2].abs().max()) == 0.0 and float(state[4].abs().max()) == 0.0    # slots no sequence holds


@DTYPES
@pytest.mark.parametrize("heads, kv_heads, dk, dv", [(2, 2, 48, 64), (4, 2, 24, 16), (1, 1, 130, 8), (3, 1, 8, 40)])
@pytest.mark.parametrize("kind", ["gated linear attention", "state space"])
def test_scan_without_correction(dtype, heads, kv_heads, dk, dv, kind):
    """Two sequences in two steps each; the second step continues from the state the first left in the slot."""
    from gpullama3.java_b200.kernels import ops

    if kind == "gated linear attention" and heads != kv_heads:
        pytest.skip("every head has its own queries and keys")
    g = torch.Generator().manual_seed(heads * dk + dv)
    lens = [37, 5]
    T = sum(lens)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype).float()
    q, k, v = rnd(T, kv_heads * dk) * 0.5, rnd(T, kv_heads * dk) * 0.5, rnd(T, heads * dv)
    per_head = kind == "state space"
    z = rnd(T, heads if per_head else heads * dk)
    bias = torch.randn(heads if per_head else heads * dk, generator=g) + (-2.0 if per_head else 3.0)
    a_log, skip = torch.randn(heads, generator=g) * 0.3 - 1.0, torch.randn(heads, generator=g)
    tau, q_scale = 7.0, dk ** -0.5
    # the plain recurrence, sequence by sequence and head by head
    ref = torch.zeros(T, heads * dv, dtype=F)
    start = 0
    for n in lens:
        sl = slice(start, start + n)
        for h in range(heads):
            kv = h // (heads // kv_heads)
            qq, kk = q[sl, kv * dk:(kv + 1) * dk].to(F), k[sl, kv * dk:(kv + 1) * dk].to(F)
            vv = v[sl, h * dv:(h + 1) * dv].to(F)
            if per_head:
                dt = P.softplus(z[sl, h].to(F) + bias[h].to(F))
                decay = torch.exp(-torch.exp(a_log[h].to(F)) * dt)[:, None].expand(n, dk)
                o = P.decayed_outer_product_scan(qq, kk, dt[:, None] * vv, decay) + skip[h].to(F) * vv
            else:
                decay = torch.sigmoid(z[sl, h * dk:(h + 1) * dk].to(F) + bias[h * dk:(h + 1) * dk].to(F)).pow(1.0 / tau)
                o = P.decayed_outer_product_scan(qq * q_scale, kk, vv, decay)
            ref[sl, h * dv:(h + 1) * dv] = o
        start += n
    state = torch.zeros(3, heads * dk * dv + 5, device="cuda")
    slots = torch.tensor([2, 0], dtype=torch.int32).cuda()
    got = torch.zeros(T, heads * dv)
    done = [0, 0]
    for portions in ([20, 2], [17, 3]):
        rows = torch.cat([torch.arange(sum(lens[:i]) + done[i], sum(lens[:i]) + done[i] + portions[i]) for i in range(2)])
        cu = torch.tensor([0, portions[0], portions[0] + portions[1]], dtype=torch.int32).cuda()
        take = lambda t: t[rows].to(dtype).cuda()
        out = torch.empty(len(rows), heads * dv, device="cuda")
        common = dict(decay_bias=bias.cuda(), decay_per_head=per_head)
        if per_head:
            ops.linear_scan(take(q), take(k), take(v), take(z), state, slots, cu, out, heads, kv_heads, dk, dv,
                            decay_kind=ops.DECAY_SOFTPLUS_RATE, a_log=a_log.cuda(), step_scales_value=True, skip=skip.cuda(), **common)
        else:
            ops.linear_scan(take(q), take(k), take(v), take(z), state, slots, cu, out, heads, kv_heads, dk, dv,
                            decay_kind=ops.DECAY_SIGMOID_POWER, power=1.0 / tau, q_scale=q_scale, **common)
        got[rows] = out.cpu()
        done = [done[i] + portions[i] for i in range(2)]
    _close(got, ref, torch.float32, kind, f32=2e-5)     # (32-bit whatever the operands' storage)
    assert float(state[1].abs().max()) == 0.0           # a slot no sequence holds stays untouched


@DTYPES
@pytest.mark.parametrize("rows, parts, d", [(5, 4, 16), (3, 1, 200), (9, 3, 40), (3, 2, 520), (2, 1, 2304)])
def test_gate_before_the_output_norm(dtype, rows, parts, d):
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(rows + d)
    x = torch.randn(rows, parts * d, generator=g) * torch.linspace(0.2, 9.0, parts * d)
    z = torch.randn(rows, parts * d + 8, generator=g).to(dtype)
    w = torch.randn(parts * d, generator=g)
    out = torch.empty((rows, parts * d), dtype=dtype, device="cuda")
    ops.gated_rmsnorm(x.cuda(), w.cuda(), z.cuda(), out, parts, d, 1e-5, "silu", gate_first=True)
    ref = P.grouped_rms_norm(x.to(F) * P.silu(z[:, :parts * d].to(F)), w.to(F), parts, 1e-5)
    _close(out, ref, dtype, "gated norm", f32=1e-5, bf16=1e-2)
    heads = torch.empty((rows, parts * d), dtype=dtype, device="cuda")
    ops.gate_rows(heads.copy_(x.to(dtype)), z.cuda(), "sigmoid")
    _close(heads, x.to(dtype).to(F) * torch.sigmoid(z[:, :parts * d].to(F)), dtype, "gate", f32=1e-6, bf16=1e-2)


@DTYPES
def test_rotation_by_position(dtype):
    """Rows that are a part of every head of a wider projection, turned by the token's position into a buffer of their
    own; stretched frequencies against the plain implementation's."""
    from gpullama3.java_b200.kernels import ops
    from gpullama3.java_b200.parts.position import YarnRotaryPositionEncoding

    rot = {"dims": 12, "base": 500.0, "scaling": {"factor": 6.0, "original": 40, "fast": 5.0, "slow": 1.5}}
    pos_enc = YarnRotaryPositionEncoding(12, 500.0, 6.0, 40, 5.0, 1.5)
    freqs, magnitude = P.yarn_frequencies(rot)
    assert torch.allclose(torch.tensor(pos_enc.frequencies(), dtype=F), freqs, rtol=1e-12) and abs(pos_enc.magnitude - magnitude) < 1e-12
    assert len({round(float(a / b), 6) for a, b in zip(freqs, P.yarn_frequencies({**rot, "scaling": {**rot["scaling"], "factor": 1.0}})[0])}) > 2
    g = torch.Generator().manual_seed(3)
    T, H, dk, dr = 7, 3, 10, 12
    src = torch.randn(T, H * (dk + dr) + 4, generator=g).to(dtype)
    positions = torch.tensor([0, 1, 2, 700, 64, 63, 5], dtype=torch.int32)
    dst = torch.zeros(T, H * (dk + dr), dtype=dtype, device="cuda")
    segs = ops.head_row_segments(
        ops.head_row_segment(0, H, dk, 0, dk, mul=1.5, src_stride=dk + dr, dst_stride=dk + dr),
        ops.head_row_segment(dk, H, dr, dk, dr, mul=1.5 * magnitude, rotate=True, src_stride=dk + dr, dst_stride=dk + dr))
    ops.head_rows(src.cuda(), dst, segs, 0.0, rotary=(positions.cuda(), pos_enc.inverse_frequencies("cuda")))
    x = src[:, :H * (dk + dr)].to(F).view(T, H, dk + dr)
    ref = torch.cat([x[..., :dk] * 1.5, P.rotate_interleaved(x[..., dk:], positions, freqs, magnitude) * 1.5], dim=-1)
    _close(dst.view(T, H, dk + dr), ref, dtype, "rotation", f32=3e-5, bf16=1e-2)


def test_routing_by_table():
    from gpullama3.java_b200.kernels import ops

    table = torch.tensor([[3, 1, 0], [2, 0, 4], [4, 3, 2]], dtype=torch.int32).cuda()
    tokens = torch.tensor([2, 0, 0, 1], dtype=torch.int32).cuda()
    chosen = torch.empty((4, 3), dtype=torch.int32, device="cuda")
    weights = torch.empty((4, 3), dtype=torch.float32, device="cuda")
    ops.moe_table_route(tokens, table, chosen, weights, 5)
    assert chosen.cpu().tolist() == [[4, 3, 2], [3, 1, 0], [3, 1, 0], [2, 0, 4]]
    assert torch.equal(weights.cpu(), torch.full((4, 3), 1.0 / 3.0))


def _single(mixer_type, mixer, mlp=None, **top):
    return {"architecture": "Gatuzen", "vocab": 64, "width": 32, "embedding": {"scale": 3.0},
            "norm": {"eps": 1e-5, "groups": top.get("groups", 1)}, "canon": {"taps": top.get("taps", 0)}, "logit_scale": 1.0,
            "residual_mult": 1.0, "initializer_range": 0.1, "layers": [{"type": mixer_type, "mixer": mixer, "mlp": mlp}]}


ALONE = {
    "gla": _single("gla", {"heads": 2, "dim": 16, "vdim": 24, "tau": 4.0, "decay_rank": 8}),
    "mamba2": _single("mamba2", {"heads": 4, "vdim": 8, "state": 12, "groups": 2, "conv": 3, "norm_groups": 2}),
    "latent": _single("latent_attention", {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 12, "kv_rank": 20, "scale": 0.4,
                                           "rot": {"base": 100.0, "dims": 4}}),
    "experts": _single("gla", {"heads": 1, "dim": 8, "vdim": 8, "tau": 2.0, "decay_rank": 2},
                       {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 3}}, taps=2, groups=4),
    "wide latent": _single("latent_attention", {"heads": 2, "dim": 24, "rot_dim": 32, "vdim": 8, "kv_rank": 200, "scale": 0.2,
                                                "rot": {"base": 9000.0, "dims": 32}}),
}


@DTYPES
@pytest.mark.parametrize("which", sorted(ALONE))
def test_one_mixer_alone(session_tmp, dtype, which):
    """A single layer of one kind, no input convolution unless the case is about it: a prompt, then decoding, then a
    second request in the slot the first gave back."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d = make_gatuzen_dir(session_tmp, ALONE[which], seed=11)
    cfg, weights = plain_inputs(d)
    model = load_model(d, dtype)
    cache = model.new_cache(64 * 4, max_slots=1)
    step = StepFunction(model, cache)
    for tokens in random_prompts(cfg["vocab"], [90, 70], seed=5):
        ref = P.forward(cfg, weights, tokens)
        slot = cache.acquire()
        got = [step([SequenceInput(slot, tokens[:66], list(range(66)))]).cpu()]
        got += [step([SequenceInput(slot, [t], [0])]).cpu().clone() for t in tokens[66:]]
        cache.release(slot)
        assert_logits(torch.cat(got), ref, dtype, which)


@DTYPES
def test_a_far_key_that_stands_out(session_tmp, dtype):
    """Among 400 positions one early token's latent is made to match every later query: the queries' and the latent's
    projections of that token are scaled up, so that the attention's result is that token's value wherever it is
    visible, and an engine that lost it (a page, a row of the latent, the rotated part) shows."""
    def peak(tensors):
        tensors["l0.mix.uk"] = tensors["l0.mix.uk"] * 3.0

    cfg_json = _single("latent_attention", {"heads": 2, "dim": 16, "rot_dim": 8, "vdim": 16, "kv_rank": 24, "scale": 2.0,
                                            "rot": {"base": 50.0, "dims": 8}})
    d = make_gatuzen_dir(session_tmp, cfg_json, seed=13, edit=peak)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [400], seed=9)[0]
    ref = P.forward(cfg, weights, tokens)
    hidden = P.forward(cfg, weights, tokens[70:])
    moved = (hidden[200:] - ref[270:]).abs().amax(dim=1) / (5e-5 * float(ref.abs().max()))
    assert float((moved > 20).float().mean()) > 0.9
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    model = load_model(d, dtype)
    cache = model.new_cache(64 * 8)
    step = StepFunction(model, cache)
    slot = cache.acquire()
    got = [step([SequenceInput(slot, tokens[:300], list(range(300)))]).cpu()]
    got += [step([SequenceInput(slot, [t], [0])]).cpu().clone() for t in tokens[300:]]
    assert_logits(torch.cat(got), ref, dtype, "a far key")
