"""A plain, slow implementation of the Gatuzen decoder: one function per mechanism, whole sequences at once,
float64 on the CPU, no cache and no state carried between calls.  It shares no code with the package; the tests
compare the engine with it.

Notation: T tokens, x [T, width]; weights are a dict of float tensors by checkpoint name, a linear weight is
[out, in] and is applied as x @ W.T."""
from __future__ import annotations

import math

import torch

F = torch.float64


# ---------------------------------------------------------------- small functions
def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def grouped_rms_norm(x, w, groups, eps):
    """The last axis in ``groups`` equal consecutive parts, each over its own root mean square; then times w."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(shape) * w


def causal_conv(h, w, bias=None):
    """y_t = sum_j w[:, j] h_(t - taps + 1 + j) per channel, zeros before the start; h [T, C], w [C, taps]."""
    T, C = h.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=h.dtype), h], dim=0)
    y = torch.zeros(T, C, dtype=h.dtype)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y if bias is None else y + bias


def with_input_convolution(h, w):
    return h + causal_conv(h, w)


# ---------------------------------------------------------------- linear recurrences
def decayed_outer_product_scan(q, k, v, decay):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t for one head: q, k, decay [T, dk], v [T, dv]."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=F)
    out = []
    for t in range(T):
        S = decay[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out.append(S.T @ q[t])
    return torch.stack(out)


def gated_linear_attention(h, W, p, m, norm_eps):
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = h.shape[0]
    q = (h @ W[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, dk)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).view(T, H, dk)
    heads = []
    for i in range(H):
        o = decayed_outer_product_scan(q[:, i], k[:, i], v[:, i], alpha[:, i])
        heads.append(o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + norm_eps) * W[p + "norm"])
    o = torch.cat(heads, dim=-1) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def mamba2(h, W, p, m, norm_eps):
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, T = H * dv, h.shape[0]
    proj = h @ W[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])                                   # [T, H]
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * dt)                     # [T, H]
    heads = []
    for i in range(H):
        g = i // (H // G)
        y = decayed_outer_product_scan(C[:, g], B[:, g], dt[:, i:i + 1] * x[:, i], decay[:, i:i + 1].expand(T, N))
        heads.append(y + W[p + "D"][i] * x[:, i])
    y = torch.cat(heads, dim=-1) * silu(z)
    y = grouped_rms_norm(y, W[p + "norm"], m["norm_groups"], norm_eps)
    return y @ W[p + "o"].T


# ---------------------------------------------------------------- latent attention
def yarn_frequencies(rot):
    """Per pair i: the rotation frequency, and the factor on cosine and sine."""
    dims, base, s = rot["dims"], float(rot["base"]), rot.get("scaling")
    if not s:       # no stretching: the plain frequencies, and nothing on cosine and sine
        return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F), 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def dim_of(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(dim_of(float(s["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(s["slow"]))), dims - 1)
    freqs = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        freqs.append(f / factor * ramp + f * (1.0 - ramp))
    return torch.tensor(freqs, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, freqs, magnitude):
    """x [T, ..., dims]: pairs (2i, 2i + 1) turned by position * freqs[i]; cosine and sine times ``magnitude``."""
    a = positions.to(F)[:, None] * freqs[None, :]
    cos, sin = torch.cos(a) * magnitude, torch.sin(a) * magnitude
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * cos - v * sin
    out[..., 1::2] = v * cos + u * sin
    return out


def latent_attention(h, W, p, m, norm_eps, start=0):
    H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(start, start + T)
    freqs, magnitude = yarn_frequencies(m["rot"])
    q = (h @ W[p + "q"].T).view(T, H, dk + dr)
    q_plain, q_rot = q[..., :dk], rotate_interleaved(q[..., dk:], pos, freqs, magnitude)
    down = h @ W[p + "dkv"].T
    c = down[:, :R]
    c = c / torch.sqrt((c * c).mean(dim=-1, keepdim=True) + norm_eps) * W[p + "dkv.norm"]
    k_rot = rotate_interleaved(down[:, R:], pos, freqs, magnitude)          # [T, dr], shared by the heads
    k_plain = (c @ W[p + "uk"].T).view(T, H, dk)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    o = torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# ---------------------------------------------------------------- feed-forward
def table_mixture_of_experts(h, tokens, W, p, top):
    """Every token runs through the experts its id names in the table, each weighted 1 / top."""
    table = W[p + "table"].to(torch.int64)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[tokens[t]].tolist():
            g, u = h[t] @ W[p + f"e{e}.gate"].T, h[t] @ W[p + f"e{e}.up"].T
            out[t] += ((silu(g) * u) @ W[p + f"e{e}.down"].T) / top
    return out


# ---------------------------------------------------------------- the model
MIXERS = {"gla": gated_linear_attention, "mamba2": mamba2, "latent_attention": latent_attention}


def layer_runs(config):
    """[(layer, pass number or None)]: the order in which layers run; the pass number stands at a pass's first layer."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(config, weights, tokens, return_layers=False, reads=None):
    """Logits [T, vocab] of one whole sequence (and, asked for, the residual stream after every layer run).
    ``reads``, if given, is applied to what every sublayer reads (to see how far a small change there moves the logits)."""
    W = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, groups, mult = float(config["norm"]["eps"]), config["norm"]["groups"], float(config["residual_mult"])
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    taps = (config.get("canon") or {}).get("taps", 0)
    convolved = (lambda h, w: with_input_convolution(h, W[w])) if taps else (lambda h, w: h)
    read = convolved if reads is None else (lambda h, w: reads(convolved(h, w)))
    x = W["embed"][tokens] * float(config["embedding"]["scale"])
    after = []
    for i, enters in layer_runs(config):
        L, p = config["layers"][i], f"l{i}."
        if enters is not None:
            x = x + W["loop.step"][enters]
        h = read(grouped_rms_norm(x, W[p + "norm1"], groups, eps), p + "canon1")
        y = MIXERS[L["type"]](h, W, p + "mix.", L["mixer"], eps)
        x = x + mult * grouped_rms_norm(y, W[p + "norm1b"], groups, eps)
        if L.get("mlp") is not None:
            h = read(grouped_rms_norm(x, W[p + "norm2"], groups, eps), p + "canon2")
            y = table_mixture_of_experts(h, tokens, W, p + "mlp.", L["mlp"]["router"]["top"])
            x = x + mult * grouped_rms_norm(y, W[p + "norm2b"], groups, eps)
        after.append(x)
    logits = grouped_rms_norm(x, W["final.norm"], groups, eps) @ W["head"].T * float(config["logit_scale"])
    return (logits, torch.stack(after)) if return_layers else logits
