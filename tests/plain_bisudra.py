"""A plain, slow implementation of the Bisudra decoder: one function per mechanism, whole sequences at once,
float64 on the CPU, no cache and no state carried between calls.  It shares no code with the package; the tests
compare the engine with it.

Notation: T tokens, x [T, width]; weights are a dict of float tensors by checkpoint name, a linear weight is
[out, in] and is applied as x @ W.T; ``p`` is a layer's name prefix (``l3.``), ``m`` a mixer's or feed-forward's record
of the configuration."""
from __future__ import annotations

import math

import torch

F = torch.float64


# ---------------------------------------------------------------- small functions
_ROUNDING = [None]   # a function applied to what every product reads and returns while ``forward(..., reads=f)`` runs
_MARGINS = [None]    # a list that receives, per routed layer, every token's routing margin while ``forward(..., margins=l)`` runs


def product(x, w):
    """x @ w.T; while a rounding is set, of the rounded x, and rounded itself."""
    f = _ROUNDING[0]
    return x @ w.T if f is None else f(f(x) @ w.T)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def squared_relu(z):
    return torch.clamp(z, min=0.0) ** 2


def over_root_mean_square(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    mean = x.mean(dim=-1, keepdim=True)
    dev = x - mean
    return dev / torch.sqrt((dev * dev).mean(dim=-1, keepdim=True) + eps) * w + b


def causal_conv(h, w):
    """y_t = sum_j w[:, j] h_(t - taps + 1 + j) per channel, zeros before the start; h [T, C], w [C, taps]."""
    T, C = h.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=h.dtype), h], dim=0)
    y = torch.zeros(T, C, dtype=h.dtype)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


def with_input_convolution(h, w):
    return h + causal_conv(h, w)


def residual_gate(h, w, b):
    """What a sublayer's result is multiplied with: a sigmoid per channel of the sublayer's own input."""
    return torch.sigmoid(product(h, w) + b)


# ---------------------------------------------------------------- attention
def rotate_interleaved(x, positions, base, dims):
    """x [T, n, d]: the pairs (2i, 2i + 1), i < dims / 2, turned by position * base^(-2i / dims); the rest as it is."""
    out = x.clone()
    for i in range(dims // 2):
        a = positions.to(F) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def windowed_softmax_attention(q, k, v, scale, window):
    """One head and one map: q, k [T, d], v [T, dv]; query i sees keys j with 0 <= i - j < window (window None: all
    j <= i).  Returns [T, dv]."""
    T = q.shape[0]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    s = (q @ k.T) * scale
    s = torch.where(seen, s, torch.full_like(s, -math.inf))
    return torch.softmax(s, dim=-1) @ v


def differential_weight(W, p, diff):
    return (math.exp(float((W[p + "mix.lq1"] * W[p + "mix.lk1"]).sum()))
            - math.exp(float((W[p + "mix.lq2"] * W[p + "mix.lk2"]).sum())) + diff)


def differential_attention(h, W, p, m, eps, positions=None):
    """Two softmax maps per head over the same values, the second taken off the first times one number of the layer."""
    T = h.shape[0]
    H, G, d, dv, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], float(m["diff"])
    positions = torch.arange(T) if positions is None else positions
    q = product(h, W[p + "mix.q"]).reshape(T, H, 2, d)
    k = product(h, W[p + "mix.k"]).reshape(T, G, 2, d)
    v = product(h, W[p + "mix.v"]).reshape(T, G, dv)
    q = over_root_mean_square(q, eps) * W[p + "mix.q.norm"]
    k = over_root_mean_square(k, eps) * W[p + "mix.k.norm"]
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = rotate_interleaved(q.reshape(T, 2 * H, d), positions, float(rot["base"]), rot["dims"]).reshape(T, H, 2, d)
        k = rotate_interleaved(k.reshape(T, 2 * G, d), positions, float(rot["base"]), rot["dims"]).reshape(T, G, 2, d)
    window = (m.get("mask") or {}).get("size")
    lam = differential_weight(W, p, diff)
    heads = []
    for a in range(H):
        g = a // (H // G)
        a1 = windowed_softmax_attention(q[:, a, 0], k[:, g, 0], v[:, g], float(m["scale"]), window)
        a2 = windowed_softmax_attention(q[:, a, 1], k[:, g, 1], v[:, g], float(m["scale"]), window)
        o = a1 - lam * a2
        heads.append(over_root_mean_square(o, eps) * (1.0 - diff))
    o = torch.cat(heads, dim=1) * torch.sigmoid(product(h, W[p + "mix.g"]))
    return product(o, W[p + "mix.o"])


# ---------------------------------------------------------------- feed-forwards
def dense_feed_forward(h, W, p):
    z = squared_relu(product(h, W[p + "mlp.up"]) + W[p + "mlp.up.b"])
    return product(z, W[p + "mlp.down"]) + W[p + "mlp.down.b"]


def router_choice(h, W, p, top):
    """Chosen experts [T, top] (largest logits first) and their weights: the softmax over the chosen logits alone."""
    w = W[p + "mlp.router"]
    z = h @ w.T + W[p + "mlp.router.b"]
    best, chosen = torch.topk(z, top, dim=-1)
    if _MARGINS[0] is not None:
        _MARGINS[0].append(routing_margin(h, w, z, top))
    return chosen, torch.softmax(best, dim=-1)


def routing_margin(h, w, z, top):
    """Per token: how far the last chosen logit lies above the best one left out, as a share of the length of the vector
    h_i (w_a,i - w_b,i) (independent relative errors of that share in every h_i move the difference of the two logits by
    about as much as it is).  Infinite when every expert is chosen."""
    if top >= z.shape[-1]:
        return torch.full((h.shape[0],), math.inf, dtype=F)
    order = torch.argsort(z, dim=-1, descending=True)
    a, b = order[:, top - 1], order[:, top]
    gap = z.gather(1, a[:, None])[:, 0] - z.gather(1, b[:, None])[:, 0]
    reach = torch.linalg.vector_norm(h * (w[a] - w[b]), dim=-1)
    return gap / (reach + 1e-300)


def mixture_of_experts(h, W, p, mlp, choice=None):
    chosen, weights = router_choice(h, W, p, mlp["router"]["top"]) if choice is None else choice
    out = torch.zeros(h.shape[0], W[p + "mlp.e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            q = f"{p}mlp.e{e}."
            out[t] += w * product(silu(product(h[t], W[q + "gate"])) * product(h[t], W[q + "up"]), W[q + "down"])
    return out


def feed_forward(h, W, p, mlp):
    return dense_feed_forward(h, W, p) if mlp["kind"] == "dense" else mixture_of_experts(h, W, p, mlp)


# ---------------------------------------------------------------- what joins the stream beside the sublayers
def token_side_input(x, tokens, W, p, layer, dim, eps):
    """A few numbers per (token id, layer), gated by the stream, projected to its width and normed."""
    e = W["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(product(x, W[p + "side.gate"])) * e
    y = product(g, W[p + "side.proj"])
    return over_root_mean_square(y, eps) * W[p + "side.norm"]


def depth_average(results, w):
    """sum_j w[j] X_j over the embedding output and every layer's result so far."""
    return sum(w[j] * X for j, X in enumerate(results))


# ---------------------------------------------------------------- the model
def layer(x, tokens, W, config, i):
    L = config["layers"][i]
    p, eps = f"l{i}.", float(config["norm"]["eps"])
    taps = (config.get("canon") or {}).get("taps")
    h = with_input_convolution(x, W[p + "canon1"]) if taps else x
    y = differential_attention(h, W, p, L["mixer"], eps) * residual_gate(x, W[p + "rg1"], W[p + "rg1.b"])
    x = x + layer_norm(y, W[p + "norm1"], W[p + "norm1.b"], eps)
    if L.get("mlp") is not None:
        y = feed_forward(x, W, p, L["mlp"]) * residual_gate(x, W[p + "rg2"], W[p + "rg2.b"])
        x = x + layer_norm(y, W[p + "norm2"], W[p + "norm2.b"], eps)
    side = config.get("token_side")
    if side and side.get("dim"):
        x = x + token_side_input(x, tokens, W, p, i, side["dim"], eps)
    return x


def forward(config, weights, tokens, return_layers=False, reads=None, margins=None):
    """Logits [T, vocab] of one sequence (float64); with ``return_layers`` also every layer's result, before the depth
    average that follows it.  ``reads``: a rounding applied to what every product reads and to what it returns (to see
    how far roundings alone move the result; the router's product is exempt, it is 32-bit in every run).  ``margins``: a
    list that receives one tensor [T] per routed layer, every token's ``routing_margin``."""
    W = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = W["embed"][tokens]
    _ROUNDING[0], _MARGINS[0] = reads, margins
    results, layers = [x], []
    for i in range(len(config["layers"])):
        X = layer(x, tokens, W, config, i)
        layers.append(X)
        results.append(X)
        x = depth_average(results, W[f"l{i}.dwa"])
    eps = float(config["norm"]["eps"])
    last = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    logits = (reads(last) if reads else last) @ W["embed"].T
    _ROUNDING[0] = _MARGINS[0] = None
    return (logits, layers) if return_layers else logits
