"""Recurrent mixers whose memory is one matrix per head that decays and gains an outer product per token, without the
delta rule's correction:  S_t = diag(g_t) S_(t-1) + k_t (b_t v_t)^T,  o_t = S_t^T q_t.  Two of them:

``GatedLinearAttention`` (``gla``): a decay per key channel from a low-rank projection,

    q = W_q x * d_k^(-1/2) ;  k = W_k x  [heads, d_k] ;  v = W_v x  [heads, d_v]
    g = sigmoid(W_a2 (W_a1 x) + bias)^(1 / tau)  [heads, d_k] ;  b = 1
    y = W_o ( o / rms(o) * norm_weight * silu(W_g x) )                          rms over d_v, per head

``StateSpaceDuality`` (``ssd``, the Mamba-2 layer): one scalar decay per head and a step size on the value,

    [z | x | B | C | dt] = W_in u ;  x, B, C pass a short causal convolution with bias, then SiLU
    dt = softplus(dt + dt_bias)  [heads] ;  g = exp(-exp(A_log[h]) dt) ;  b = dt
    k = B, q = C  [groups, state] (head h reads group h / (heads / groups)) ;  v = x  [heads, d_v]
    o_t += D_h x_t ;  y = W_o ( norm( o * silu(z) ) )       the gate first, then an RMS norm in ``norm_groups`` equal parts

Both keep, per sequence, S of every head in 32 bits (and the convolution's last inputs) in one row of their cache slot,
starting from zero.  Decays, step sizes, the recurrence and the output norms are 32-bit in both precisions; projections
and the convolution are computed in the run's precision.  The scan is the kernel of the delta rule, told to leave out
the correction."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import StateNeed, StateView
from ..config.base import ConfigError
from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import Mixer, StepContext, register_mixer
from .linear import Linear


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


def _stacked(groups: list[torch.Tensor], device) -> tuple[Linear, list[int]]:
    """One product for several weights: their rows one after the other, each group padded to a multiple of 8 rows."""
    common = torch.float32 if any(g.dtype == torch.float32 for g in groups) else groups[0].dtype
    rows, offsets, at = [], [], 0
    for g in groups:
        offsets.append(at)
        rows.append(g.to(common))
        pad = _pad8(g.shape[0]) - g.shape[0]
        if pad:
            rows.append(torch.zeros((pad, g.shape[1]), dtype=common, device=device))
        at += _pad8(g.shape[0])
    return Linear(torch.cat(rows, dim=0).contiguous()), offsets


class GatedLinearAttention(Mixer):
    graph_safe = True   # slots and lengths reach the kernels through the step's device tensors
    pad_safe = False    # every token it sees enters the state

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, value_dim: int, decay_temperature: float,
                 norm_eps: float, decay_rank: int | None = None):
        """``decay_temperature`` tau: the decay is sigmoid(.)^(1 / tau).  ``decay_rank``: inner size of the decay's two
        products; None reads it from the checkpoint's shapes (it is needed to make random weights)."""
        if min(n_heads, head_dim, value_dim) < 1 or head_dim > 512:
            raise ConfigError(f"gated linear attention: key size {head_dim} must be between 1 and 512, heads and value size positive")
        if not decay_temperature > 0:
            raise ConfigError(f"gated linear attention: the decay's temperature must be positive, got {decay_temperature}")
        self.hidden_size, self.n_heads, self.key_dim, self.value_dim = int(hidden_size), int(n_heads), int(head_dim), int(value_dim)
        self.tau, self.norm_eps, self.decay_rank = float(decay_temperature), float(norm_eps), decay_rank
        self.state_floats = self.n_heads * self.key_dim * self.value_dim

    def parameters(self):
        H, dk, dv, h = self.n_heads, self.key_dim, self.value_dim, self.hidden_size
        r = self.decay_rank if self.decay_rank is not None else -1
        return {"q": ParamSpec((H * dk, h)), "k": ParamSpec((H * dk, h)), "v": ParamSpec((H * dv, h)),
                "g": ParamSpec((H * dv, h)), "o": ParamSpec((h, H * dv)), "norm": ParamSpec((dv,), "norm"),
                "a1": ParamSpec((r, h)), "a2": ParamSpec((H * dk, r)), "a2_bias": ParamSpec((H * dk,), "normal", 2.0, 1.0)}

    def cache_need(self):
        return StateNeed((self.state_floats,), torch.float32)

    def load(self, tensors, dtype, device):
        run = lambda t: t.to(device).to(torch.float32 if dtype == torch.float32 else t.dtype)
        f32 = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        self.inputs, (self.q_off, self.k_off, self.v_off, self.g_off, self.a1_off) = _stacked(
            [run(tensors[n]) for n in ("q", "k", "v", "g", "a1")], device)
        self.decay_rank = tensors["a1"].shape[0]
        self.a2 = Linear(run(tensors["a2"]).contiguous())
        self.o = Linear(run(tensors["o"]).contiguous())
        self.decay_bias, self.norm_weight = f32("a2_bias"), f32("norm")
        if device.type == "cuda" and not ops.delta_rule_supported(self.key_dim):
            raise ConfigError(f"gated linear attention: no kernel holds a state column of {self.key_dim} rows")

    def forward(self, x, ctx: StepContext, cache: StateView, residual, writes_cache=True, then_norm=None):
        H, dk, dv, T = self.n_heads, self.key_dim, self.value_dim, x.shape[0]
        proj = self.inputs.store(x, ctx.dtype, ctx.empty)
        decay = self.a2.store(proj[:, self.a1_off:self.a1_off + self.decay_rank], ctx.dtype, ctx.empty)    # [T, H dk]
        o = ctx.empty((T, H * dv), torch.float32)
        ops.linear_scan(proj[:, self.q_off:], proj[:, self.k_off:], proj[:, self.v_off:], decay, cache.data, ctx.slots_dev,
                        ctx.cu_seqlens, o, H, H, dk, dv, decay_kind=ops.DECAY_SIGMOID_POWER, decay_bias=self.decay_bias,
                        power=1.0 / self.tau, q_scale=dk ** -0.5, alloc=ctx.empty)
        gated = ctx.empty((T, H * dv), ctx.dtype)
        ops.gated_rmsnorm(o, self.norm_weight, proj[:, self.g_off:], gated, H, dv, self.norm_eps, "silu")
        return self.o.add_to(gated, residual, then_norm)


class StateSpaceDuality(Mixer):
    graph_safe = True
    pad_safe = False

    def __init__(self, hidden_size: int, n_heads: int, value_dim: int, state_dim: int, n_groups: int, conv_taps: int,
                 norm_eps: float, norm_groups: int = 1):
        if min(n_heads, value_dim, state_dim, n_groups, norm_groups) < 1 or state_dim > 512:
            raise ConfigError(f"state-space mixer: state size {state_dim} must be between 1 and 512, the other sizes positive")
        if n_heads % n_groups:
            raise ConfigError(f"state-space mixer: {n_heads} heads do not share {n_groups} groups equally")
        if (n_heads * value_dim) % norm_groups:
            raise ConfigError(f"state-space mixer: {n_heads * value_dim} numbers cannot be normed in {norm_groups} equal parts")
        if not (1 <= conv_taps <= ops.MAX_CONV_TAPS):
            raise ConfigError(f"conv taps {conv_taps}: the convolution kernel takes 1 to {ops.MAX_CONV_TAPS}")
        self.hidden_size, self.n_heads, self.value_dim, self.state_dim = int(hidden_size), int(n_heads), int(value_dim), int(state_dim)
        self.n_groups, self.taps, self.norm_eps, self.norm_groups = int(n_groups), int(conv_taps), float(norm_eps), int(norm_groups)
        self.inner = self.n_heads * self.value_dim
        self.channels = self.inner + 2 * self.n_groups * self.state_dim      # what the convolution runs over: x, B, C
        self.state_floats = self.n_heads * self.state_dim * self.value_dim
        self.conv_floats = (self.taps - 1) * self.channels

    def parameters(self):
        H, h = self.n_heads, self.hidden_size
        return {"in": ParamSpec((2 * self.inner + 2 * self.n_groups * self.state_dim + H, h)),
                "conv": ParamSpec((self.channels, self.taps), "normal", 0.0, 1.0 / self.taps ** 0.5),
                "conv_bias": ParamSpec((self.channels,), "normal", 0.0, 0.1),
                "dt_bias": ParamSpec((H,), "normal", 0.0, 1.0), "A_log": ParamSpec((H,), "normal", -1.0, 0.5),
                "D": ParamSpec((H,), "normal", 1.0, 0.2), "norm": ParamSpec((self.inner,), "norm"),
                "o": ParamSpec((h, self.inner))}

    def cache_need(self):
        return StateNeed((self.state_floats + self.conv_floats,), torch.float32)

    def load(self, tensors, dtype, device):
        run = lambda t: t.to(device).to(torch.float32 if dtype == torch.float32 else t.dtype)
        f32 = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        w = run(tensors["in"])
        i, gn = self.inner, self.n_groups * self.state_dim
        # rows as stored: z, then x | B | C (one run of columns for the convolution), then dt; dt's group starts on a multiple of 8
        self.inputs, (self.z_off, self.conv_off, self.dt_off) = _stacked([w[:i], w[i:2 * i + 2 * gn], w[2 * i + 2 * gn:]], device)
        self.o = Linear(run(tensors["o"]).contiguous())
        self.conv_weight, self.conv_bias = f32("conv"), f32("conv_bias")
        self.dt_bias, self.a_log, self.skip, self.norm_weight = f32("dt_bias"), f32("A_log"), f32("D"), f32("norm")
        if device.type == "cuda" and not ops.delta_rule_supported(self.state_dim):
            raise ConfigError(f"state-space mixer: no kernel holds a state column of {self.state_dim} rows")

    def forward(self, x, ctx: StepContext, cache: StateView, residual, writes_cache=True, then_norm=None):
        H, G, N, dv, T, gn = self.n_heads, self.n_groups, self.state_dim, self.value_dim, x.shape[0], self.n_groups * self.state_dim
        state = cache.data                                                    # [slots, S of every head | convolution inputs]
        proj = self.inputs.store(x, ctx.dtype, ctx.empty)
        xbc = ctx.empty((T, self.channels), ctx.dtype)
        ops.causal_conv(proj[:, self.conv_off:], self.conv_weight, state[:, self.state_floats:], ctx.slots_dev, ctx.seq_ids,
                        ctx.cu_seqlens, xbc, self.channels, bias=self.conv_bias, activation="silu", update_state=writes_cache)
        o = ctx.empty((T, self.inner), torch.float32)
        ops.linear_scan(xbc[:, self.inner + gn:], xbc[:, self.inner:], xbc, proj[:, self.dt_off:], state, ctx.slots_dev,
                        ctx.cu_seqlens, o, H, G, N, dv, decay_kind=ops.DECAY_SOFTPLUS_RATE, decay_per_head=True,
                        decay_bias=self.dt_bias, a_log=self.a_log, step_scales_value=True, skip=self.skip, alloc=ctx.empty)
        gated = ctx.empty((T, self.inner), ctx.dtype)
        ops.gated_rmsnorm(o, self.norm_weight, proj[:, self.z_off:], gated, self.norm_groups, self.inner // self.norm_groups,
                          self.norm_eps, "silu", gate_first=True)
        return self.o.add_to(gated, residual, then_norm)


register_mixer("gla", GatedLinearAttention)
register_mixer("ssd", StateSpaceDuality)
