"""The dense gated feed-forward of the Llama 3 decoder (SwiGLU):
down( silu(gate(x)) * up(x) ), inference/InferenceCore.java:154-172 of the reference project.
Gate and up rows are interleaved into one weight at load so that one matrix product's epilogue
sees a gate value and its up value side by side (the reference fuses the same pair in one kernel,
tornadovm/TransformerComputeKernelsLayered.java:808-826)."""
from __future__ import annotations

import torch

from ..config.base import ConfigError
from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import FeedForward, StepContext, register_feed_forward
from .linear import Linear


class SwiGLUFeedForward(FeedForward):
    graph_safe = True
    pad_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", limit: float | None = None,
                 slope: float = 1.0):
        """``activation`` of the gate: ``silu`` (SwiGLU), ``gelu_tanh`` (GELU in its tanh form), or
        ``clamped_sigmoid``: with g = min(gate, limit) and u = clamp(up, -limit, limit) the unit's value is
        g sigmoid(slope g) (u + 1)."""
        if activation not in ops.ACTIVATION_CODES:
            raise ConfigError(f"feed-forward activation {activation!r}; known: {', '.join(sorted(ops.ACTIVATION_CODES))}")
        if activation == "clamped_sigmoid" and (limit is None or not limit > 0):
            raise ConfigError(f"the clamped feed-forward needs a positive limit, got {limit!r}")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.gate_args = (float(limit or 0.0), float(slope))
        self.gate_up: Linear | None = None
        self.down: Linear | None = None

    def parameters(self):
        return {"gate": ParamSpec((self.intermediate_size, self.hidden_size)),
                "up": ParamSpec((self.intermediate_size, self.hidden_size)),
                "down": ParamSpec((self.hidden_size, self.intermediate_size))}

    def load(self, tensors, dtype, device):
        gate, up, down = (tensors[n].to(device) for n in ("gate", "up", "down"))
        common = torch.float32 if (dtype == torch.float32 or torch.float32 in (gate.dtype, up.dtype)) else gate.dtype
        fused = torch.stack([gate.to(common), up.to(common)], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        self.gate_up = Linear(fused.contiguous())
        self.down = Linear(down.to(torch.float32 if dtype == torch.float32 else down.dtype).contiguous())

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        return ctx.all_decode and self.activation == "silu" and self.gate_up.links_with(ctx.n_tokens, ctx.dtype)

    def forward(self, x, ctx: StepContext, residual, then_norm=None):
        h = self.gate_up.gated(x, ctx.dtype, ctx.empty, self.activation, self.gate_args)  # [T, intermediate]
        return self.down.add_to(h, residual, then_norm)


class DenseFeedForward(FeedForward):
    """down( act(up(x) + b_up) ) + b_down without a gate; ``activation``: ``relu_squared``, max(., 0)^2.  The biases are
    kept and added in 32 bits: the first joins the product's result as the activation is applied, the second joins
    what the down product added into the caller's rows."""
    graph_safe = True
    pad_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu_squared", bias: bool = True):
        if activation not in ops.UNGATED_ACTIVATIONS:
            raise ConfigError(f"feed-forward activation {activation!r}; known: {', '.join(sorted(ops.UNGATED_ACTIVATIONS))}")
        self.hidden_size, self.intermediate_size, self.activation, self.bias = hidden_size, intermediate_size, activation, bool(bias)
        self.up: Linear | None = None
        self.down: Linear | None = None
        self.up_bias = self.down_bias = None

    def parameters(self):
        p = {"up": ParamSpec((self.intermediate_size, self.hidden_size)), "down": ParamSpec((self.hidden_size, self.intermediate_size))}
        if self.bias:
            p["up_bias"] = ParamSpec((self.intermediate_size,), "normal", 0.0, 0.02)
            p["down_bias"] = ParamSpec((self.hidden_size,), "normal", 0.0, 0.02)
        return p

    def load(self, tensors, dtype, device):
        keep = lambda w: w.to(device).to(torch.float32 if dtype == torch.float32 else w.dtype).contiguous()
        self.up, self.down = Linear(keep(tensors["up"])), Linear(keep(tensors["down"]))
        if self.bias:
            self.up_bias = tensors["up_bias"].to(device=device, dtype=torch.float32).contiguous()
            self.down_bias = tensors["down_bias"].to(device=device, dtype=torch.float32).contiguous()

    def result_bias(self):
        """The vector that still has to join the result when ``forward`` was told to leave it out (a caller whose next
        kernel reads the result anyway adds it there)."""
        return self.down_bias

    def forward(self, x, ctx: StepContext, residual, then_norm=None, add_result_bias: bool = True):
        u = self.up.store(x, ctx.dtype, ctx.empty)
        ops.bias_act_rows(u, self.up_bias, self.activation)
        self.down.add_to(u, residual)
        if add_result_bias and self.down_bias is not None:
            ops.add_row(residual, self.down_bias)
        return None


register_feed_forward("swiglu", SwiGLUFeedForward)
register_feed_forward("dense", DenseFeedForward)
register_feed_forward("gated", SwiGLUFeedForward)   # the same arrangement, the gate's activation named by the configuration
