"""A routed feed-forward (mixture of experts): every token runs through a few of many small gated feed-forwards.

    z = W_r h (32-bit) ;  s = softmax(z) over all experts
    the experts form ``groups`` equal groups of neighbours; a group's score is its best expert's; only experts of the
    ``keep_groups`` best groups can be chosen; the ``top`` best of those are
    y = sum over the chosen e of  s_e / (sum of the chosen s + 1e-20) * down_e( act(gate_e h, up_e h) )

With ``router_bias`` a learned vector joins the logits z.  With one group and ``weight_eps`` 0 the weights are the softmax
over the chosen logits alone (s_e over the chosen s is exp(z_e) over the chosen exp(z)).

With ``router="table"`` there is no router product: row ``token id`` of an integer table [vocabulary, top] names the token's
experts, and every one of them weighs 1 / top.

The router and the weights are 32-bit in both precisions.  The (token, choice) pairs are ordered by expert.  A step of
few tokens then runs every expert's rows as a weight-streaming product whose row counts are read on the device, so a
decode step's launches do not depend on the routing and can be recorded; an expert's weights are read once for all the
tokens that chose it, and not at all when none did.  A prompt's rows are gathered into the order of their experts and
multiplied by one launch of the tcgen05 product over all experts' tiles (gated epilogue included), which reads the runs
on the device as well.  Only where that kernel does not take the operands (the float32 run, sizes off its grid) do
the per-expert row counts come back to the host, for one product per expert through the kernels the dense feed-forward
uses; that wait is why a prompt pass of this part is not replayed from a recording."""
from __future__ import annotations

import torch

from ..config.base import ConfigError
from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import FeedForward, StepContext, register_feed_forward
from .linear import Linear


class RoutedFeedForward(FeedForward):
    graph_safe = True    # (decode steps: the pair kernels read the routing from device memory)
    pad_safe = False     # a prompt pass may read the experts' row counts on the host

    def __init__(self, hidden_size: int, intermediate_size: int, n_experts: int, top: int, groups: int = 1,
                 keep_groups: int | None = None, activation: str = "silu", limit: float | None = None, slope: float = 1.0,
                 weight_eps: float = 1e-20, router: str = "learned", vocab_size: int | None = None,
                 router_bias: bool = False):
        keep_groups = groups if keep_groups is None else keep_groups
        if router not in ("learned", "table"):
            raise ConfigError(f"routed feed-forward: router {router!r}; known: learned, table")
        if router == "table" and not vocab_size:
            raise ConfigError("routed feed-forward: a routing table needs the vocabulary's size")
        if router_bias and router != "learned":
            raise ConfigError("routed feed-forward: only a learned router has logits a bias can join")
        self.routing, self.vocab_size, self.router_bias = router, int(vocab_size or 0), bool(router_bias)
        if activation not in ops.ACTIVATION_CODES:
            raise ConfigError(f"feed-forward activation {activation!r}; known: {', '.join(sorted(ops.ACTIVATION_CODES))}")
        if activation == "clamped_sigmoid" and (limit is None or not limit > 0):
            raise ConfigError(f"the clamped feed-forward needs a positive limit, got {limit!r}")
        if not (1 <= n_experts <= ops.MAX_EXPERTS) or not (1 <= top <= min(n_experts, ops.MAX_EXPERTS_PER_TOKEN)):
            raise ConfigError(f"routed feed-forward: {top} of {n_experts} experts (at most {ops.MAX_EXPERTS_PER_TOKEN} of "
                              f"{ops.MAX_EXPERTS})")
        if groups < 1 or n_experts % groups or not (1 <= keep_groups <= groups):
            raise ConfigError(f"routed feed-forward: {n_experts} experts do not form {groups} equal groups of which "
                              f"{keep_groups} are kept")
        if top > keep_groups * (n_experts // groups):
            raise ConfigError(f"routed feed-forward: {top} experts cannot come from {keep_groups} groups of {n_experts // groups}")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.n_experts, self.top, self.groups, self.keep_groups = int(n_experts), int(top), int(groups), int(keep_groups)
        self.activation, self.gate_args, self.weight_eps = activation, (float(limit or 0.0), float(slope)), float(weight_eps)

    def parameters(self):
        p = ({"router": ParamSpec((self.n_experts, self.hidden_size))} if self.routing == "learned" else
             {"table": ParamSpec((self.vocab_size, self.top), "int_table", float(self.n_experts))})
        if self.router_bias:
            p["router_bias"] = ParamSpec((self.n_experts,), "normal", 0.0, 0.02)
        for e in range(self.n_experts):
            p[f"e{e}.gate"] = ParamSpec((self.intermediate_size, self.hidden_size))
            p[f"e{e}.up"] = ParamSpec((self.intermediate_size, self.hidden_size))
            p[f"e{e}.down"] = ParamSpec((self.hidden_size, self.intermediate_size))
        return p

    def load(self, tensors, dtype, device):
        run = torch.float32 if dtype == torch.float32 else torch.bfloat16
        E, ff, h = self.n_experts, self.intermediate_size, self.hidden_size
        if self.routing == "learned":
            self.router = tensors["router"].to(device=device, dtype=torch.float32).contiguous()
            self.bias = tensors["router_bias"].to(device=device, dtype=torch.float32).contiguous() if self.router_bias else None
        else:
            self.table = tensors["table"].to(device=device, dtype=torch.int32).contiguous()
        self.w_gate_up = torch.empty((E, 2 * ff, h), dtype=run, device=device)   # gate and up rows interleaved
        self.w_down = torch.empty((E, h, ff), dtype=run, device=device)
        for e in range(E):
            self.w_gate_up[e, 0::2] = tensors[f"e{e}.gate"].to(device=device, dtype=run)
            self.w_gate_up[e, 1::2] = tensors[f"e{e}.up"].to(device=device, dtype=run)
            self.w_down[e] = tensors[f"e{e}.down"].to(device=device, dtype=run)
        self.gate_up = [Linear(self.w_gate_up[e]) for e in range(E)]
        self.down = [Linear(self.w_down[e]) for e in range(E)]
        # a decode step's launches depend on device memory alone when the streaming kernel takes the rows, or else when
        # the grouped product does (the per-expert products need the runs' lengths on the host)
        grouped = run == torch.bfloat16 and E <= ops.MAX_GEMM_GROUPS and h % 8 == 0 and ff % 8 == 0
        self.graph_safe = ops.moe_rows_takes(max(h, ff), run) or grouped

    def route(self, x: torch.Tensor, ctx: StepContext, scores: torch.Tensor | None = None):
        T = x.shape[0]
        chosen = ctx.empty((T, self.top), torch.int32)
        weights = ctx.empty((T, self.top), torch.float32)
        if self.routing == "table":
            ops.moe_table_route(ctx.tokens, self.table, chosen, weights, self.n_experts)
            return chosen, weights
        ops.moe_route(x, self.router, chosen, weights, self.groups, self.keep_groups, self.weight_eps, scores, self.bias)
        return chosen, weights

    def as_prompt(self, ctx: StepContext, n_tokens: int) -> bool:
        """Whether the experts' rows are gathered and multiplied as dense products (prompts), or streamed past the
        experts' weights a few rows at a time (steps of few tokens)."""
        if not ops.moe_rows_takes(max(self.hidden_size, self.intermediate_size), ctx.dtype):
            return True     # (rows too long to stage for the streaming kernel)
        return (not ctx.all_decode) and n_tokens > 64 and n_tokens * self.top >= 16 * self.n_experts

    def forward(self, x, ctx: StepContext, residual, then_norm=None):
        T = x.shape[0]
        chosen, weights = self.route(x, ctx)
        pairs = T * self.top
        offsets = ctx.empty((self.n_experts + 1,), torch.int32)
        order, place = ctx.empty((pairs,), torch.int32), ctx.empty((pairs,), torch.int32)
        ops.moe_group(chosen, self.n_experts, offsets, order, place)
        y = ctx.empty((pairs, self.intermediate_size), ctx.dtype)
        o = ctx.empty((pairs, self.hidden_size), torch.float32)
        if not self.as_prompt(ctx, T):
            ops.moe_rows(x, self.w_gate_up, offsets, y, order=order, top=self.top, activation=self.activation,
                         gate_args=self.gate_args)
            ops.moe_rows(y, self.w_down, offsets, o)
        else:
            xs = ctx.empty((pairs, self.hidden_size), ctx.dtype)
            ops.moe_gather(x, order, xs, self.top)
            # one launch over all experts' tiles, the runs read on the device; where that kernel does not take the operands
            # (the float32 run, odd sizes) one product per expert, for which the runs' lengths come back to the host
            if not (ops.gemm_tcgen05_grouped(xs, self.w_gate_up, offsets, y, ops.GATED_EPILOGUE_OF[self.activation], self.gate_args)
                    and ops.gemm_tcgen05_grouped(y, self.w_down, offsets, o)):
                bounds = offsets.tolist()
                for e in range(self.n_experts):
                    lo, hi = bounds[e], bounds[e + 1]
                    if hi > lo:
                        self.gate_up[e].gated_into(xs[lo:hi], y[lo:hi], self.activation, self.gate_args)
                        self.down[e].into(y[lo:hi], o[lo:hi])
        ops.moe_combine(o, place, weights, residual)
        return None


register_feed_forward("routed", RoutedFeedForward)
