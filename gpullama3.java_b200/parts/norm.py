"""Norms over the rows of the residual stream.  RMSNorm, the only norm of the Llama 3 decoder (inference/InferenceCore.java:47-56 of the
reference project): used before the mixer, before the feed-forward and before the output head."""
from __future__ import annotations

import torch

from ..config.base import ConfigError
from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import Norm, register_norm


class RMSNorm(Norm):
    graph_safe = True
    pad_safe = True

    def __init__(self, dim: int, eps: float, offset: float = 0.0, groups: int = 1):
        """``offset``: what is added to the stored weight (1.0 for a weight that is stored around zero and applied
        as 1 + w); the sum is formed once at load, in 32 bits, and the weight is then kept in 32 bits.
        ``groups``: the row is cut into that many equal consecutive parts and each part is divided by its own root
        mean square (eps inside the root); the weight, one number per element, is kept in 32 bits."""
        self.dim, self.eps, self.offset, self.groups = int(dim), float(eps), float(offset), int(groups)
        if self.groups < 1 or self.dim % self.groups:
            raise ConfigError(f"a norm over {self.dim} numbers cannot be cut into {groups} equal parts")
        self.weight: torch.Tensor | None = None

    def parameters(self):
        return {"weight": ParamSpec((self.dim,), "norm" if self.offset == 0.0 else "matrix")}

    def load(self, tensors, dtype, device):
        w = tensors["weight"]
        # a weight stored in 32 bits stays so; the float32 run takes everything in 32 bits
        keep = torch.float32 if (dtype == torch.float32 or w.dtype == torch.float32 or self.offset != 0.0
                                 or self.groups > 1) else torch.bfloat16
        self.weight = w.to(device=device, dtype=keep).contiguous()
        if self.offset != 0.0:
            self.weight += self.offset

    def row_factor_form(self):
        return (self.weight, self.eps, self.dim) if self.groups == 1 else None   # (in groups a row has several factors)

    def group_form(self):
        """(float32 weight [dim], eps, groups): the norm as the kernels that norm in groups take it."""
        w = self.weight
        if w.dtype != torch.float32:
            w = getattr(self, "_weight_f32", None)
            if w is None:
                w = self._weight_f32 = self.weight.to(torch.float32)
        return w, self.eps, self.groups

    def forward(self, x, out_dtype, rows=None, alloc=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = alloc((n, self.dim), out_dtype) if alloc is not None else torch.empty((n, self.dim), dtype=out_dtype, device=x.device)
        if self.groups > 1:
            ops.group_rmsnorm(x, self.weight, out, self.eps, self.groups, rows)
        else:
            ops.rmsnorm(x, self.weight, out, self.eps, rows)
        return out


class LayerNorm(Norm):
    """(x - mean) / sqrt(variance + eps) * weight + bias over the residual stream's rows, the variance being the mean of
    the squared deviations.  Weight and bias are kept, and applied, in 32 bits."""
    graph_safe = True
    pad_safe = True

    def __init__(self, dim: int, eps: float):
        self.dim, self.eps = int(dim), float(eps)
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def parameters(self):
        return {"weight": ParamSpec((self.dim,), "norm"), "bias": ParamSpec((self.dim,), "normal", 0.0, 0.02)}

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"].to(device=device, dtype=torch.float32).contiguous()
        self.bias = tensors["bias"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, out_dtype, rows=None, alloc=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = alloc((n, self.dim), out_dtype) if alloc is not None else torch.empty((n, self.dim), dtype=out_dtype, device=x.device)
        ops.layernorm(x, self.weight, self.bias, out, self.eps, rows)
        return out


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
