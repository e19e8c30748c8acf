"""RMS norm: ``x * 1/sqrt(mean(x^2) + eps) * weight``, and layer norm:
``(x - mean) / sqrt(var + eps) * weight + bias``.

garuda/src/simd/mod.rs:166-173 (eps inside the root, added to the mean) and
garuda/src/llama/mod.rs:733-738 (scale, then a plain multiply by the weight).
The sum, the root and both multiplies are 32-bit in the kernel; only the result
is rounded to the compute dtype.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import Norm, TensorSpec, register_norm


@register_norm("rms")
class RMSNorm(Norm):
    """``weight_name``: the tensor's local name. ``unit_offset``: the stored weight lies about
    zero and the norm multiplies by ``1 + weight`` (the sum is taken once, in 32-bit, when the
    weights are loaded). A residual kept as several streams ``x [T, S, d]`` is normed as the
    weighted sum of its streams (``stream_weights [S]``; None: the plain sum)."""
    graph_safe = True

    def __init__(self, width: int, eps: float, weight_init=("ones",), weight_name: str = "weight",
                 unit_offset: bool = False):
        self.width = int(width)
        self.eps = float(eps)
        self.weight_name = weight_name
        self.unit_offset = bool(unit_offset)
        self.weight_init = ("normal", 0.1) if self.unit_offset and tuple(weight_init) == ("ones",) else tuple(weight_init)

    def tensors(self):
        return {self.weight_name: TensorSpec((self.width,), role="vector", init=self.weight_init)}

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.weight = tensors[self.weight_name]
        if self.unit_offset:
            self.weight = (1.0 + self.weight.float()).contiguous()
        self._weight32 = None
        self._ones = {}

    def fold(self):
        """(weight in 32-bit, eps) for a product that folds this norm in, see
        ``CudaOps.linear``'s ``emit_norm``."""
        if getattr(self, "_weight32", None) is None:
            self._weight32 = self.weight.float().contiguous()
        return self._weight32, self.eps

    def forward(self, ctx, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                out_name: str = "normed", stream_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.get(out_name, (n, self.width), self.dtype)
        if x.dim() == 3:
            if stream_weights is None:
                S = x.shape[1]
                if S not in self._ones:
                    self._ones[S] = torch.ones(S, dtype=torch.float32, device=x.device)
                stream_weights = self._ones[S]
            self.ops.streams_rmsnorm(x, stream_weights, self.weight, self.eps, out, rows)
        else:
            self.ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out


@register_norm("layer")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * weight + bias`` with ``var`` the mean of the squared
    deviations; 32-bit in the kernel, the result rounded to the compute dtype. ``weight_name``
    and ``bias_name`` are the tensors' local names (``bias_name`` None: no bias)."""
    graph_safe = True

    def __init__(self, width: int, eps: float, weight_name: str = "weight", bias_name: Optional[str] = "bias",
                 weight_init=("ones",)):
        self.width, self.eps = int(width), float(eps)
        self.weight_name, self.bias_name = weight_name, bias_name
        self.weight_init = tuple(weight_init)

    def tensors(self):
        t = {self.weight_name: TensorSpec((self.width,), role="vector", init=self.weight_init)}
        if self.bias_name is not None:
            t[self.bias_name] = TensorSpec((self.width,), role="vector", init=("normal", 0.02))
        return t

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.weight = tensors[self.weight_name]
        self.bias = tensors[self.bias_name] if self.bias_name is not None else None

    def forward(self, ctx, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                out_name: str = "normed") -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.get(out_name, (n, self.width), self.dtype)
        self.ops.layernorm(x, self.weight, self.bias, self.eps, out, rows)
        return out
