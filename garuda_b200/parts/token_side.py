"""A per-layer token input added to the residual stream.

Every layer owns ``dim`` columns of one table ``[vocab, layers * dim]``; with
``e`` the token's row of those columns,

    g = gelu_tanh(W_gate x) * e,   y = W_proj g,   x += alpha * y / sqrt(mean(y^2) + eps) * w

(an RMS norm with a plain weight). ``x`` is the stream after the layer's
feed-forward. The table is a tensor of the model, shared by the layers' parts.
"""
from __future__ import annotations

import torch

from .base import ResidualBranch, TensorSpec, register_branch


@register_branch("token_side")
class TokenSide(ResidualBranch):
    graph_safe = True

    def __init__(self, width: int, dim: int, vocab: int, table: str, table_width: int, column: int, eps: float,
                 names=("gate", "proj", "norm"), init_std: float = 0.02):
        """``table``: the model-level name of the shared table, ``table_width`` its columns, of
        which this part reads ``[column, column + dim)``."""
        self.width, self.dim, self.vocab = int(width), int(dim), int(vocab)
        self.table, self.table_width, self.column = table, int(table_width), int(column)
        if not 0 <= self.column <= self.table_width - self.dim:
            raise ValueError(f"columns {column}..{column + dim} are outside a table {table_width} wide")
        self.eps = float(eps)
        self.names = tuple(names)
        self.init_std = float(init_std)

    def tensors(self):
        gate, proj, norm = self.names
        return {"@" + self.table: TensorSpec((self.vocab, self.table_width), init=("normal", 1.0)),
                gate: TensorSpec((self.dim, self.width), init=("normal", self.init_std)),
                proj: TensorSpec((self.width, self.dim), init=("normal", self.init_std)),
                norm: TensorSpec((self.width,), role="vector", init=("ones",))}

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        gate, proj, norm = self.names
        self.table_t = tensors["@" + self.table]
        self.w_gate, self.w_proj, self.norm_w = tensors[gate].contiguous(), tensors[proj].contiguous(), tensors[norm]

    def forward(self, ctx, x, alpha: float = 1.0):
        ops, ws, b = self.ops, ctx.ws, ctx.batch
        T = x.shape[0]
        xin = x
        if self.dtype != torch.float32:
            xin = ws.get("side_in", (T, self.width), self.dtype)
            ops.cast(x, xin)
        z = ws.get("side_z", (T, self.dim), torch.float32)
        ops.linear(xin, self.w_gate, z)
        g = ws.get("side_g", (T, self.dim), self.dtype)
        ops.gelu_gather_mul(z, self.table_t, b.token_ids, self.column, g)
        y = ws.get("side_y", (T, self.width), torch.float32)
        ops.linear(g, self.w_proj, y)
        ops.rms_add(x, y, self.norm_w, self.eps, alpha)
