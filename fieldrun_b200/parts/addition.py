"""Additions: parts behind a layer's block that add to the stream once more.

``token_side_input``: a further input per layer and token.  A table holds, for every token id, ``dim`` entries for each
layer (layer i its columns [i * dim, (i + 1) * dim)); with e the token's entries,

    g = activation(W_gate x) * e,   y = W_proj g,   x <- x + y / sqrt(mean(y^2) + eps) * w

where x is the stream after the layer's feed-forward.  The table is one tensor that all layers read; it is fetched once.
The norm's statistic, the sum and the stream are float32; the two products take x and g in the model type."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorNeed, TensorSource
from .base import Addition, as_tensor, register_part, shared_fetch
from .linear import linear


class TokenSideInput(Addition):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.width = int(a["width"])
        self.dim = int(a["dim"])
        self.index = int(a["index"])
        self.shares = int(a["shares"])                 # how many layers have a share of the table's columns
        self.vocab_size = int(a["vocab_size"])
        self.eps = float(a["eps"])
        self.activation = a.get("activation", "gelu_tanh")
        if self.activation != "gelu_tanh":
            raise ValueError(f"a token side input with activation {self.activation!r}: the kernel has 'gelu_tanh'")
        if not 0 <= self.index < self.shares:
            raise ValueError(f"share {self.index} of {self.shares}")
        self.table: Optional[torch.Tensor] = None
        self.w_gate: Optional[torch.Tensor] = None
        self.w_proj: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None

    def _needs(self):
        return (TensorNeed(self.name_of("table"), (self.vocab_size, self.shares * self.dim), MATRIX, "normal"),
                TensorNeed(self.name_of("gate"), (self.dim, self.width), MATRIX, "normal"),
                TensorNeed(self.name_of("proj"), (self.width, self.dim), MATRIX, "normal"),
                TensorNeed(self.name_of("norm"), (self.width,), VECTOR, "around_one"))

    def tensor_needs(self):
        return list(self._needs())

    def load(self, source: TensorSource) -> None:
        table, gate, proj, norm = self._needs()
        self.table = shared_fetch(source, table)
        self.w_gate, self.w_proj, self.norm = source.fetch(gate), source.fetch(proj), source.fetch(norm)

    def forward(self, ctx, x, pending):
        rows = x.shape[0]
        delta = as_tensor(ctx, pending)
        if self.dtype == torch.float32:
            if delta is not None:
                ops.add_rows(x, delta)
            act = x
        else:
            act = ctx.buffer("side.act", (rows, self.width), self.dtype)
            ops.add_typed_copy(x, delta, act)                      # the block's update is added on the way
        gated = ctx.buffer("side.gated", (rows, self.dim), self.dtype)
        ops.token_side_gate(linear(act, self.w_gate), ctx.step_tokens, self.table, self.index * self.dim, gated)
        ops.add_rms_normed(x, linear(gated, self.w_proj), self.norm, self.eps)
        return x, None


register_part("addition", "token_side_input", TokenSideInput, replace=True)
