"""RMSNorm: x * (1 / sqrt(mean(x^2) + eps)) * w per row, the weight used as it is
(src/minimax.rs:56-66).  The kernel also performs the residual sum that precedes
the norm, in float32, so the update of the stream and the norm read it once.
``weight_offset`` (default 0) is added to the stored weight when it is loaded: a file that keeps the weight less one
(stored around zero, used as 1 + w) gives 1.  The norm also serves behind a sublayer (``normed``, ``add_normed``), and
an update that comes with such a norm (``NormedUpdate``) is normed, added and normed again in one kernel."""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import VECTOR, TensorNeed, TensorSource
from .base import Norm, NormedUpdate, UpdateSum, WeightedPair, WeightedRows, as_tensor, register_part

# FIELDRUN_B200_FUSED_OUTPUT_NORM=0: an update with a norm of its own is normed and added by kernels of their own first
FUSED_OUTPUT_NORM = os.environ.get("FIELDRUN_B200_FUSED_OUTPUT_NORM", "1") != "0"


class RMSNorm(Norm):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.width = int(spec.args["width"])
        self.eps = float(spec.args["eps"])
        self.weight_offset = float(spec.args.get("weight_offset", 0.0))
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.width,), VECTOR, "around_zero" if self.weight_offset else "around_one")]

    def load(self, source: TensorSource) -> None:
        self.weight = source.fetch(self.tensor_needs()[0])
        if self.weight_offset:
            self.weight = (self.weight.to(torch.float32) + self.weight_offset).contiguous()      # float32, rounded once

    accepts_deferred = True

    def _parts_of(self, ctx, inner):
        """(a, b, ca, cb, experts) of an update that the fused kernel sums itself; anything else as one tensor."""
        if isinstance(inner, WeightedPair):
            return inner.a, inner.b, inner.wa, inner.wb, None
        if isinstance(inner, WeightedRows) and inner.top_k <= ops.NORM_MAX_SUMMED_ROWS:
            return None, None, 1.0, 1.0, (inner.rows, inner.weights, inner.row_map)
        if isinstance(inner, UpdateSum) and len(inner.tensors) <= 2 and all(w.top_k <= ops.NORM_MAX_SUMMED_ROWS for w in inner.weighted):
            tensors = list(inner.tensors) + [None, None]
            weighted = inner.weighted[0] if inner.weighted else None
            return tensors[0], tensors[1], 1.0, 1.0, (weighted.rows, weighted.weights, weighted.row_map) if weighted else None
        return as_tensor(ctx, inner), None, 1.0, 1.0, None

    def normed(self, ctx, update):
        out = ctx.buffer(f"norm.normed.{self.width}", tuple(update.shape), torch.float32)
        out.zero_()
        ops.add_rms_normed(out, update, self.weight, self.eps)
        return out

    def add_normed(self, ctx, update, x):
        ops.add_rms_normed(x, as_tensor(ctx, update), self.weight, self.eps)
        if self.dtype == torch.float32:
            return x
        act = ctx.buffer("stream.act", tuple(x.shape), self.dtype)
        act.copy_(x)
        return act

    def forward(self, ctx, x, *, delta=None, rows=None, want32=False, write_back=True):
        if (isinstance(delta, NormedUpdate) and FUSED_OUTPUT_NORM and isinstance(delta.norm, RMSNorm)
                and delta.norm.width == self.width and self.weight.dtype == torch.float32):
            # the update's own norm, the sum and this norm in one pass over the row
            a, b, ca, cb, experts = self._parts_of(ctx, delta.inner)
            count = rows.numel() if rows is not None else x.shape[0]
            out = ctx.buffer(f"norm.out.{self.width}", (count, self.width), self.dtype)
            out32 = None
            if want32:
                out32 = out if self.dtype == torch.float32 else ctx.buffer(f"norm.out32.{self.width}", (count, self.width),
                                                                           torch.float32)
            ops.sandwich_norm(x, delta.norm.weight, delta.norm.eps, a=a, b=b, ca=ca, cb=cb, experts=experts, rows=rows,
                              weight=self.weight, eps=self.eps, out=out, out32=None if out32 is out else out32,
                              write_back=write_back)
            return out, out32
        experts = None
        if isinstance(delta, WeightedRows) and delta.top_k <= ops.NORM_MAX_SUMMED_ROWS:
            experts, delta = (delta.rows, delta.weights, delta.row_map), None      # the kernel sums them as it reads x
        else:
            delta = as_tensor(ctx, delta)
        count = rows.numel() if rows is not None else x.shape[0]
        out = ctx.buffer(f"norm.out.{self.width}", (count, self.width), self.dtype)
        out32 = None
        if want32:
            out32 = out if self.dtype == torch.float32 else ctx.buffer(f"norm.out32.{self.width}", (count, self.width),
                                                                       torch.float32)
        ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows, out32=None if out32 is out else out32,
                    write_back=write_back and (delta is not None or experts is not None), experts=experts)
        return out, out32


class LayerNorm(Norm):
    """(v - mean) / sqrt(var + eps) * weight + bias per row, var the mean of the squared deviations, float32
    statistics; the bias is optional (``bias: False``).  It serves in both places of a norm: on the stream
    (``forward``: a model's last norm, or a pre-norm block) and on a sublayer's output (``add_normed``), where
    one kernel norms the update, adds it to the float32 stream and writes the stream's copy in the model dtype."""

    replayable = True
    STREAM_COPY = "stream.act"           # the workspace buffer that holds the stream in the model dtype

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.width = int(spec.args["width"])
        self.eps = float(spec.args["eps"])
        self.has_bias = bool(spec.args.get("bias", True))
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_needs(self):
        needs = [TensorNeed(self.name_of("weight"), (self.width,), VECTOR, "around_one")]
        if self.has_bias:
            needs.append(TensorNeed(self.name_of("bias"), (self.width,), VECTOR, "bias"))
        return needs

    def load(self, source: TensorSource) -> None:
        needs = self.tensor_needs()
        self.weight = source.fetch(needs[0])
        self.bias = source.fetch(needs[1]) if self.has_bias else None

    def forward(self, ctx, x, *, delta=None, rows=None, want32=False, write_back=True):
        delta = as_tensor(ctx, delta)
        if delta is not None:
            if write_back:
                ops.add_rows(x, delta)
            else:
                x = x + delta
        count = rows.numel() if rows is not None else x.shape[0]
        out = ctx.buffer(f"norm.out.{self.width}", (count, self.width), self.dtype)
        ops.layernorm(x, self.weight, self.bias, self.eps, rows=rows, act=out)
        out32 = None
        if want32:
            out32 = out
            if self.dtype != torch.float32:
                out32 = ctx.buffer(f"norm.out32.{self.width}", (count, self.width), torch.float32)
                ops.layernorm(x, self.weight, self.bias, self.eps, rows=rows, act=out32)
        return out, out32

    def add_normed(self, ctx, update, x):
        if self.dtype == torch.float32:
            ops.layernorm(update, self.weight, self.bias, self.eps, stream=x)
            return x
        act = ctx.buffer(self.STREAM_COPY, tuple(x.shape), self.dtype)
        ops.layernorm(update, self.weight, self.bias, self.eps, stream=x, act=act)
        return act


class DynamicTanh(Norm):
    """tanh(alpha v) * weight + bias with one learned scalar alpha: a norm without statistics.  Two of them that read
    the same stream (a block whose sublayers run side by side) go through one kernel (``forward_pair``), which also
    adds the updates that the block before left: float32 tensors and the experts' weighted rows."""

    replayable = True
    accepts_deferred = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.width = int(spec.args["width"])
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.alpha: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.width,), VECTOR, "around_one"),
                TensorNeed(self.name_of("bias"), (self.width,), VECTOR, "bias"),
                TensorNeed(self.name_of("alpha"), (), VECTOR, "around_half")]

    def load(self, source: TensorSource) -> None:
        self.weight, self.bias, alpha = (source.fetch(need) for need in self.tensor_needs())
        self.alpha = alpha.reshape(1)                    # stays on the device: the kernel reads it there

    def triple(self):
        return self.weight, self.bias, self.alpha

    @staticmethod
    def split(ctx, delta):
        """(float32 tensors, experts' rows or None) of whatever form the update came in."""
        if delta is None:
            return (), None
        if isinstance(delta, torch.Tensor):
            return (delta,), None
        if isinstance(delta, WeightedRows) and delta.top_k <= ops.NORM_MAX_SUMMED_ROWS:
            return (), (delta.rows, delta.weights, delta.row_map)
        if isinstance(delta, UpdateSum) and len(delta.tensors) <= 2 and all(
                w.top_k <= ops.NORM_MAX_SUMMED_ROWS for w in delta.weighted):
            weighted = delta.weighted[0] if delta.weighted else None
            return tuple(delta.tensors), (weighted.rows, weighted.weights, weighted.row_map) if weighted else None
        return (as_tensor(ctx, delta),), None

    def forward(self, ctx, x, *, delta=None, rows=None, want32=False, write_back=True):
        deltas, experts = self.split(ctx, delta)
        count = rows.numel() if rows is not None else x.shape[0]
        out = ctx.buffer(f"norm.out.{self.width}", (count, self.width), self.dtype)
        ops.dyt_norm(x, self.triple(), out, deltas=deltas, experts=experts, rows=rows,
                     write_back=write_back and rows is None and (bool(deltas) or experts is not None))
        out32 = None
        if want32:
            out32 = out
            if self.dtype != torch.float32:
                out32 = ctx.buffer(f"norm.out32.{self.width}", (count, self.width), torch.float32)
                ops.dyt_norm(x, self.triple(), out32, rows=rows)       # x holds the sum by now (or nothing was added)
        return out, out32

    def forward_pair(self, ctx, x, other: "DynamicTanh", *, delta=None, want32=False):
        """This norm and ``other`` of the same x + delta (the sum stored back): (out, other's out, other's out in
        float32 or None)."""
        deltas, experts = self.split(ctx, delta)
        rows = x.shape[0]
        out1 = ctx.buffer(f"norm.out.{self.width}", (rows, self.width), self.dtype)
        out2 = ctx.buffer(f"norm.out2.{self.width}", (rows, self.width), self.dtype)
        out2_32 = None
        if want32 and self.dtype != torch.float32:
            out2_32 = ctx.buffer(f"norm.out32.{self.width}", (rows, self.width), torch.float32)
        ops.dyt_norm(x, self.triple(), out1, second=other.triple(), out2=out2, out2_32=out2_32, deltas=deltas, experts=experts,
                     write_back=bool(deltas) or experts is not None)
        return out1, out2, (out2 if self.dtype == torch.float32 else out2_32) if want32 else None


register_part("norm", "dynamic_tanh", DynamicTanh, replace=True)
register_part("norm", "rmsnorm", RMSNorm, replace=True)
register_part("norm", "layernorm", LayerNorm, replace=True)
