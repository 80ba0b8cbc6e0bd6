"""Two mixers side by side on the same input.  ``blend: rms`` (the default): out = share * (left / rms(left) * w_left +
right / rms(right) * w_right), each output divided by its root mean square over the model width (eps inside the root)
and multiplied by a plain weight vector.  ``blend: weighted``: out = left_weight * left + right_weight * right with two
constants and no tensors of its own; the two outputs are then left unsummed (``WeightedPair``) for the norm that takes
the update.  The two are parts of any registered kinds, given as ``PartSpec`` in the arguments ``left`` and
``right``; they share the run's cache line, so at most one of them may keep keys and values and at most one a state."""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed, LineView
from ..csrc import ops
from ..weights.loader import VECTOR, TensorNeed, TensorSource
from .base import Mixer, WeightedPair, as_tensor, build_part, register_part


class MixerPair(Mixer):
    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size = int(a["hidden_size"])
        self.blend = a.get("blend", "rms")
        if self.blend not in ("rms", "weighted"):
            raise ValueError(f"a pair of mixers blended by {self.blend!r}: known are 'rms' and 'weighted'")
        self.eps = float(a.get("norm_eps", 1e-6))
        self.share = float(a.get("share", 0.5))
        self.left_weight, self.right_weight = float(a.get("left_weight", 1.0)), float(a.get("right_weight", 1.0))
        self.left: Mixer = build_part("mixer", a["left"], dtype)
        self.right: Mixer = build_part("mixer", a["right"], dtype)
        self.left_norm: Optional[torch.Tensor] = None
        self.right_norm: Optional[torch.Tensor] = None
        self.cache_need()                                  # refuses a pair that cannot share a line, now

    @property
    def replayable(self) -> bool:
        return True                                        # its own kernel reads no host tables; the two count for themselves

    def children(self):
        return [self.left, self.right]

    def tensor_needs(self):
        if self.blend == "weighted":
            return []
        return [TensorNeed(self.name_of("left_norm"), (self.hidden_size,), VECTOR, "around_one"),
                TensorNeed(self.name_of("right_norm"), (self.hidden_size,), VECTOR, "around_one")]

    def load(self, source: TensorSource) -> None:
        if self.blend == "rms":
            self.left_norm, self.right_norm = (source.fetch(need) for need in self.tensor_needs())
        self.left.load(source)
        self.right.load(source)

    def cache_need(self) -> CacheNeed:
        a, b = self.left.cache_need(), self.right.cache_need()
        if a.kv_heads and b.kv_heads:
            raise ValueError("a pair of mixers shares one cache line: only one of the two may keep keys and values")
        if a.state_shape and b.state_shape:
            raise ValueError("a pair of mixers shares one cache line: only one of the two may keep a state")
        kv, st = (a if a.kv_heads else b), (a if a.state_shape else b)
        return CacheNeed(kv_heads=kv.kv_heads, head_dim=kv.head_dim, window=kv.window, value_dim=kv.value_dim, chunk=kv.chunk,
                         state_shape=st.state_shape, state_dtype=st.state_dtype)

    def prepare(self, num_positions: int, device) -> None:
        self.left.prepare(num_positions, device)
        self.right.prepare(num_positions, device)

    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        a = as_tensor(ctx, self.left.forward(ctx, act, line, writes_cache))
        b = as_tensor(ctx, self.right.forward(ctx, act, line, writes_cache))
        if self.blend == "weighted":
            return WeightedPair(a, b, self.left_weight, self.right_weight)
        out = ctx.buffer("mixer_pair.out", (act.shape[0], self.hidden_size), torch.float32)
        ops.rms_blend(a, b, self.left_norm, self.right_norm, out, self.eps, self.share)
        return out


register_part("mixer", "mixer_pair", MixerPair, replace=True)
