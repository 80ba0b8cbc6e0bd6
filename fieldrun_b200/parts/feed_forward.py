"""Feed-forward parts: experts chosen by a router, and a dense gated unit.

Routed experts (src/minimax.rs:88-126): router logits z = act W_r^T in float32;
score s = sigmoid(z) (or, with ``score: softmax``, the softmax of z over all experts; ``weight_floor`` then adds
1e-20 to the sum of the picked scores); choice c = s + bias (the bias decides only who is picked);
the ``top_k`` largest c, ties to the lower id; weights s / sum of the picked s;
each picked expert computes silu(x W1^T) * (x W3^T) then W2; the outputs are
summed with their weights in rank order.  The experts' matrices are stacked:
``w13`` [E, 2I, d] holds each expert's gate rows then its up rows, ``w2`` [E, d, I].
Rows are grouped by expert with a counting sort on the device, so no step of the
feed-forward waits for the host.

Two more forms, each an argument: ``gate_limit`` > 0 makes an expert's unit the clamped gate g = min(x W1^T, limit),
u = clamp(x W3^T, -limit, limit), g sigmoid(1.702 g) (u + 1); ``weight_on_input`` puts an expert's weight on what goes
in instead of on what comes out: the token's output is the sum of expert(w x) over its experts.  The rows are then
scaled and sorted by a kernel of their own (product in float32, rounded once) and summed with weights of one.

``groups`` ``{"count", "keep"}``: the experts form ``count`` equal groups of neighbours; a group's value is its largest
choice value, and only experts of the ``keep`` groups with the largest values can be picked.  ``shared_expert``
``{"width", "gate"}``: one more expert of the same form that every token uses; its output is added to the routed
experts' sum, with ``gate`` multiplied by sigmoid(w_sg . x), one number per token.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorNeed, TensorSource
from .base import FeedForward, UpdateSum, WeightedRows, register_part
from .linear import linear

TILE_ROWS = 32        # rows of one expert that a block of the expert kernels takes
# Above this many rows per expert (on average) a step's expert products run on tcgen05: tiles of 32 rows and more
# read an expert's weights once however its rows are spread, at the speed of the memory.  Measured on a B200 at
# MiniMax-M2's sizes: the streaming kernel with tiles of 8 rows is as fast while no expert gets more than 8 rows
# (a decode step of 64 sequences, two rows per expert on average: 1,087 against 1,094 us a layer), but a prompt's
# tokens crowd on fewer experts, and every tile beyond an expert's first reads its weights again (a prompt of 64
# tokens: 525 against 419 us a layer, of 256: 1,400 against 617).
TENSOR_CORE_ROWS_PER_EXPERT = {"decode": 4.0, "prompt": 1.0}


class RoutedExperts(FeedForward):
    kernel_groups = ("common", "streams", "experts", "products")

    wants_float32_input = True          # the router reads the normed rows before they are rounded
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size = int(a["hidden_size"])
        self.num_experts = int(a["num_experts"])
        self.top_k = int(a["top_k"])
        self.expert_width = int(a["expert_width"])
        self.score = a.get("score", "sigmoid")
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"router score {self.score!r} is neither 'sigmoid' nor 'softmax'")
        self.choice_bias = bool(a.get("choice_bias", False))
        floor = float(a.get("weight_floor") or 0.0)
        if floor not in (0.0, ops.ROUTE_WEIGHT_FLOOR):
            raise ValueError(f"a floor of {floor} under the sum of the picked scores: the kernels have 0 and {ops.ROUTE_WEIGHT_FLOOR}")
        # what the kernels take as their ``renormalize``: bit 0 divides by the sum of the picked scores, bit 1 makes the
        # scores a softmax over all experts (else sigmoids), bit 2 adds the floor to that sum
        groups = a.get("groups") or {}
        self.group_count, self.group_keep = int(groups.get("count", 1)), int(groups.get("keep", groups.get("count", 1)))
        if self.group_count < 1 or not 1 <= self.group_keep <= self.group_count or int(a["num_experts"]) % self.group_count:
            raise ValueError(f"{a['num_experts']} experts in {self.group_count} groups of which {self.group_keep} stay")
        if self.group_keep * (int(a["num_experts"]) // self.group_count) < int(a["top_k"]):
            raise ValueError(f"{self.group_keep} groups of {int(a['num_experts']) // self.group_count} experts hold fewer than the "
                             f"{a['top_k']} experts a token picks")
        # bits 8 and up: the groups (``ops.route_groups``)
        self.renormalize = (int(bool(a.get("renormalize", True))) | (ops.ROUTE_SOFTMAX if self.score == "softmax" else 0)
                            | (ops.ROUTE_FLOOR if floor else 0) | ops.route_groups(self.group_count, self.group_keep))
        shared = a.get("shared_expert")
        self.shared_width = int(shared["width"]) if shared else 0
        self.shared_gate = bool(shared.get("gate", False)) if shared else False
        if shared and self.shared_width < 1:
            raise ValueError(f"a shared expert of width {self.shared_width}")
        self.w_shared_in: Optional[torch.Tensor] = None       # gate rows, up rows, the token gate's row, zero rows up to a multiple of 16
        self.w_shared_down: Optional[torch.Tensor] = None
        self.routed_scale = float(a.get("routed_scale", 1.0))
        self.gate_limit = float(a.get("gate_limit") or 0.0)
        if self.gate_limit < 0.0:
            raise ValueError(f"a gate limit of {self.gate_limit}")
        self.weight_on_input = bool(a.get("weight_on_input", False))
        self._ones: Optional[torch.Tensor] = None
        if not 1 <= self.top_k <= self.num_experts:
            raise ValueError(f"top_k {self.top_k} is outside 1..{self.num_experts} experts")
        if not (dtype == torch.bfloat16 and self.hidden_size % 128 == 0 and self.expert_width % 128 == 0):
            self.kernel_groups = ("common", "streams", "experts")      # sizes the tcgen05 products never take
        self.router: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.w13: Optional[torch.Tensor] = None
        self.w2: Optional[torch.Tensor] = None
        self.on_route = None              # called with the picked ids [T, k] of every step (for measurements)
        # int32 [rows >= T, k] on the device, or None: when set, every step copies its picked ids into the first
        # T rows.  The copy is a device operation, so unlike ``on_route`` it also happens in a recorded step.
        self.route_log: Optional[torch.Tensor] = None

    def _expert_needs(self, e: int) -> tuple[TensorNeed, TensorNeed, TensorNeed]:
        d, i = self.hidden_size, self.expert_width
        return (TensorNeed(self.name_of("w_gate").format(e=e), (i, d), MATRIX, "normal"),
                TensorNeed(self.name_of("w_up").format(e=e), (i, d), MATRIX, "normal"),
                TensorNeed(self.name_of("w_down").format(e=e), (d, i), MATRIX, "normal"))

    def _shared_needs(self) -> list[TensorNeed]:
        if not self.shared_width:
            return []
        d, i = self.hidden_size, self.shared_width
        needs = [TensorNeed(self.name_of("shared_gate"), (i, d), MATRIX, "normal"),
                 TensorNeed(self.name_of("shared_up"), (i, d), MATRIX, "normal"),
                 TensorNeed(self.name_of("shared_down"), (d, i), MATRIX, "normal")]
        if self.shared_gate:
            needs.append(TensorNeed(self.name_of("shared_token_gate"), (1, d), MATRIX, "normal"))
        return needs

    def tensor_needs(self):
        needs = [TensorNeed(self.name_of("router"), (self.num_experts, self.hidden_size), VECTOR, "normal")]
        if self.choice_bias:
            needs.append(TensorNeed(self.name_of("choice_bias"), (self.num_experts,), VECTOR, "bias"))
        for e in range(self.num_experts):
            needs.extend(self._expert_needs(e))
        return needs + self._shared_needs()

    def load(self, source: TensorSource) -> None:
        d, i, n = self.hidden_size, self.expert_width, self.num_experts
        self.router = source.fetch(TensorNeed(self.name_of("router"), (n, d), VECTOR, "normal"))
        if self.choice_bias:
            self.bias = source.fetch(TensorNeed(self.name_of("choice_bias"), (n,), VECTOR, "bias"))
        for e in range(n):
            gate, up, down = (source.fetch(need) for need in self._expert_needs(e))
            if self.w13 is None:
                self.w13 = torch.empty((n, 2 * i, d), dtype=gate.dtype, device=gate.device)
                self.w2 = torch.empty((n, d, i), dtype=gate.dtype, device=gate.device)
            self.w13[e, :i].copy_(gate)
            self.w13[e, i:].copy_(up)
            self.w2[e].copy_(down)
        if self.shared_width:
            fetched = [source.fetch(need) for need in self._shared_needs()]
            width = self.shared_width
            rows = -(-(2 * width + 1) // 16) * 16           # a product's features in steps of 16 (the streaming kernels' rule)
            self.w_shared_in = torch.zeros((rows, d), dtype=fetched[0].dtype, device=fetched[0].device)
            self.w_shared_in[:width].copy_(fetched[0])
            self.w_shared_in[width:2 * width].copy_(fetched[1])
            if self.shared_gate:
                self.w_shared_in[2 * width].copy_(fetched[3].reshape(-1))
            self.w_shared_down = fetched[2]

    def shared(self, ctx, act: torch.Tensor) -> torch.Tensor:
        """The shared expert's output [T, d] float32: silu(gate) * up, times the token's sigmoid gate where the part has one
        (put on the hidden rows: the product behind it is linear), then the product out."""
        both = linear(act, self.w_shared_in)
        hidden = ctx.buffer("experts.shared_hidden", (act.shape[0], self.shared_width), self.dtype)
        ops.gated_unit(both, hidden, "silu", row_gate=2 * self.shared_width if self.shared_gate else None)
        return linear(hidden, self.w_shared_down)

    # -- one step --------------------------------------------------------------------------------------
    def logits(self, ctx, act32: torch.Tensor) -> torch.Tensor:
        """Router logits: float32 rows, float32 weight, no rounding.  Few rows: this library's kernel (the
        library's float32 product is slow on a handful of rows); many: the library."""
        tokens = act32.shape[0]
        if tokens <= ops.ROUTER_LOGITS_TOKENS and self.hidden_size % 4 == 0:
            out = ctx.buffer("experts.logits", (tokens, self.num_experts), torch.float32)
            ops.router_logits(act32, self.router, out)
            return out
        return linear(act32, self.router)

    def route(self, ctx, act32: torch.Tensor):
        tokens = act32.shape[0]
        logits = self.logits(ctx, act32)
        ids = ctx.buffer("experts.ids", (tokens, self.top_k), torch.int32)
        weights = ctx.buffer("experts.weights", (tokens, self.top_k), torch.float32)
        ops.router_topk(logits, self.bias, self.top_k, self.renormalize, self.routed_scale, ids, weights)
        return ids, weights

    def streams(self) -> bool:
        """Whether the tensor-core streaming kernel takes this part's sizes (bfloat16, sizes in steps of 32)."""
        return (self.dtype == torch.bfloat16 and self.hidden_size % 32 == 0 and self.expert_width % 32 == 0)

    def on_tensor_cores(self, assignments: int, decode: bool = False) -> bool:
        """Whether the tcgen05 kernel runs the step: bfloat16, sizes in steps of 128, and enough rows per
        expert that the products, not the weights alone, are the work."""
        return (self.dtype == torch.bfloat16 and self.hidden_size % 128 == 0 and self.expert_width % 128 == 0
                and assignments > TENSOR_CORE_ROWS_PER_EXPERT["decode" if decode else "prompt"] * self.num_experts)

    def tile_rows(self, assignments: int, decode: bool = False) -> int:
        """Rows of one expert that one block takes: few when experts get few rows each, so that no block
        carries accumulators it does not need; enough that most experts fit one tile when they get many."""
        per_expert = assignments / self.num_experts
        if self.on_tensor_cores(assignments, decode):
            return next((t for t in (32, 64, 128, 256) if t >= 1.3 * per_expert), 256)
        if not self.streams():
            return TILE_ROWS
        return 8 if per_expert <= 4 else 16 if per_expert <= 12 else 32

    def plan(self, ctx, ids: torch.Tensor):
        tokens = ids.shape[0]
        n = tokens * self.top_k
        chunks = (n + 1023) // 1024
        tile_rows = self.tile_rows(n, ctx.is_decode)
        max_tiles = (n + tile_rows - 1) // tile_rows + min(self.num_experts, n)
        p = {
            "counts": ctx.buffer("experts.counts", (chunks * self.num_experts,), torch.int32),
            "offsets": ctx.buffer("experts.offsets", (self.num_experts + 1,), torch.int32),
            "sorted_token": ctx.buffer("experts.sorted_token", (n,), torch.int32),
            "row_of_assign": ctx.buffer("experts.row_of_assign", (n,), torch.int32),
            "tile_expert": ctx.buffer("experts.tile_expert", (max_tiles,), torch.int32),
            "tile_row0": ctx.buffer("experts.tile_row0", (max_tiles,), torch.int32),
            "num_tiles": ctx.buffer("experts.num_tiles", (1,), torch.int32),
            "max_tiles": max_tiles,
            "rows": n,
            "tile_rows": tile_rows,
        }
        ops.expert_plan(ids, self.num_experts, tile_rows, p["counts"], p["offsets"], p["sorted_token"],
                        p["row_of_assign"], p["tile_expert"], p["tile_row0"], p["num_tiles"])
        return p

    def experts(self, ctx, act: torch.Tensor, p, scaled: Optional[torch.Tensor] = None) -> torch.Tensor:
        """y [N, d] float32: the output of its expert for every (token, rank), in expert-sorted order.  ``scaled``: the
        experts' input rows already in that order (each token's row times its expert's weight) instead of ``act``."""
        hidden = ctx.buffer("experts.hidden", (p["rows"], self.expert_width), self.dtype)
        y = ctx.buffer("experts.y", (p["rows"], self.hidden_size), torch.float32)
        limit = self.gate_limit
        sorted_token = p["sorted_token"]
        if scaled is not None:
            act, sorted_token = scaled, None
        if self.on_tensor_cores(p["rows"], ctx.is_decode):
            gathered = scaled
            if gathered is None:
                gathered = ctx.buffer("experts.gathered", (p["rows"], self.hidden_size), self.dtype)
                ops.gather_rows(act, p["sorted_token"], gathered)
            ops.expert_gemm_tc(self.w13, gathered, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                               p["max_tiles"], p["tile_rows"], hidden, paired=True, gate_limit=limit)
            ops.expert_gemm_tc(self.w2, hidden, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                               p["max_tiles"], p["tile_rows"], y, paired=False)
            return y
        if self.streams() and ops.weight_stream_takes(self.expert_width, self.hidden_size, paired=True) \
                and ops.weight_stream_takes(self.hidden_size, self.expert_width, paired=False):
            ops.weight_stream(self.w13, act, sorted_token, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                              p["max_tiles"], p["tile_rows"], hidden, paired=True, gate_limit=limit)
            # the second product's lists are the first one's: its weights may be on their way while the first still runs
            ops.weight_stream(self.w2, hidden, None, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                              p["max_tiles"], p["tile_rows"], y, paired=False, lists_final=True)
            return y
        if self.streams():
            tiles = min(p["rows"], self.num_experts)           # about as many tiles as experts that got rows
            ops.expert_gemm_mma(self.w13, act, sorted_token, p["tile_expert"], p["tile_row0"], p["num_tiles"],
                                p["offsets"], p["max_tiles"], p["tile_rows"], hidden, paired=True, gate_limit=limit,
                                **ops.stream_shape(tiles, self.expert_width, self.hidden_size, p["tile_rows"], paired=True))
            ops.expert_gemm_mma(self.w2, hidden, None, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                                p["max_tiles"], p["tile_rows"], y, paired=False,
                                **ops.stream_shape(tiles, self.hidden_size, self.expert_width, p["tile_rows"]))
            return y
        ops.expert_gemm_generic(self.w13, act, sorted_token, p["tile_expert"], p["tile_row0"], p["num_tiles"],
                                p["offsets"], p["max_tiles"], hidden, paired=True, gate_limit=limit)
        ops.expert_gemm_generic(self.w2, hidden, None, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                                p["max_tiles"], y, paired=False)
        return y

    def route_and_plan(self, ctx, act32: torch.Tensor):
        """For steps of few tokens: choice and lists in one launch."""
        tokens = act32.shape[0]
        n = tokens * self.top_k
        tile_rows = self.tile_rows(n, ctx.is_decode)
        max_tiles = (n + tile_rows - 1) // tile_rows + min(self.num_experts, n)
        ids = ctx.buffer("experts.ids", (tokens, self.top_k), torch.int32)
        weights = ctx.buffer("experts.weights", (tokens, self.top_k), torch.float32)
        p = {
            "offsets": ctx.buffer("experts.offsets", (self.num_experts + 1,), torch.int32),
            "sorted_token": ctx.buffer("experts.sorted_token", (n,), torch.int32),
            "row_of_assign": ctx.buffer("experts.row_of_assign", (n,), torch.int32),
            "tile_expert": ctx.buffer("experts.tile_expert", (max_tiles,), torch.int32),
            "tile_row0": ctx.buffer("experts.tile_row0", (max_tiles,), torch.int32),
            "num_tiles": ctx.buffer("experts.num_tiles", (1,), torch.int32),
            "max_tiles": max_tiles, "rows": n, "tile_rows": tile_rows,
        }
        if self.hidden_size % 4 == 0 and tokens <= ops.ROUTER_SMALL_TOKENS:
            logits = ctx.buffer("experts.logits", (tokens, self.num_experts), torch.float32)
            ops.router_small(act32, self.router, logits, self.bias, self.top_k, self.renormalize, self.routed_scale, tile_rows,
                             ids, weights, p["offsets"], p["sorted_token"], p["row_of_assign"], p["tile_expert"],
                             p["tile_row0"], p["num_tiles"])
        else:
            logits = self.logits(ctx, act32)
            ops.route_plan_small(logits, self.bias, self.top_k, self.renormalize, self.routed_scale, tile_rows, ids, weights,
                                 p["offsets"], p["sorted_token"], p["row_of_assign"], p["tile_expert"], p["tile_row0"],
                                 p["num_tiles"])
        return ids, weights, p

    def _tell_route(self, ids: torch.Tensor) -> None:
        if self.on_route is not None:
            self.on_route(ids)
        if self.route_log is not None:
            self.route_log[:ids.shape[0]].copy_(ids)

    def forward(self, ctx, act, act32):
        return self.forward_deferred(ctx, act, act32).materialize(ctx)

    def forward_deferred(self, ctx, act, act32):
        if act32 is None:
            raise ValueError("routed experts need the normed rows in float32 for the router")
        if (act.shape[0] <= ops.SMALL_ROUTE_TOKENS and act.shape[0] * self.top_k <= ops.SMALL_ROUTE_ASSIGNMENTS
                and self.num_experts <= 1024):
            ids, weights, p = self.route_and_plan(ctx, act32)
            self._tell_route(ids)
        else:
            ids, weights = self.route(ctx, act32)
            self._tell_route(ids)
            p = self.plan(ctx, ids)
        if self.weight_on_input:
            # the weight belongs on what goes in: a row per (token, rank), scaled (float32 row times weight, rounded once)
            scaled = ctx.buffer("experts.scaled", (p["rows"], self.hidden_size), self.dtype)
            ops.scaled_rows(act32, weights, p["row_of_assign"], scaled)
            y = self.experts(ctx, act, p, scaled)
            if self._ones is None or self._ones.shape[0] < weights.shape[0] or self._ones.device != weights.device:
                self._ones = torch.ones((max(weights.shape[0], 1024), self.top_k), dtype=torch.float32, device=weights.device)
            routed = WeightedRows(y, self._ones[:weights.shape[0]], p["row_of_assign"])
            return UpdateSum([self.shared(ctx, act), routed]) if self.shared_width else routed
        y = self.experts(ctx, act, p)
        # each token's expert outputs, not yet summed: the norm after this layer adds them in rank order
        routed = WeightedRows(y, weights, p["row_of_assign"])
        if self.shared_width:
            return UpdateSum([self.shared(ctx, act), routed])
        return routed


class DenseGatedUnit(FeedForward):
    """act(x W_gate^T) * (x W_up^T), then W_down: one expert's formula for every row (src/minimax.rs:116-120), with
    ``activation`` silu (the default) or gelu_tanh."""

    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden_size = int(spec.args["hidden_size"])
        self.width = int(spec.args["width"])
        self.activation = str(spec.args.get("activation", "silu"))
        if self.activation not in ops.GATED_ACTIVATIONS:
            raise ValueError(f"a gated unit with activation {self.activation!r}: known are {sorted(ops.GATED_ACTIVATIONS)}")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def _needs(self):
        d, i = self.hidden_size, self.width
        return (TensorNeed(self.name_of("w_gate"), (i, d), MATRIX, "normal"),
                TensorNeed(self.name_of("w_up"), (i, d), MATRIX, "normal"),
                TensorNeed(self.name_of("w_down"), (d, i), MATRIX, "normal"))

    def tensor_needs(self):
        return list(self._needs())

    def load(self, source: TensorSource) -> None:
        gate, up, down = (source.fetch(n) for n in self._needs())
        self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = down

    def forward(self, ctx, act, act32):
        both = linear(act, self.w_gate_up)                         # float32 [T, 2I]
        hidden = ctx.buffer("dense.hidden", (act.shape[0], self.width), self.dtype)
        ops.gated_unit(both, hidden, self.activation)
        return linear(hidden, self.w_down)


FUSED_ACTIVATION_ROWS = 64      # from this many rows of a prompt step on, a dense unit's first product carries its activation


class DenseUnit(FeedForward):
    """W_down act(W_up x): one product in, an activation, one product out.  ``activation`` is one of
    ``ops.ACTIVATIONS`` (``relu_squared``: relu(z)^2, ``gelu_tanh``, ``silu``, ``relu``).  A prompt's rows in bfloat16
    take the first product on tcgen05 with the activation in its epilogue (the step as one expert's rows); few rows,
    float32 and sizes that kernel does not take go through the plain product and the activation kernel."""

    replayable = True
    kernel_groups = ("common", "streams", "products")

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden_size = int(spec.args["hidden_size"])
        self.width = int(spec.args["width"])
        self.activation = str(spec.args["activation"])
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is none of {sorted(ops.ACTIVATIONS)}")
        if not (dtype == torch.bfloat16 and self.width % 128 == 0 and self.hidden_size % 64 == 0):
            self.kernel_groups = ("common", "streams")         # sizes the tcgen05 product never takes
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self._tiles: dict = {}

    def _needs(self):
        d, i = self.hidden_size, self.width
        return (TensorNeed(self.name_of("w_up"), (i, d), MATRIX, "normal"),
                TensorNeed(self.name_of("w_down"), (d, i), MATRIX, "normal"))

    def tensor_needs(self):
        return list(self._needs())

    def load(self, source: TensorSource) -> None:
        self.w_up, self.w_down = (source.fetch(n) for n in self._needs())

    def fused_tiles(self, ctx, rows: int):
        """The lists that make the step one expert's rows in tiles, for the tcgen05 product; they depend on the number
        of rows alone and are kept."""
        tile_rows = 256 if rows >= 256 else 128 if rows > 64 else 64 if rows > 32 else 32
        key = (str(ctx.device), rows)
        made = self._tiles.get(key)
        if made is None:
            if len(self._tiles) > 64:
                self._tiles.clear()
            count = (rows + tile_rows - 1) // tile_rows
            flat = torch.tensor([0] * count + [tile_rows * i for i in range(count)] + [count, 0, rows], dtype=torch.int32).to(ctx.device)
            made = self._tiles[key] = (flat[:count], flat[count:2 * count], flat[2 * count:2 * count + 1], flat[2 * count + 1:], count,
                                       tile_rows)
        return made

    def forward(self, ctx, act, act32):
        rows = act.shape[0]
        hidden = ctx.buffer("dense.hidden", (rows, self.width), self.dtype)
        if (self.dtype == torch.bfloat16 and rows >= FUSED_ACTIVATION_ROWS and not ctx.is_decode and self.width % 128 == 0
                and self.hidden_size % 64 == 0):
            # a prompt's rows: product and activation in one kernel on tcgen05, the result rounded once to bfloat16
            tile_expert, tile_row0, num_tiles, offsets, count, tile_rows = self.fused_tiles(ctx, rows)
            ops.expert_gemm_tc(self.w_up.view(1, self.width, self.hidden_size), act, tile_expert, tile_row0, num_tiles, offsets,
                               count, tile_rows, hidden, paired=False, activation=self.activation)
        else:
            up = linear(act, self.w_up)                            # float32 [T, I]
            ops.unary_unit(up, hidden, self.activation)
        return linear(hidden, self.w_down)


register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
register_part("feed_forward", "dense_unit", DenseUnit, replace=True)
register_part("feed_forward", "dense_gated", DenseGatedUnit, replace=True)
